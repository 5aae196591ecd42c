// Kernels that join the outputs of sublayers which read the same input:
//
//   sigmoid gate:   out[t][c] *= sigmoid(gate[t][c])                    (an output gate ahead of a projection)
//   normed mean:    out[t] = scale * sum_k rms(in_k[t]) * gain_k  (+ add[t])      as float32
//
//   head mix:       out[t][h][c] = sum_g mix[h][g] * in[t][g][kv(h)][c]                  (attention weights mixed over heads)
//
// where rms(v) = v / sqrt(mean(v^2) + eps).  Every input may be the activation dtype, float32, or the
// float32 partial sums of a split-k product (added up in order while they are read); sums, roots and the
// result are float32.
#include "common.cuh"
#include "operand.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace lily {

constexpr int MEAN_MAX = 4;

struct NormedMeanArgs {
    Operand in[MEAN_MAX];
    const float* gain[MEAN_MAX];
    int count;
    Operand add;
    float* out;
    int width;
    float eps, scale;
};

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const Operand gate, size_t total) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
        out[i] = from_float<T>(to_float(out[i]) / (1.f + expf(-gate(i))));
}

// bfloat16 in place with a bfloat16 gate in one piece, eight entries a thread and turn (16-byte accesses)
__global__ void sigmoid_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate, size_t total) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x * 8;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += step) {
        uint4 ov = *reinterpret_cast<const uint4*>(out + i);
        const uint4 gv = *reinterpret_cast<const uint4*>(gate + i);
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 o = __bfloat1622float2(o2[k]), g = __bfloat1622float2(g2[k]);
            o2[k] = __floats2bfloat162_rn(__fdividef(o.x, 1.f + __expf(-g.x)), __fdividef(o.y, 1.f + __expf(-g.y)));
        }
        *reinterpret_cast<uint4*>(out + i) = ov;
    }
}

// The heads' attention weights mixed by a matrix, applied behind the weighted sums: `in` holds, for every query head g,
// its weights' sums over the values of every kv head; head h takes the sums over its own kv head's values from all query
// heads.  Two layouts of `in`: rows [tokens][nq][nkv][dv] (float32, the CUDA-core attention kernel's), or planes
// [nkv][tokens][nq][dv] where plane s holds, for a head of kv head g, the sums over kv head (g + s) % nkv (one launch of
// the mma.sync attention kernel a plane).  The matrix [nq][nq] in shared memory.
// VEC neighbouring columns of one head a thread (8 from bfloat16 planes, 4 from float32, 16 bytes a load; 1 when the
// value size does not divide); grid (tokens, blocks of columns).
template <typename IN, int VEC>
__device__ __forceinline__ void load_columns(const IN* __restrict__ src, float (&v)[VEC]) {
    if constexpr (VEC == 8 && sizeof(IN) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(p[k]);
            v[2 * k] = f.x;
            v[2 * k + 1] = f.y;
        }
    } else if constexpr (VEC == 4 && sizeof(IN) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(src);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = to_float(src[k]);
    }
}

template <typename T, typename IN, int VEC>
__global__ void head_mix_kernel(const IN* __restrict__ in, int planes, size_t plane_stride, const float* __restrict__ mix,
                                T* __restrict__ out, int nq, int nkv, int dv) {
    extern __shared__ float mix_s[];
    pdl_enter_small();
    for (int i = threadIdx.x; i < nq * nq; i += blockDim.x) mix_s[i] = mix[i];
    __syncthreads();
    const int e = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;      // this thread's first column among the token's nq * dv
    if (e >= nq * dv) return;
    const int group = nq / nkv, h = e / dv, c = e % dv, own = h / group;
    const size_t tok = blockIdx.x;
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
    for (int gk = 0; gk < nkv; ++gk) {
        // the heads of kv head gk looked at kv head `own` in plane (own - gk) mod nkv
        const IN* src = planes ? in + (size_t)((own - gk + nkv) % nkv) * plane_stride + (tok * nq + (size_t)gk * group) * dv + c
                               : in + ((tok * nq + (size_t)gk * group) * nkv + own) * dv + c;
        const size_t step = planes ? (size_t)dv : (size_t)nkv * dv;
        const float* w = mix_s + h * nq + gk * group;
#pragma unroll 4
        for (int gi = 0; gi < group; ++gi) {
            float v[VEC];
            load_columns<IN, VEC>(src + gi * step, v);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] = fmaf(w[gi], v[k], acc[k]);
        }
    }
    T* dst = out + tok * nq * dv + e;
#pragma unroll
    for (int k = 0; k < VEC; ++k) dst[k] = from_float<T>(acc[k]);
}

// One block a token.  VEC 4: four columns a thread and turn (the width a multiple of four, everything 16-byte aligned).
template <int VEC>
__global__ void normed_mean_kernel(const NormedMeanArgs a) {
    __shared__ float red[33];
    pdl_enter_small();
    const size_t base = (size_t)blockIdx.x * a.width;
    float inv[MEAN_MAX];
#pragma unroll
    for (int k = 0; k < MEAN_MAX; ++k) {
        inv[k] = 0.f;
        if (k < a.count) {
            float ssq = 0.f;
            for (int i = threadIdx.x * VEC; i < a.width; i += blockDim.x * VEC) {
                if (VEC == 4) {
                    const float4 v = a.in[k].four(base + i);
                    ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                } else {
                    const float v = a.in[k](base + i);
                    ssq = fmaf(v, v, ssq);
                }
            }
            inv[k] = rsqrtf(block_sum(ssq, red) / (float)a.width + a.eps);
        }
    }
    for (int i = threadIdx.x * VEC; i < a.width; i += blockDim.x * VEC) {
        if (VEC == 4) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < MEAN_MAX; ++k) {
                if (k < a.count) {
                    const float4 v = a.in[k].four(base + i);
                    const float4 g = *reinterpret_cast<const float4*>(a.gain[k] + i);
                    o.x += (v.x * inv[k]) * g.x; o.y += (v.y * inv[k]) * g.y;
                    o.z += (v.z * inv[k]) * g.z; o.w += (v.w * inv[k]) * g.w;
                }
            }
            o.x *= a.scale; o.y *= a.scale; o.z *= a.scale; o.w *= a.scale;
            if (a.add.p) {
                const float4 f = a.add.four(base + i);
                o.x += f.x; o.y += f.y; o.z += f.z; o.w += f.w;
            }
            *reinterpret_cast<float4*>(a.out + base + i) = o;
        } else {
            float o = 0.f;
#pragma unroll
            for (int k = 0; k < MEAN_MAX; ++k)
                if (k < a.count) o += (a.in[k](base + i) * inv[k]) * a.gain[k][i];
            o *= a.scale;
            if (a.add.p) o += a.add(base + i);
            a.out[base + i] = o;
        }
    }
}

// The same for a few tokens (decode): a thread-block cluster of CL blocks shares one token, each block takes
// width / CL columns (four a thread) and the blocks exchange their sums of squares through distributed shared
// memory, so that 8 tokens keep 64 SMs busy instead of 8.  grid (CL, tokens), cluster (CL, 1, 1);
// width % (4 * CL) == 0; block = width / (4 * CL) threads.
template <int CL>
__global__ void normed_mean_cluster_kernel(const NormedMeanArgs a) {
    __shared__ float red[MEAN_MAX][33];
    __shared__ float share[MEAN_MAX][CL];
    cg::cluster_group cluster = cg::this_cluster();
    pdl_enter_small();
    const size_t base = (size_t)blockIdx.y * a.width;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;       // this thread's four columns
    float4 v[MEAN_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int k = 0; k < MEAN_MAX; ++k) {
        float ssq = 0.f;
        if (k < a.count) {
            v[k] = a.in[k].four(base + i);
            ssq = v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
        ssq = warp_sum(ssq);
        if (lane == 0) red[k][warp] = ssq;
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < MEAN_MAX; ++k) {
            const float t = warp_sum(lane < nwarp ? red[k][lane] : 0.f);
            if (lane == 0) red[k][32] = t;
        }
    }
    __syncthreads();
    // each block tells every block of the cluster its sums; after the one barrier nobody touches another block's
    // shared memory again
    if (threadIdx.x < CL) {
#pragma unroll
        for (int k = 0; k < MEAN_MAX; ++k) cluster.map_shared_rank(&share[k][0], threadIdx.x)[blockIdx.x] = red[k][32];
    }
    cluster.sync();
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < MEAN_MAX; ++k) {
        if (k < a.count) {
            float total = 0.f;
#pragma unroll
            for (int r = 0; r < CL; ++r) total += share[k][r];       // same order in every block
            const float inv = rsqrtf(total / (float)a.width + a.eps);
            const float4 g = *reinterpret_cast<const float4*>(a.gain[k] + i);
            o.x += (v[k].x * inv) * g.x; o.y += (v[k].y * inv) * g.y;
            o.z += (v[k].z * inv) * g.z; o.w += (v[k].w * inv) * g.w;
        }
    }
    o.x *= a.scale; o.y *= a.scale; o.z *= a.scale; o.w *= a.scale;
    if (a.add.p) {
        const float4 f = a.add.four(base + i);
        o.x += f.x; o.y += f.y; o.z += f.z; o.w += f.w;
    }
    *reinterpret_cast<float4*>(a.out + base + i) = o;
}

}  // namespace lily

using namespace lily;

LILY_API int lily_sigmoid_gate(void* out, int out_dtype, const void* gate, int gate_dtype, int gate_splits,
                               size_t gate_stride, size_t total, cudaStream_t stream) {
    if (total == 0) return 0;
    LILY_REQUIRE(gate_splits >= 1 && (gate_splits == 1 || gate_dtype == kF32), "sigmoid_gate: only float32 partial sums come in several splits");
    const Operand g{gate, gate_dtype == kBF16, gate_splits, gate_stride};
    const int blocks = (int)((total + 255) / 256 < (size_t)sm_count() * 16 ? (total + 255) / 256 : (size_t)sm_count() * 16);
    if (out_dtype == kBF16 && gate_dtype == kBF16 && total % 8 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)gate & 15) == 0) {
        const size_t work = total / 8;
        const int b8 = (int)((work + 255) / 256 < (size_t)sm_count() * 16 ? (work + 255) / 256 : (size_t)sm_count() * 16);
        launch_pdl(sigmoid_gate_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, total);
    } else if (out_dtype == kBF16) launch_pdl(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, g, total);
    else launch_pdl(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, g, total);
    LILY_CHECK_LAUNCH("sigmoid_gate");
    return 0;
}

LILY_API int lily_head_mix(const void* in, int in_dtype, int planes, const float* mix, void* out, int tokens, int nq, int nkv,
                           int dv, int out_dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && dv > 0, "head_mix: %d heads over %d kv heads of %d value columns", nq, nkv, dv);
    LILY_REQUIRE(planes || in_dtype == kF32, "head_mix: rows of sums over all kv heads are float32");
    const size_t smem = sizeof(float) * (size_t)nq * nq;
    LILY_REQUIRE(smem <= 48 * 1024, "head_mix: a matrix over %d heads does not fit shared memory", nq);
    const bool aligned = ((uintptr_t)in & 15) == 0;
    const int vec = in_dtype == kBF16 ? (dv % 8 == 0 && aligned ? 8 : 1) : (dv % 4 == 0 && aligned ? 4 : 1);
    const int threads = tokens <= 64 ? 64 : 128;                     // few tokens: more blocks a token
    const size_t plane = (size_t)tokens * nq * dv;
    dim3 grid(tokens, (nq * dv / vec + threads - 1) / threads);
    LILY_REQUIRE(grid.y <= 65535, "head_mix: %d heads of %d value columns", nq, dv);
#define GO(T, IN, V) launch_pdl(head_mix_kernel<T, IN, V>, grid, dim3(threads), smem, stream, (const IN*)in, planes, plane, mix, (T*)out, nq, nkv, dv)
    if (out_dtype == kBF16) {
        if (in_dtype == kBF16) { if (vec == 8) GO(__nv_bfloat16, __nv_bfloat16, 8); else GO(__nv_bfloat16, __nv_bfloat16, 1); }
        else { if (vec == 4) GO(__nv_bfloat16, float, 4); else GO(__nv_bfloat16, float, 1); }
    } else {
        if (in_dtype == kBF16) { if (vec == 8) GO(float, __nv_bfloat16, 8); else GO(float, __nv_bfloat16, 1); }
        else { if (vec == 4) GO(float, float, 4); else GO(float, float, 1); }
    }
#undef GO
    LILY_CHECK_LAUNCH("head_mix");
    return 0;
}

LILY_API int lily_normed_mean_max() { return MEAN_MAX; }

// ins / dtypes / splits / strides / gains: `count` entries each; `add` may be null.
LILY_API int lily_normed_mean(const void* const* ins, const int* dtypes, const int* splits, const size_t* strides,
                              const float* const* gains, int count, const void* add, int add_dtype, int add_splits,
                              size_t add_stride, float* out, int tokens, int width, float eps, float scale,
                              cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(count >= 1 && count <= MEAN_MAX, "normed_mean: %d inputs (1 to %d)", count, MEAN_MAX);
    NormedMeanArgs a{};
    for (int k = 0; k < count; ++k) {
        LILY_REQUIRE(splits[k] >= 1 && (splits[k] == 1 || dtypes[k] == kF32), "normed_mean: only float32 partial sums come in several splits");
        a.in[k] = Operand{ins[k], dtypes[k] == kBF16, splits[k], strides[k]};
        a.gain[k] = gains[k];
    }
    a.count = count;
    a.add = Operand{add, add_dtype == kBF16, add_splits < 1 ? 1 : add_splits, add_stride};
    a.out = out; a.width = width; a.eps = eps; a.scale = scale;
    bool vec = width % 4 == 0 && a.add.vector_ok() && ((uintptr_t)out & 15) == 0;
    for (int k = 0; k < count; ++k) vec = vec && a.in[k].vector_ok() && ((uintptr_t)gains[k] & 15) == 0;
    constexpr int CL = 8;
    if (vec && tokens <= 64 && width % (4 * CL) == 0 && width / (4 * CL) >= 32 && width / (4 * CL) <= 1024) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CL, tokens);
        cfg.blockDim = dim3(width / (4 * CL));
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaLaunchKernelEx(&cfg, normed_mean_cluster_kernel<CL>, a);
        LILY_CHECK_LAUNCH("normed_mean");
        return 0;
    }
    const int threads = width >= 2048 ? 512 : 256;
    if (vec) launch_pdl(normed_mean_kernel<4>, dim3(tokens), dim3(threads), 0, stream, a);
    else launch_pdl(normed_mean_kernel<1>, dim3(tokens), dim3(threads), 0, stream, a);
    LILY_CHECK_LAUNCH("normed_mean");
    return 0;
}
