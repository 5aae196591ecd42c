// Kernels around a sublayer that has a norm behind it as well as ahead of it, and the plain (ungated) feed-forward.
//
//   add_normed_rmsnorm:  u = delta / sqrt(mean(delta^2) + eps_post) * gain_post         (the norm behind the sublayer; or, with
//                                                                                         `normalise` 0, u = delta * gain_post: a gain
//                                                                                         per column alone, a layer scale)
//                        v = resid + mult * u;  resid = v (when asked)                   (the add, float32)
//                        out = v / sqrt(mean(v^2) + eps) * weight                        (the norm ahead of the next one)
//   activation:          out = act(in), act = SiLU, the tanh form of GELU, or the square of max(., 0)
//
// `delta` and `in` may be the activation dtype, float32, or the float32 partial sums of a split-k product.  Sums of
// squares, roots and the residual stream are float32 whatever the activation dtype.
#include "common.cuh"
#include "operand.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace lily {

struct NormedAddArgs {
    float* resid;             // [tokens, hidden]
    Operand delta;            // [tokens, hidden]
    const float* post_gain;   // [hidden]
    const void* weight;       // [hidden], float32 or bfloat16; null: no output, the add alone
    int weight_bf16;
    void* out;                // [rows or tokens, hidden]
    const int* rows;          // null: every token; else the tokens whose output is wanted (nothing is written back then)
    int hidden;
    float post_eps, eps, mult;
    int write_residual;
    int normalise;            // 0: the delta is not divided by its root mean square (post_gain alone scales it)
};

__device__ __forceinline__ float gain_at(const void* w, int bf16, int i) {
    return bf16 ? __bfloat162float(((const __nv_bfloat16*)w)[i]) : ((const float*)w)[i];
}

// One block per output row; the row is kept in shared memory between the passes.
template <typename T, int VEC>
__global__ void add_normed_rmsnorm_kernel(const NormedAddArgs a) {
    extern __shared__ __align__(16) float smem[];
    pdl_enter_small();
    float* red = smem;             // 33 floats
    float* row = smem + 40;        // hidden floats
    const int m = blockIdx.x, hidden = a.hidden;
    const size_t src = (size_t)(a.rows ? a.rows[m] : m) * hidden;
    float ssq = 0.f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            const float4 d = a.delta.four(src + i);
            *reinterpret_cast<float4*>(row + i) = d;
            ssq += d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float d = a.delta(src + i);
            row[i] = d;
            ssq = fmaf(d, d, ssq);
        }
    }
    const float inv_d = a.normalise ? rsqrtf(block_sum(ssq, red) / (float)hidden + a.post_eps) : 1.f;
    __syncthreads();               // the row is whole before other threads' entries are read (the sum above may be skipped)
    ssq = 0.f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            const float4 d = *reinterpret_cast<const float4*>(row + i);
            const float4 g = *reinterpret_cast<const float4*>(a.post_gain + i);
            float4 v = *reinterpret_cast<const float4*>(a.resid + src + i);
            v.x += a.mult * ((d.x * inv_d) * g.x);
            v.y += a.mult * ((d.y * inv_d) * g.y);
            v.z += a.mult * ((d.z * inv_d) * g.z);
            v.w += a.mult * ((d.w * inv_d) * g.w);
            if (a.write_residual) *reinterpret_cast<float4*>(a.resid + src + i) = v;
            *reinterpret_cast<float4*>(row + i) = v;
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = a.resid[src + i] + a.mult * ((row[i] * inv_d) * a.post_gain[i]);
            if (a.write_residual) a.resid[src + i] = v;
            row[i] = v;
            ssq = fmaf(v, v, ssq);
        }
    }
    if (a.weight == nullptr) return;
    const float inv = rsqrtf(block_sum(ssq, red) / (float)hidden + a.eps);
    T* dst = (T*)a.out + (size_t)m * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = from_float<T>((row[i] * inv) * gain_at(a.weight, a.weight_bf16, i));
}

// Sum over the block with one barrier: every thread adds the warps' sums in the same order.  `slots` holds a float per
// warp and is not used again before the next barrier of the block.
__device__ __forceinline__ float block_sum_once(float v, float* slots) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += slots[w];
    return t;
}

template <typename T> __device__ __forceinline__ void store_four(T* dst, float4 v);
template <> __device__ __forceinline__ void store_four<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <> __device__ __forceinline__ void store_four<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = w;
}

// One block per output row with the row in registers: PER pieces of four columns a thread (hidden = 4 * PER * threads),
// a barrier per sum of squares, outputs stored four at a time.  Bases 16-byte aligned.
template <typename T, int PER>
__global__ void add_normed_rmsnorm_reg_kernel(const NormedAddArgs a) {
    __shared__ float slots[2][32];
    pdl_enter_small();
    const int m = blockIdx.x, hidden = a.hidden;
    const size_t src = (size_t)(a.rows ? a.rows[m] : m) * hidden;
    float4 d[PER], v[PER];
    float ssq = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = (k * blockDim.x + threadIdx.x) * 4;
        d[k] = a.delta.four(src + i);
        v[k] = *reinterpret_cast<const float4*>(a.resid + src + i);
        ssq += d[k].x * d[k].x + d[k].y * d[k].y + d[k].z * d[k].z + d[k].w * d[k].w;
    }
    const float inv_d = a.normalise ? rsqrtf(block_sum_once(ssq, slots[0]) / (float)hidden + a.post_eps) : 1.f;
    ssq = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = (k * blockDim.x + threadIdx.x) * 4;
        const float4 g = *reinterpret_cast<const float4*>(a.post_gain + i);
        v[k].x += a.mult * ((d[k].x * inv_d) * g.x);
        v[k].y += a.mult * ((d[k].y * inv_d) * g.y);
        v[k].z += a.mult * ((d[k].z * inv_d) * g.z);
        v[k].w += a.mult * ((d[k].w * inv_d) * g.w);
        if (a.write_residual) *reinterpret_cast<float4*>(a.resid + src + i) = v[k];
        ssq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
    if (a.weight == nullptr) return;
    const float inv = rsqrtf(block_sum_once(ssq, slots[1]) / (float)hidden + a.eps);
    T* dst = (T*)a.out + (size_t)m * hidden;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = (k * blockDim.x + threadIdx.x) * 4;
        store_four<T>(dst + i, make_float4((v[k].x * inv) * gain_at(a.weight, a.weight_bf16, i), (v[k].y * inv) * gain_at(a.weight, a.weight_bf16, i + 1),
                                           (v[k].z * inv) * gain_at(a.weight, a.weight_bf16, i + 2), (v[k].w * inv) * gain_at(a.weight, a.weight_bf16, i + 3)));
    }
}

// The same for a few rows: a cluster of CL blocks shares a row, each block takes hidden / CL columns (four a thread)
// and the blocks exchange their two sums of squares through distributed shared memory, so that 8 rows keep 64 SMs
// busy instead of 8.  grid (CL, rows), cluster (CL, 1, 1); hidden % (4 * CL) == 0; block = hidden / (4 * CL) threads.
template <typename T, int CL>
__global__ void add_normed_rmsnorm_cluster_kernel(const NormedAddArgs a) {
    __shared__ float red[40];
    __shared__ float share[2][CL];
    cg::cluster_group cluster = cg::this_cluster();
    pdl_enter_small();
    const int m = blockIdx.y, hidden = a.hidden;
    const size_t src = (size_t)(a.rows ? a.rows[m] : m) * hidden;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const float4 d = a.delta.four(src + i);
    const float4 g = *reinterpret_cast<const float4*>(a.post_gain + i);
    float4 v = *reinterpret_cast<const float4*>(a.resid + src + i);
    float mine = 0.f, total = 0.f, inv_d = 1.f;
    if (a.normalise) {                                                  // the same branch in every block of the launch
        mine = block_sum(d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w, red);
        if (threadIdx.x < CL) cluster.map_shared_rank(&share[0][0], threadIdx.x)[blockIdx.x] = mine;
        cluster.sync();
#pragma unroll
        for (int r = 0; r < CL; ++r) total += share[0][r];              // same order in every block
        inv_d = rsqrtf(total / (float)hidden + a.post_eps);
    }
    v.x += a.mult * ((d.x * inv_d) * g.x);
    v.y += a.mult * ((d.y * inv_d) * g.y);
    v.z += a.mult * ((d.z * inv_d) * g.z);
    v.w += a.mult * ((d.w * inv_d) * g.w);
    if (a.write_residual) *reinterpret_cast<float4*>(a.resid + src + i) = v;
    mine = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, red);
    if (threadIdx.x < CL) cluster.map_shared_rank(&share[1][0], threadIdx.x)[blockIdx.x] = mine;
    cluster.sync();                 // after it nobody touches another block's shared memory again
    if (a.weight == nullptr) return;
    total = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) total += share[1][r];
    const float inv = rsqrtf(total / (float)hidden + a.eps);
    T* dst = (T*)a.out + (size_t)m * hidden + i;
    dst[0] = from_float<T>((v.x * inv) * gain_at(a.weight, a.weight_bf16, i));
    dst[1] = from_float<T>((v.y * inv) * gain_at(a.weight, a.weight_bf16, i + 1));
    dst[2] = from_float<T>((v.z * inv) * gain_at(a.weight, a.weight_bf16, i + 2));
    dst[3] = from_float<T>((v.w * inv) * gain_at(a.weight, a.weight_bf16, i + 3));
}

// act: 0 SiLU, 1 the tanh form of GELU, 2 the square of max(., 0)
__device__ __forceinline__ float activate(int act, float z) {
    if (act == 2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (act == 0) return z / (1.f + expf(-z));
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T, int VEC>
__global__ void activation_kernel(const Operand in, T* __restrict__ out, size_t total, int act) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x * VEC;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += step) {
        if (VEC == 4) {
            const float4 z = in.four(i);
            out[i] = from_float<T>(activate(act, z.x));
            out[i + 1] = from_float<T>(activate(act, z.y));
            out[i + 2] = from_float<T>(activate(act, z.z));
            out[i + 3] = from_float<T>(activate(act, z.w));
        } else {
            out[i] = from_float<T>(activate(act, in(i)));
        }
    }
}

// bfloat16 in one piece to bfloat16, eight entries a thread and turn (16-byte accesses)
__global__ void activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t total, int act) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x * 8;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += step) {
        uint4 v = *reinterpret_cast<const uint4*>(in + i);
        __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 z = __bfloat1622float2(v2[k]);
            v2[k] = __floats2bfloat162_rn(activate(act, z.x), activate(act, z.y));
        }
        *reinterpret_cast<uint4*>(out + i) = v;
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_add_normed_rmsnorm(float* resid, const void* delta, int delta_dtype, int delta_splits, size_t delta_stride,
                                     const float* post_gain, float post_eps, float mult, const void* weight, int weight_dtype,
                                     void* out, int out_dtype, const int* rows, int n_out, int hidden, float eps,
                                     int write_residual, int normalise, cudaStream_t stream) {
    if (n_out == 0) return 0;
    LILY_REQUIRE(delta_splits >= 1 && (delta_splits == 1 || delta_dtype == kF32), "add_normed_rmsnorm: only float32 partial sums come in several splits");
    LILY_REQUIRE(hidden > 0 && hidden <= 48 * 1024, "add_normed_rmsnorm: width %d", hidden);
    LILY_REQUIRE(weight == nullptr || out != nullptr, "add_normed_rmsnorm: a gain without an output");
    LILY_REQUIRE(!(rows && write_residual), "add_normed_rmsnorm: gathered rows are not written back");
    NormedAddArgs a{};
    a.resid = resid; a.delta = Operand{delta, delta_dtype == kBF16, delta_splits, delta_stride}; a.post_gain = post_gain;
    a.weight = weight; a.weight_bf16 = weight_dtype == kBF16; a.out = out; a.rows = rows; a.hidden = hidden;
    a.post_eps = post_eps; a.eps = eps; a.mult = mult; a.write_residual = write_residual; a.normalise = normalise;
    const bool vec = hidden % 4 == 0 && a.delta.vector_ok() && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)post_gain & 15) == 0;
    constexpr int CL = 8;
    if (vec && n_out <= 64 && hidden % (4 * CL * 32) == 0 && hidden / (4 * CL) <= 1024) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CL, n_out);
        cfg.blockDim = dim3(hidden / (4 * CL));
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t e = out_dtype == kBF16 ? cudaLaunchKernelEx(&cfg, add_normed_rmsnorm_cluster_kernel<__nv_bfloat16, CL>, a)
                                           : cudaLaunchKernelEx(&cfg, add_normed_rmsnorm_cluster_kernel<float, CL>, a);
        if (e != cudaSuccess) { set_error("add_normed_rmsnorm: launch failed: %s", cudaGetErrorString(e)); return 2; }
        return 0;
    }
    // whole rows in registers: 32 to 256 threads with 1, 2, 4 or 8 pieces of four columns each
    if (vec && ((uintptr_t)out & 15) == 0) {
        int t = 0, per = 0;
        for (int threads = 256; threads >= 32 && !per; threads /= 2)
            for (int pieces = 1; pieces <= 8 && !per; pieces *= 2)
                if (hidden == 4 * threads * pieces) { t = threads; per = pieces; }
        if (per == 1 || per == 2 || per == 4 || per == 8) {
#define REG(T)                                                                                        \
            do {                                                                                      \
                if (per == 1) launch_pdl(add_normed_rmsnorm_reg_kernel<T, 1>, dim3(n_out), dim3(t), 0, stream, a);       \
                else if (per == 2) launch_pdl(add_normed_rmsnorm_reg_kernel<T, 2>, dim3(n_out), dim3(t), 0, stream, a);  \
                else if (per == 4) launch_pdl(add_normed_rmsnorm_reg_kernel<T, 4>, dim3(n_out), dim3(t), 0, stream, a);  \
                else launch_pdl(add_normed_rmsnorm_reg_kernel<T, 8>, dim3(n_out), dim3(t), 0, stream, a);                \
            } while (0)
            if (out_dtype == kBF16) REG(__nv_bfloat16); else REG(float);
#undef REG
            LILY_CHECK_LAUNCH("add_normed_rmsnorm");
            return 0;
        }
    }
    const size_t smem = sizeof(float) * (40 + (size_t)hidden);
    int threads = vec ? (hidden / 4 + 31) / 32 * 32 : (hidden + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
#define GO(T, V)                                                                                                    \
    do {                                                                                                            \
        auto kern = add_normed_rmsnorm_kernel<T, V>;                                                                \
        static size_t granted = 48 * 1024;                                                                          \
        if (smem > granted) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
            if (e != cudaSuccess) { set_error("add_normed_rmsnorm: cannot get %zu bytes of shared memory", smem); return 2; } \
            granted = smem;                                                                                         \
        }                                                                                                           \
        launch_pdl(kern, dim3(n_out), dim3(threads), smem, stream, a);                                              \
    } while (0)
    if (out_dtype == kBF16) { if (vec) GO(__nv_bfloat16, 4); else GO(__nv_bfloat16, 1); }
    else { if (vec) GO(float, 4); else GO(float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("add_normed_rmsnorm");
    return 0;
}

LILY_API int lily_activation(const void* in, int in_dtype, int in_splits, size_t in_stride, void* out, int out_dtype,
                             size_t total, int act, cudaStream_t stream) {
    if (total == 0) return 0;
    LILY_REQUIRE(act >= 0 && act <= 2, "activation: code %d (0 SiLU, 1 GELU tanh, 2 squared ReLU)", act);
    LILY_REQUIRE(in_splits >= 1 && (in_splits == 1 || in_dtype == kF32), "activation: only float32 partial sums come in several splits");
    const Operand x{in, in_dtype == kBF16, in_splits, in_stride};
    auto blocks_for = [](size_t work) { return (int)((work + 255) / 256 < (size_t)sm_count() * 16 ? (work + 255) / 256 : (size_t)sm_count() * 16); };
    if (in_dtype == kBF16 && out_dtype == kBF16 && total % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        launch_pdl(activation_bf16x8_kernel, dim3(blocks_for(total / 8)), dim3(256), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, act);
    } else if (total % 4 == 0 && x.vector_ok()) {
        if (out_dtype == kBF16) launch_pdl(activation_kernel<__nv_bfloat16, 4>, dim3(blocks_for(total / 4)), dim3(256), 0, stream, x, (__nv_bfloat16*)out, total, act);
        else launch_pdl(activation_kernel<float, 4>, dim3(blocks_for(total / 4)), dim3(256), 0, stream, x, (float*)out, total, act);
    } else {
        if (out_dtype == kBF16) launch_pdl(activation_kernel<__nv_bfloat16, 1>, dim3(blocks_for(total)), dim3(256), 0, stream, x, (__nv_bfloat16*)out, total, act);
        else launch_pdl(activation_kernel<float, 1>, dim3(blocks_for(total)), dim3(256), 0, stream, x, (float*)out, total, act);
    }
    LILY_CHECK_LAUNCH("activation");
    return 0;
}
