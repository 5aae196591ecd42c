// Kernels of the differential attention mixer, around the attention kernels it shares with the plain one.
//
// A head carries `maps` softmax maps with queries and keys of their own (d columns each) over the same values (dv).
// The projection's rows are [head][map][d] for q and [kv head][map][d] for k, so a kv head's cached key row is its
// maps' keys side by side (kd = maps * d columns).
//
//   diff_prepare:  q of map m of head h becomes query head h * maps + m of kd columns: the map's d numbers, times the
//                  query temperature 1 + coef * ln(floor((p + 1) / every) + 1) of the token's position p, in columns
//                  [m d, (m + 1) d) and zeros elsewhere, so that its scores over a whole key row are the map's;
//                  k and v go to the token's place in its page.
//   diff_combine:  o = a_0 - lambda a_1 per head, divided by its root mean square over dv (float32), times a constant,
//                  times sigmoid(gate of the head), where the gate numbers are columns of the projection.
//
// Page layout as the attention kernels': keys [kv_heads, page_size, kd] followed by values [kv_heads, page_size, dv].
#include "common.cuh"

namespace lily {

struct DiffPrepareArgs {
    const void* proj;         // [tokens, width]: q | k | v | ... in the cache's dtype
    int width;
    const int* positions;     // [tokens]
    const int* token_req;     // [tokens]
    const int* block_table;   // [requests, bt_stride]
    int bt_stride;
    void* kv;                 // layer base
    void* q_out;              // [tokens, heads * maps, kd]
    int heads, nkv, d, dv, maps, page_size;
    float coef;
    int every;
    int write_kv;
};

// grid (tokens), block 256
template <typename T>
__global__ void diff_prepare_kernel(const DiffPrepareArgs a) {
    pdl_enter_small();
    const int t = blockIdx.x;
    const int kd = a.maps * a.d;
    const T* row = (const T*)a.proj + (size_t)t * a.width;
    const int pos = a.positions[t];
    const float temp = a.coef != 0.f ? 1.f + a.coef * logf((float)((pos + 1) / a.every) + 1.f) : 1.f;
    T* q = (T*)a.q_out + (size_t)t * a.heads * a.maps * kd;
    const int qn = a.heads * a.maps * kd;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) {
        const int c = i % kd, hm = i / kd, m = hm % a.maps, h = hm / a.maps;
        const float v = (c / a.d == m) ? to_float(row[h * kd + c]) * temp : 0.f;
        q[i] = from_float<T>(v);
    }
    if (!a.write_kv) return;
    const int page = a.block_table[(size_t)a.token_req[t] * a.bt_stride + pos / a.page_size];
    const int within = pos % a.page_size;
    const size_t khead = (size_t)a.page_size * kd, vhead = (size_t)a.page_size * a.dv;
    T* base = (T*)a.kv + (size_t)page * a.nkv * (khead + vhead);
    const T* ksrc = row + a.heads * kd;
    const T* vsrc = ksrc + a.nkv * kd;
    for (int i = threadIdx.x; i < a.nkv * kd; i += blockDim.x) {
        const int g = i / kd, c = i % kd;
        base[(size_t)g * khead + (size_t)within * kd + c] = ksrc[i];
    }
    for (int i = threadIdx.x; i < a.nkv * a.dv; i += blockDim.x) {
        const int g = i / a.dv, c = i % a.dv;
        base[(size_t)a.nkv * khead + (size_t)g * vhead + (size_t)within * a.dv + c] = vsrc[i];
    }
}

// The same in pieces of 16 bytes (V = 8 bfloat16 or 4 float32 numbers): d, dv and the row widths are multiples of V and
// every base is 16-byte aligned, so a piece never straddles a map, a head or a row.  grid (tokens), block 256.
template <typename T>
__global__ void diff_prepare_vec_kernel(const DiffPrepareArgs a) {
    constexpr int V = 16 / sizeof(T);
    pdl_enter_small();
    const int t = blockIdx.x;
    const int kd = a.maps * a.d;
    const T* row = (const T*)a.proj + (size_t)t * a.width;
    const int pos = a.positions[t];
    const float temp = a.coef != 0.f ? 1.f + a.coef * logf((float)((pos + 1) / a.every) + 1.f) : 1.f;
    T* q = (T*)a.q_out + (size_t)t * a.heads * a.maps * kd;
    const int per_head = kd / V, qn = a.heads * a.maps * per_head;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) {
        const int c = (i % per_head) * V, hm = i / per_head, m = hm % a.maps, h = hm / a.maps;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c / a.d == m) {
            raw = *reinterpret_cast<const uint4*>(row + h * kd + c);
            T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int k = 0; k < V; ++k) e[k] = from_float<T>(to_float(e[k]) * temp);
        }
        *reinterpret_cast<uint4*>(q + (size_t)hm * kd + c) = raw;
    }
    if (!a.write_kv) return;
    const int page = a.block_table[(size_t)a.token_req[t] * a.bt_stride + pos / a.page_size];
    const int within = pos % a.page_size;
    const size_t khead = (size_t)a.page_size * kd, vhead = (size_t)a.page_size * a.dv;
    T* base = (T*)a.kv + (size_t)page * a.nkv * (khead + vhead);
    const T* ksrc = row + a.heads * kd;
    const T* vsrc = ksrc + a.nkv * kd;
    const int kn = a.nkv * per_head, per_v = a.dv / V, vn = a.nkv * per_v;
    for (int i = threadIdx.x; i < kn + vn; i += blockDim.x) {
        if (i < kn) {
            const int g = i / per_head, c = (i % per_head) * V;
            *reinterpret_cast<uint4*>(base + (size_t)g * khead + (size_t)within * kd + c) = *reinterpret_cast<const uint4*>(ksrc + g * kd + c);
        } else {
            const int j = i - kn, g = j / per_v, c = (j % per_v) * V;
            *reinterpret_cast<uint4*>(base + (size_t)a.nkv * khead + (size_t)g * vhead + (size_t)within * a.dv + c) =
                *reinterpret_cast<const uint4*>(vsrc + g * a.dv + c);
        }
    }
}

// a warp per (token, head); block of 4 warps
template <typename T>
__global__ void diff_combine_kernel(const T* __restrict__ maps_out, const T* __restrict__ proj, int width, int gate_col,
                                    T* __restrict__ out, int tokens, int heads, int dv, float lam, float out_scale, float eps) {
    pdl_enter_small();
    const int lane = threadIdx.x & 31;
    const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (size_t)tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const T* a0 = maps_out + ((size_t)t * heads + h) * 2 * dv;
    const T* a1 = a0 + dv;
    float ssq = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float o = to_float(a0[c]) - lam * to_float(a1[c]);
        ssq = fmaf(o, o, ssq);
    }
    ssq = warp_sum(ssq);
    const float gate = 1.f / (1.f + expf(-to_float(proj[(size_t)t * width + gate_col + h])));
    const float f = rsqrtf(ssq / (float)dv + eps) * out_scale * gate;
    T* dst = out + ((size_t)t * heads + h) * dv;
    for (int c = lane; c < dv; c += 32) {
        const float o = to_float(a0[c]) - lam * to_float(a1[c]);
        dst[c] = from_float<T>(o * f);
    }
}

// The same with 16-byte pieces (V = 8 bfloat16 or 4 float32 numbers) kept in registers between the sum of squares and
// the output.  `lanes` (a power of two up to 32) neighbouring lanes share a (token, head), so that a warp takes
// 32 / lanes of them at once; dv is a multiple of V and at most lanes * V * R; every base is 16-byte aligned.
template <typename T, int R>
__global__ void diff_combine_vec_kernel(const T* __restrict__ maps_out, const T* __restrict__ proj, int width, int gate_col,
                                        T* __restrict__ out, int tokens, int heads, int dv, int lanes, float lam, float out_scale,
                                        float eps) {
    constexpr int V = 16 / sizeof(T);
    pdl_enter_small();
    const int lane = threadIdx.x & 31, sub = lane / lanes, l = lane % lanes;
    const size_t item = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32 / lanes) + sub;
    const bool live = item < (size_t)tokens * heads;
    const int t = live ? (int)(item / heads) : 0, h = live ? (int)(item % heads) : 0;
    const T* a0 = maps_out + ((size_t)t * heads + h) * 2 * dv;
    const T* a1 = a0 + dv;
    float o[R][V];
    float ssq = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = (r * lanes + l) * V;
        if (live && c < dv) {
            const uint4 x = *reinterpret_cast<const uint4*>(a0 + c), y = *reinterpret_cast<const uint4*>(a1 + c);
            const T* xe = reinterpret_cast<const T*>(&x);
            const T* ye = reinterpret_cast<const T*>(&y);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                o[r][k] = to_float(xe[k]) - lam * to_float(ye[k]);
                ssq = fmaf(o[r][k], o[r][k], ssq);
            }
        }
    }
    for (int off = lanes >> 1; off > 0; off >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, off);
    if (!live) return;
    const float gate = 1.f / (1.f + expf(-to_float(proj[(size_t)t * width + gate_col + h])));
    const float f = rsqrtf(ssq / (float)dv + eps) * out_scale * gate;
    T* dst = out + ((size_t)t * heads + h) * dv;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = (r * lanes + l) * V;
        if (c < dv) {
            uint4 w;
            T* we = reinterpret_cast<T*>(&w);
#pragma unroll
            for (int k = 0; k < V; ++k) we[k] = from_float<T>(o[r][k] * f);
            *reinterpret_cast<uint4*>(dst + c) = w;
        }
    }
}

}  // namespace lily

using namespace lily;

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

LILY_API int lily_diff_prepare(const void* proj, int width, const int* positions, const int* token_req,
                               const int* block_table, int bt_stride, void* kv, void* q_out, int tokens, int heads,
                               int nkv, int d, int dv, int maps, int page_size, float coef, int every, int write_kv,
                               int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(heads > 0 && nkv > 0 && heads % nkv == 0 && d > 0 && dv > 0 && maps >= 1, "diff_prepare: %d heads over %d kv heads, sizes %d / %d, %d maps", heads, nkv, d, dv, maps);
    LILY_REQUIRE(every >= 1 && page_size > 0, "diff_prepare: temperature step %d, page size %d", every, page_size);
    LILY_REQUIRE(width >= (heads + nkv) * maps * d + nkv * dv, "diff_prepare: rows of %d columns do not hold q, k and v", width);
    DiffPrepareArgs a{proj, width, positions, token_req, block_table, bt_stride, kv, q_out, heads, nkv, d, dv, maps, page_size, coef, every, write_kv};
    const int v = dtype == kBF16 ? 8 : 4;
    const bool vec = d % v == 0 && dv % v == 0 && width % v == 0 && aligned16(proj) && aligned16(kv) && aligned16(q_out);
    if (dtype == kBF16) {
        if (vec) launch_pdl(diff_prepare_vec_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, a);
        else launch_pdl(diff_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, a);
    } else {
        if (vec) launch_pdl(diff_prepare_vec_kernel<float>, dim3(tokens), dim3(256), 0, stream, a);
        else launch_pdl(diff_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, a);
    }
    LILY_CHECK_LAUNCH("diff_prepare");
    return 0;
}

LILY_API int lily_diff_combine(const void* maps_out, const void* proj, int width, int gate_col, void* out, int tokens,
                               int heads, int dv, int maps, float lam, float out_scale, float eps, int dtype,
                               cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(maps == 2, "diff_combine: %d maps (the difference is of two)", maps);
    LILY_REQUIRE(gate_col >= 0 && gate_col + heads <= width, "diff_combine: gate columns %d.. of %d", gate_col, width);
    const size_t items = (size_t)tokens * heads;
    const int v = dtype == kBF16 ? 8 : 4;
    if (dv % v == 0 && dv <= 32 * v * 2 && aligned16(maps_out) && aligned16(out)) {
        int lanes = 1;
        while (lanes < 32 && lanes * v < dv) lanes *= 2;                  // a power of two: the pieces of a head, up to a warp
        const size_t per_block = (size_t)4 * (32 / lanes);
        const dim3 grid((unsigned)((items + per_block - 1) / per_block)), block(128);
        if (dtype == kBF16)
            launch_pdl(diff_combine_vec_kernel<__nv_bfloat16, 2>, grid, block, 0, stream, (const __nv_bfloat16*)maps_out, (const __nv_bfloat16*)proj, width, gate_col, (__nv_bfloat16*)out, tokens, heads, dv, lanes, lam, out_scale, eps);
        else
            launch_pdl(diff_combine_vec_kernel<float, 2>, grid, block, 0, stream, (const float*)maps_out, (const float*)proj, width, gate_col, (float*)out, tokens, heads, dv, lanes, lam, out_scale, eps);
        LILY_CHECK_LAUNCH("diff_combine");
        return 0;
    }
    const dim3 grid((unsigned)((items + 3) / 4)), block(128);
    if (dtype == kBF16)
        launch_pdl(diff_combine_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)maps_out, (const __nv_bfloat16*)proj, width, gate_col, (__nv_bfloat16*)out, tokens, heads, dv, lam, out_scale, eps);
    else
        launch_pdl(diff_combine_kernel<float>, grid, block, 0, stream, (const float*)maps_out, (const float*)proj, width, gate_col, (float*)out, tokens, heads, dv, lam, out_scale, eps);
    LILY_CHECK_LAUNCH("diff_combine");
    return 0;
}
