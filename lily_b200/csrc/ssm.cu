// Kernels of the state-space mixer (Mamba-2 / state-space duality): the short causal convolution with its
// carried inputs, the selective scan with its carried state, and the gated, grouped RMSNorm behind it.
//
// Everything that enters the recurrence is float32: the step size softplus(dt + bias), the decay
// exp(-exp(A_log) * dt), the state and the sums over it.  Activations (`T`) are float or bfloat16.
//
// Per request the state lives in one float32 row of a slot table: first the scan state
// [heads][head_dim][state] (state index fastest), then the last (taps - 1) inputs of the convolution
// [(taps - 1)][channels], oldest first.  A request's row is zero when it starts.
//
//   conv:  u_t[c] = silu(bias[c] + sum_j w[c][j] * in_(t - (taps-1) + j)[c])        (inputs before the start are 0)
//   scan:  S_t = exp(a * dt_t) S_(t-1) + dt_t * B_t x_t^T,   y_t = S_t^T C_t + D x_t     per head, a = -exp(A_log)
//   norm:  v = y * silu(z);  out = v / sqrt(mean_over_group(v^2) + eps) * gain
#include "common.cuh"

namespace lily {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
// SiLU where the result is rounded to bfloat16 anyway: the fast exponential and quotient (float32 keeps the exact ones)
template <typename T> __device__ __forceinline__ float silu_for(float v) { return silu_f(v); }
template <> __device__ __forceinline__ float silu_for<__nv_bfloat16>(float v) { return __fdividef(v, 1.f + __expf(-v)); }

__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src));
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void copies_wait_all_but_one() { asm volatile("cp.async.wait_group 1;\n" ::); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---------------------------------------------------------------------------- causal convolution + SiLU

// grid (ceil(channels / 128), chunks), block 128: a thread owns one channel of one chunk of up to `chunk_len`
// consecutive new tokens of one request (chunks start at multiples of chunk_len >= taps - 1 from the portion's
// first token, so only a portion's first chunk reads the carried inputs; the thread of that chunk also writes
// them back, after it has read them, so no other thread touches what it reads).
// SILU false: the convolution alone (a mixer that convolves its projections and applies no activation).
template <typename T, int TAPS, bool SILU = true>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int in_stride, int col0, int channels,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        float* __restrict__ state, size_t state_stride, size_t state_off,
                                        T* __restrict__ out, const int* __restrict__ chunk_req,
                                        const int* __restrict__ chunk_start, int chunk_len,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
    pdl_enter_small();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int r = chunk_req[blockIdx.y], start = chunk_start[blockIdx.y];
    const int tok0 = cu_seqlens[r], len = cu_seqlens[r + 1] - tok0;
    const int n = min(chunk_len, len - start);
    if (n <= 0) return;
    constexpr int K1 = TAPS - 1;
    float* st = state + (size_t)slots[r] * state_stride + state_off + c;
    const T* src = in + (size_t)tok0 * in_stride + col0 + c;
    float win[K1 > 0 ? K1 : 1];
    if (start == 0) {
#pragma unroll
        for (int j = 0; j < K1; ++j) win[j] = st[(size_t)j * channels];
        if (len > chunk_len) {
#pragma unroll
            for (int j = 0; j < K1; ++j) st[(size_t)j * channels] = to_float(src[(size_t)(len - K1 + j) * in_stride]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < K1; ++j) win[j] = to_float(src[(size_t)(start - K1 + j) * in_stride]);
    }
    float wt[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)c * TAPS + j];
    const float b = bias ? bias[c] : 0.f;
    T* dst = out + (size_t)(tok0 + start) * channels + c;
    const T* from = src + (size_t)start * in_stride;
    for (int t = 0; t < n; t += 4) {                 // four tokens' inputs asked for before the first is used
        float xs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) xs[u] = t + u < n ? to_float(from[(size_t)u * in_stride]) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t + u < n) {
                const float x = xs[u];
                float acc = b;
#pragma unroll
                for (int j = 0; j < K1; ++j) acc = fmaf(win[j], wt[j], acc);
                acc = fmaf(x, wt[K1], acc);
#pragma unroll
                for (int j = 0; j + 1 < K1; ++j) win[j] = win[j + 1];
                if (K1 > 0) win[K1 - 1] = x;
                dst[(size_t)u * channels] = from_float<T>(SILU ? silu_for<T>(acc) : acc);
            }
        }
        from += (size_t)4 * in_stride;
        dst += (size_t)4 * channels;
    }
    if (start == 0 && len <= chunk_len) {
#pragma unroll
        for (int j = 0; j < K1; ++j) st[(size_t)j * channels] = win[j];
    }
}

// ---------------------------------------------------------------------------- selective scan

// grid (heads, requests, ceil(head_dim / pb)), block (pb / PC) * ns threads: `ns` neighbouring lanes share PC
// neighbouring value columns of the head's state and hold a run of NPT of their `n_state` entries each in registers
// (PC * NPT numbers a thread, so that one B and one C entry read from shared memory serve 2 * PC multiply-adds); the tokens of the request run one after another, staged `tt` at a time in shared memory (B and C
// of the head's group, the head's x, step sizes and decays).
//
// A work item (blockIdx.y) is a run of consecutive new tokens of one request.  Without item lists it is a request's
// whole portion, from the state in the request's slot to the state in the request's slot (mode 0).  A long portion
// is cut into chunks that run side by side: mode 1 starts each chunk from zero and leaves the chunk's own state and
// the product of its decays in a workspace (EMIT false: no outputs, and no recurrence either: the chunk's state is
// the sum over its tokens of w_t B_t x_t^T with w_t = dt_t times the decays of the tokens after t, which the block
// works out first, so that a state entry costs one multiply-add a token); a combine kernel then walks the chunks in order,
// S <- decay_c S + state_c, leaving in the workspace the state each chunk starts from and in the slot the last one;
// mode 2 runs each chunk again from that state and writes the outputs.
template <typename T, int NPT, int PC, bool EMIT>
__global__ void __launch_bounds__(256, 2)
ssd_scan_kernel(const T* __restrict__ xbc, int channels, const T* __restrict__ proj, int proj_stride,
                int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const float* __restrict__ d_skip, float* __restrict__ state, size_t state_stride,
                float* __restrict__ y, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int heads, int pd, int n_state, int groups, int ns,
                int pb, int tt, const int* __restrict__ item_req, const int* __restrict__ item_start,
                const int* __restrict__ item_len, int mode, float* __restrict__ chunk_state,
                float* __restrict__ chunk_decay, int ahead, int max_len, int wide) {
    extern __shared__ __align__(16) float smem[];
    pdl_enter_small();
    // Lane j of the ns lanes that share PC columns holds entries [j * NPT, (j + 1) * NPT) of each column's state.  In
    // shared memory a token's B (and C) is laid out lane by lane in rows of NPT + 4, so that the lanes' 16-byte reads
    // fall into different banks; entries past n_state are zero there and leave their (zero) state entries alone.
    constexpr int ROW = NPT + 4;
    const int h = blockIdx.x, item = blockIdx.y, p0 = blockIdx.z * pb;
    const int r = item_req ? item_req[item] : item;
    const int tid = threadIdx.x, j = tid % ns, pl = (tid / ns) * PC, p = p0 + pl;     // this thread's first column
    const int tok0 = cu_seqlens[r] + (item_start ? item_start[item] : 0);
    const int len = item_len ? item_len[item] : cu_seqlens[r + 1] - cu_seqlens[r];
    if (len <= 0) return;
    const int padded = ns * NPT, row = ns * ROW;
    float* Bs = smem;                        // [tt][ns][ROW]
    float* Cs = Bs + (size_t)tt * row;       // [tt][ns][ROW]
    float* xs = Cs + (size_t)tt * row;       // [tt][pb]
    float* dts = xs + (size_t)tt * pb;       // [tt]
    float* das = dts + tt;                   // [tt]
    float* wts = das + tt;                   // mode 1: [max_len] weights w_t, then [max_len] decays
    const int inner = heads * pd;
    const int g = h / (heads / groups);
    const int bcol = inner + g * n_state, ccol = inner + (groups + g) * n_state;
    // `ahead`: the next stage's B, C and x rows are copied as they are (16-byte pieces, asynchronously) into one of two
    // raw buffers while this stage is worked on, and spread into the padded float32 layout when their turn comes
    const int ex = 16 / (int)sizeof(T);                                   // elements a piece
    const int pieces_b = n_state / ex, pieces_x = pb / ex, pieces = 2 * pieces_b + pieces_x;     // of one token
    T* raw = reinterpret_cast<T*>(wts + (EMIT ? 0 : 2 * max_len));        // [2][tt][pieces * ex]
    float dt_ahead = 0.f;
    auto ask = [&](int t0, int buf) {
        const int now = min(tt, len - t0);
        for (int q = tid; q < now * pieces; q += blockDim.x) {
            const int ti = q / pieces, k = q - ti * pieces;
            const T* src = xbc + (size_t)(tok0 + t0 + ti) * channels;
            const T* from = k < pieces_b ? src + bcol + k * ex
                          : (k < 2 * pieces_b ? src + ccol + (k - pieces_b) * ex : src + h * pd + p0 + (k - 2 * pieces_b) * ex);
            if (k < 2 * pieces_b || p0 + (k - 2 * pieces_b) * ex < pd)
                copy16_async(raw + ((size_t)(buf * tt + ti) * pieces + k) * ex, from);
        }
        if (EMIT && tid < now) dt_ahead = to_float(proj[(size_t)(tok0 + t0 + tid) * proj_stride + dt_col + h]);
    };
    float* st = (mode == 0 ? state + (size_t)slots[r] * state_stride : chunk_state + (size_t)item * heads * pd * n_state) +
                (size_t)h * pd * n_state;
    float S[PC][NPT];
    // 16-byte accesses to the state where its rows allow them (`wide`: n_state a multiple of four, aligned bases)
    const bool whole_run = wide && (j + 1) * NPT <= n_state;
#pragma unroll
    for (int c = 0; c < PC; ++c) {
        if (whole_run && mode != 1 && p + c < pd) {
            const float4* src4 = reinterpret_cast<const float4*>(st + (size_t)(p + c) * n_state + j * NPT);
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                const float4 v = src4[q];
                S[c][4 * q] = v.x; S[c][4 * q + 1] = v.y; S[c][4 * q + 2] = v.z; S[c][4 * q + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const int n = j * NPT + i;
                S[c][i] = (mode != 1 && p + c < pd && n < n_state) ? st[(size_t)(p + c) * n_state + n] : 0.f;
            }
        }
    }
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = d_skip[h];
    float decayed = 1.f;                     // the product of the item's decays
    if (!EMIT) {
        float* dec = wts + len;
        for (int t = tid; t < len; t += blockDim.x) {
            const float dtv = softplus_f(to_float(proj[(size_t)(tok0 + t) * proj_stride + dt_col + h]) + bias);
            wts[t] = dtv;
            dec[t] = expf(A * dtv);
        }
        __syncthreads();
        if (tid == 0) {
            float after = 1.f;               // the decays of the tokens behind t
            for (int t = len - 1; t >= 0; --t) {
                wts[t] *= after;
                after *= dec[t];
            }
            dec[0] = after;
        }
        __syncthreads();
        decayed = dec[0];
    }
    if (ahead) {
        for (int q = tid; q < 2 * tt * row; q += blockDim.x) Bs[q] = 0.f;        // entries past n_state stay zero
        ask(0, 0);
        copies_commit();
    }
    for (int t0 = 0; t0 < len; t0 += tt) {
        const int now = min(tt, len - t0);
        if (ahead) {
            const int buf = (t0 / tt) & 1;
            const float dt_now = dt_ahead;
            __syncthreads();                                   // the stage before has been worked through
            if (t0 + tt < len) ask(t0 + tt, buf ^ 1);
            copies_commit();
            copies_wait_all_but_one();
            __syncthreads();                                   // this stage's pieces have landed, for every thread
            for (int q = tid; q < now * pieces; q += blockDim.x) {
                const int ti = q / pieces, k = q - ti * pieces;
                const T* at = raw + ((size_t)(buf * tt + ti) * pieces + k) * ex;
                float* to;
                int first;
                if (k < 2 * pieces_b) {
                    first = (k < pieces_b ? k : k - pieces_b) * ex;
                    to = (k < pieces_b ? Bs : Cs) + ti * row;
                    for (int e = 0; e < ex; ++e) to[((first + e) / NPT) * ROW + (first + e) % NPT] = to_float(at[e]);
                } else {
                    first = (k - 2 * pieces_b) * ex;
                    for (int e = 0; e < ex; ++e) xs[ti * pb + first + e] = p0 + first + e < pd ? to_float(at[e]) : 0.f;
                }
            }
            if (EMIT && tid < now) {
                const float dtv = softplus_f(dt_now + bias);
                dts[tid] = dtv;
                das[tid] = expf(A * dtv);
            }
            __syncthreads();
        } else {
        __syncthreads();
#pragma unroll 4
        for (int ti = 0; ti < now; ++ti) {
            const T* src = xbc + (size_t)(tok0 + t0 + ti) * channels;
            for (int n = tid; n < padded; n += blockDim.x) {
                const int at = ti * row + (n / NPT) * ROW + (n % NPT);
                Bs[at] = n < n_state ? to_float(src[bcol + n]) : 0.f;
                Cs[at] = n < n_state ? to_float(src[ccol + n]) : 0.f;
            }
            for (int q = tid; q < pb; q += blockDim.x)
                xs[ti * pb + q] = p0 + q < pd ? to_float(src[h * pd + p0 + q]) : 0.f;
        }
        if (EMIT && tid < now) {
            const float dtv = softplus_f(to_float(proj[(size_t)(tok0 + t0 + tid) * proj_stride + dt_col + h]) + bias);
            dts[tid] = dtv;
            das[tid] = expf(A * dtv);
        }
        __syncthreads();
        }
        for (int ti = 0; ti < now; ++ti) {
            const float da = EMIT ? das[ti] : 1.f, dtv = EMIT ? dts[ti] : wts[t0 + ti];
            const float4* b4 = reinterpret_cast<const float4*>(Bs + ti * row + j * ROW);
            const float4* c4 = reinterpret_cast<const float4*>(Cs + ti * row + j * ROW);
            float xv[PC], coef[PC], acc[PC];
#pragma unroll
            for (int c = 0; c < PC; ++c) {
                xv[c] = xs[ti * pb + pl + c];
                coef[c] = dtv * xv[c];
                acc[c] = 0.f;
            }
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                const float4 bv = b4[q], cv = c4[q];
                const float bb[4] = {bv.x, bv.y, bv.z, bv.w}, cc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int c = 0; c < PC; ++c) {
                        if (EMIT) {
                            S[c][4 * q + e] = fmaf(da, S[c][4 * q + e], coef[c] * bb[e]);
                            acc[c] = fmaf(S[c][4 * q + e], cc[e], acc[c]);
                        } else {
                            S[c][4 * q + e] = fmaf(coef[c], bb[e], S[c][4 * q + e]);
                        }
                    }
                }
            }
            if (EMIT && PC == 4 && ns >= 4) {
                // four sums over ns lanes in 2 + 1 + log2(ns / 4) exchanges: partners swap halves, then quarters, and
                // lane j < 4 ends with the sum of column 2 (j & 1) + (j >> 1)
                const bool odd = j & 1, upper = j & 2;
                float k0 = odd ? acc[PC - 2] : acc[0], k1 = odd ? acc[PC - 1] : acc[1];
                k0 += __shfl_xor_sync(0xffffffffu, odd ? acc[0] : acc[PC - 2], 1);
                k1 += __shfl_xor_sync(0xffffffffu, odd ? acc[1] : acc[PC - 1], 1);
                float k = upper ? k1 : k0;
                k += __shfl_xor_sync(0xffffffffu, upper ? k0 : k1, 2);
#pragma unroll
                for (int o = 4; o < 32; o <<= 1)
                    if (o < ns) k += __shfl_xor_sync(0xffffffffu, k, o);
                const int col = 2 * (j & 1) + ((j >> 1) & 1);
                const float xcol = col == 0 ? xv[0] : (col == 1 ? xv[1] : (col == 2 ? xv[PC - 2] : xv[PC - 1]));
                if (j < 4 && p + col < pd) y[(size_t)(tok0 + t0 + ti) * inner + h * pd + p + col] = fmaf(D, xcol, k);
            } else if (EMIT) {
#pragma unroll
                for (int c = 0; c < PC; ++c) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
                        if (o < ns) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
                    if (j == 0 && p + c < pd) y[(size_t)(tok0 + t0 + ti) * inner + h * pd + p + c] = fmaf(D, xv[c], acc[c]);
                }
            }
        }
    }
    if (mode == 2) return;
#pragma unroll
    for (int c = 0; c < PC; ++c) {
        if (whole_run && p + c < pd) {
            float4* dst4 = reinterpret_cast<float4*>(st + (size_t)(p + c) * n_state + j * NPT);
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) dst4[q] = make_float4(S[c][4 * q], S[c][4 * q + 1], S[c][4 * q + 2], S[c][4 * q + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const int n = j * NPT + i;
                if (p + c < pd && n < n_state) st[(size_t)(p + c) * n_state + n] = S[c][i];
            }
        }
    }
    if (mode == 1 && tid == 0 && blockIdx.z == 0) chunk_decay[(size_t)item * heads + h] = decayed;
}

// grid (ceil(elements / 256), long portions), block 256: one entry of the scan state through the chunks of a portion.
__global__ void ssd_combine_kernel(float* __restrict__ state, size_t state_stride, const int* __restrict__ slots,
                                   float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                   const int* __restrict__ long_req, const int* __restrict__ long_first,
                                   const int* __restrict__ long_count, int heads, int per_head) {
    pdl_enter_small();
    const size_t elements = (size_t)heads * per_head;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elements) return;
    const int k = blockIdx.y, h = (int)(e / per_head);
    float* st = state + (size_t)slots[long_req[k]] * state_stride + e;
    float S = *st;
    const int first = long_first[k], count = long_count[k];
    for (int c = first; c < first + count; ++c) {
        float* cs = chunk_state + (size_t)c * elements + e;
        const float own = *cs;
        *cs = S;
        S = fmaf(chunk_decay[(size_t)c * heads + h], S, own);
    }
    *st = S;
}

// ---------------------------------------------------------------------------- gate, then grouped RMSNorm

// grid (tokens, groups), block 256: v = y * silu(z) over one group of `gsize` columns, normalised by the
// group's own root mean square, times the gain.
__device__ __forceinline__ float4 quad_of(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 quad_of(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void put_quad(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void put_quad(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// `quads`: four columns a thread and turn (sizes and offsets multiples of four, aligned bases; the launcher checks).
// The gated values of the group are kept in shared memory (`stash`), so every input is read once.
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                           const float* __restrict__ gain, T* __restrict__ out, int inner,
                                           int gsize, float eps, int stash, int quads) {
    extern __shared__ __align__(16) float gated[];          // [gsize] when `stash`
    __shared__ float red[33];
    pdl_enter_small();
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * gsize;
    const float* yr = y + t * inner + c0;
    const T* zr = z + t * z_stride + c0;
    float ssq = 0.f;
    if (quads) {
        for (int i = 4 * threadIdx.x; i < gsize; i += 4 * blockDim.x) {
            const float4 yv = quad_of(yr + i), zv = quad_of(zr + i);
            const float4 v = make_float4(yv.x * silu_for<T>(zv.x), yv.y * silu_for<T>(zv.y), yv.z * silu_for<T>(zv.z),
                                         yv.w * silu_for<T>(zv.w));
            if (stash) *reinterpret_cast<float4*>(gated + i) = v;
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
            const float v = yr[i] * silu_for<T>(to_float(zr[i]));
            if (stash) gated[i] = v;
            ssq = fmaf(v, v, ssq);
        }
    }
    const float inv = rsqrtf(block_sum(ssq, red) / (float)gsize + eps);      // (its barriers also publish `gated`)
    T* dst = out + t * inner + c0;
    if (quads) {
        for (int i = 4 * threadIdx.x; i < gsize; i += 4 * blockDim.x) {
            float4 v;
            if (stash) {
                v = *reinterpret_cast<const float4*>(gated + i);
            } else {
                const float4 yv = quad_of(yr + i), zv = quad_of(zr + i);
                v = make_float4(yv.x * silu_for<T>(zv.x), yv.y * silu_for<T>(zv.y), yv.z * silu_for<T>(zv.z), yv.w * silu_for<T>(zv.w));
            }
            const float4 gv = quad_of(gain + c0 + i);
            put_quad(dst + i, make_float4((v.x * inv) * gv.x, (v.y * inv) * gv.y, (v.z * inv) * gv.z, (v.w * inv) * gv.w));
        }
        return;
    }
    for (int i = threadIdx.x; i < gsize; i += blockDim.x) {
        const float v = stash ? gated[i] : yr[i] * silu_for<T>(to_float(zr[i]));
        dst[i] = from_float<T>((v * inv) * gain[c0 + i]);
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_conv_max_taps() { return 8; }

// act: 1 SiLU, 0 none
LILY_API int lily_causal_conv(const void* in, int in_stride, int col0, int channels, int taps, const float* w,
                              const float* bias, float* state, size_t state_stride, size_t state_off, void* out,
                              const int* chunk_req, const int* chunk_start, int chunks, int chunk_len,
                              const int* cu_seqlens, const int* slots, int dtype, int act, cudaStream_t stream) {
    if (chunks == 0 || channels == 0) return 0;
    LILY_REQUIRE(act == 0 || act == 1, "causal_conv: activation %d (0 none, 1 SiLU)", act);
    LILY_REQUIRE(taps >= 1 && taps <= 8, "causal_conv_silu: %d taps (1 to 8)", taps);
    LILY_REQUIRE(chunk_len >= taps - 1 && chunk_len >= 1, "causal_conv_silu: chunks of %d tokens for %d taps", chunk_len, taps);
    LILY_REQUIRE(chunks <= 65535, "causal_conv_silu: %d chunks", chunks);
    dim3 grid((channels + 127) / 128, chunks), block(128);
#define GO(T, K, A)                                                                                                  \
    launch_pdl(causal_conv_silu_kernel<T, K, A>, grid, block, 0, stream, (const T*)in, in_stride, col0, channels, w, bias, \
               state, state_stride, state_off, (T*)out, chunk_req, chunk_start, chunk_len, cu_seqlens, slots)
#define TAPS_CASE(K) case K:                                                                \
        if (dtype == kBF16) { if (act) GO(__nv_bfloat16, K, true); else GO(__nv_bfloat16, K, false); } \
        else { if (act) GO(float, K, true); else GO(float, K, false); }                     \
        break;
    switch (taps) {
        TAPS_CASE(1) TAPS_CASE(2) TAPS_CASE(3) TAPS_CASE(4) TAPS_CASE(5) TAPS_CASE(6) TAPS_CASE(7) TAPS_CASE(8)
    }
#undef TAPS_CASE
#undef GO
    LILY_CHECK_LAUNCH("causal_conv_silu");
    return 0;
}

LILY_API int lily_causal_conv_silu(const void* in, int in_stride, int col0, int channels, int taps, const float* w,
                                   const float* bias, float* state, size_t state_stride, size_t state_off, void* out,
                                   const int* chunk_req, const int* chunk_start, int chunks, int chunk_len,
                                   const int* cu_seqlens, const int* slots, int dtype, cudaStream_t stream) {
    return lily_causal_conv(in, in_stride, col0, channels, taps, w, bias, state, state_stride, state_off, out, chunk_req,
                            chunk_start, chunks, chunk_len, cu_seqlens, slots, dtype, 1, stream);
}

LILY_API int lily_ssd_scan_max_state() { return 512; }

LILY_API int lily_ssd_scan(const void* xbc, int channels, const void* proj, int proj_stride, int dt_col,
                           const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                           size_t state_stride, float* y, const int* cu_seqlens, const int* slots, int requests,
                           int heads, int pd, int n_state, int groups, int dtype, const int* item_req,
                           const int* item_start, const int* item_len, int mode, float* chunk_state, float* chunk_decay,
                           int max_item_len, cudaStream_t stream) {
    if (requests == 0) return 0;
    LILY_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || (chunk_state && chunk_decay && item_req && item_start && item_len)),
                 "ssd_scan: mode %d needs item lists and a workspace", mode);
    LILY_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "ssd_scan: %d heads over %d groups", heads, groups);
    LILY_REQUIRE(n_state >= 1 && n_state <= 512 && pd >= 1, "ssd_scan: state %d (1 to 512), head size %d", n_state, pd);
    LILY_REQUIRE(requests <= 65535, "ssd_scan: %d requests", requests);
    // ns lanes share pc value columns, each lane with npt = 4, 8 or 16 entries of a column's state
    int npt = n_state <= 32 ? 4 : (n_state <= 128 ? 8 : 16);
    int ns = 1;
    while (ns * npt < n_state) ns <<= 1;
    if (ns > 32) { ns = 32; npt = 16; }
    if (npt == 8 && ns >= 16) { npt = 16; ns >>= 1; }    // fewer lanes to add up over
    int pc = pd % 4 == 0 && pd >= 16 ? 4 : (pd % 2 == 0 && pd >= 8 ? 2 : 1);
    const int lanes_cols = 32 / ns > 0 ? 32 / ns : 1;    // column groups that fill a warp
    int groups_needed = (pd + pc - 1) / pc;              // column groups of a head
    int cg = groups_needed;                              // column groups a block: the whole head when it fits 256 threads
    while (cg * ns > 256) cg = (cg + 1) / 2;
    cg = (cg + lanes_cols - 1) / lanes_cols * lanes_cols;    // whole warps
    const int pb = cg * pc;
    const int row = ns * (npt + 4);                      // a token's B (or C) in shared memory, padded lane by lane
    int tt = 16;
    while (tt > 1 && (size_t)tt * (2 * row + pb + 2) * sizeof(float) > 36 * 1024) tt >>= 1;
    // (a block is whole warps, so it has at least as many threads as a stage has tokens)
    LILY_REQUIRE(mode != 1 || (max_item_len >= 1 && max_item_len <= 1024), "ssd_scan: chunks of up to %d tokens (1 to 1024)", max_item_len);
    const int max_len = mode == 1 ? max_item_len : 0;
    // rows are copied ahead where every piece of 16 bytes is whole and aligned (and the items are longer than a stage)
    const size_t item = dtype == kBF16 ? 2 : 4;
    const int ahead = ((uintptr_t)xbc % 16 == 0 && (channels * item) % 16 == 0 && (heads * pd * item) % 16 == 0 &&
                       (n_state * item) % 16 == 0 && (pd * item) % 16 == 0 && (pb * item) % 16 == 0 && tt % 2 == 0 && (item_len != nullptr)) ? 1 : 0;
    const int wide = (n_state % 4 == 0 && state_stride % 4 == 0 && (uintptr_t)state % 16 == 0 && (uintptr_t)chunk_state % 16 == 0) ? 1 : 0;
    const size_t raw_bytes = ahead ? 2 * (size_t)tt * (2 * n_state + pb) * item : 0;
    const size_t smem = ((size_t)tt * (2 * row + pb + 2) + 2 * (size_t)max_len) * sizeof(float) + raw_bytes;
    LILY_REQUIRE(smem <= 200 * 1024, "ssd_scan: %zu bytes of shared memory", smem);
    dim3 grid(heads, requests, (pd + pb - 1) / pb), block(cg * ns);
#define GO(T, N, C, E)                                                                                                 \
    do {                                                                                                               \
        auto kern = ssd_scan_kernel<T, N, C, E>;                                                                       \
        static size_t granted = 48 * 1024;      /* raised once per kernel, never while a graph is captured */           \
        if (smem > granted) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (e != cudaSuccess) { set_error("ssd_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; } \
            granted = smem;                                                                                            \
        }                                                                                                              \
        launch_pdl(kern, grid, block, smem, stream, (const T*)xbc, channels, (const T*)proj, proj_stride,              \
                   dt_col, dt_bias, a_log, d_skip, state, state_stride, y, cu_seqlens, slots, heads, pd, n_state, groups, ns, \
                   pb, tt, item_req, item_start, item_len, mode, chunk_state, chunk_decay, ahead, max_len, wide);      \
    } while (0)
#define GO_E(T, N, C) do { if (mode == 1) GO(T, N, C, false); else GO(T, N, C, true); } while (0)
#define GO_C(T, N) do { if (pc == 4) GO_E(T, N, 4); else if (pc == 2) GO_E(T, N, 2); else GO_E(T, N, 1); } while (0)
    if (dtype == kBF16) {
        if (npt == 4) GO_C(__nv_bfloat16, 4); else if (npt == 8) GO_C(__nv_bfloat16, 8); else GO_C(__nv_bfloat16, 16);
    } else {
        if (npt == 4) GO_C(float, 4); else if (npt == 8) GO_C(float, 8); else GO_C(float, 16);
    }
#undef GO_C
#undef GO_E
#undef GO
    LILY_CHECK_LAUNCH("ssd_scan");
    return 0;
}

LILY_API int lily_ssd_combine(float* state, size_t state_stride, const int* slots, float* chunk_state,
                              const float* chunk_decay, const int* long_req, const int* long_first,
                              const int* long_count, int portions, int heads, int per_head, cudaStream_t stream) {
    if (portions == 0) return 0;
    LILY_REQUIRE(portions <= 65535, "ssd_combine: %d portions", portions);
    const size_t elements = (size_t)heads * per_head;
    launch_pdl(ssd_combine_kernel, dim3((unsigned)((elements + 255) / 256), portions), dim3(256), 0, stream, state,
               state_stride, slots, chunk_state, chunk_decay, long_req, long_first, long_count, heads, per_head);
    LILY_CHECK_LAUNCH("ssd_combine");
    return 0;
}

LILY_API int lily_gated_group_rmsnorm(const float* y, const void* z, int z_stride, const float* gain, void* out,
                                      int tokens, int inner, int groups, float eps, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(groups >= 1 && inner % groups == 0, "gated_group_rmsnorm: %d columns in %d groups", inner, groups);
    LILY_REQUIRE(groups <= 65535, "gated_group_rmsnorm: %d groups", groups);
    dim3 grid(tokens, groups), block(256);
    const int gsize = inner / groups;
    const int stash = gsize <= 10240;              // 40 KB of shared memory hold the group's gated values
    const size_t smem = stash ? (size_t)gsize * sizeof(float) : 0;
    const size_t item = dtype == kBF16 ? 2 : 4;
    const int quads = gsize % 4 == 0 && inner % 4 == 0 && z_stride % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)gain % 16 == 0 &&
                      (uintptr_t)z % (4 * item) == 0 && (uintptr_t)out % (4 * item) == 0;
    if (dtype == kBF16)
        launch_pdl(gated_group_rmsnorm_kernel<__nv_bfloat16>, grid, block, smem, stream, y, (const __nv_bfloat16*)z, z_stride,
                   gain, (__nv_bfloat16*)out, inner, gsize, eps, stash, quads);
    else
        launch_pdl(gated_group_rmsnorm_kernel<float>, grid, block, smem, stream, y, (const float*)z, z_stride, gain,
                   (float*)out, inner, gsize, eps, stash, quads);
    LILY_CHECK_LAUNCH("gated_group_rmsnorm");
    return 0;
}
