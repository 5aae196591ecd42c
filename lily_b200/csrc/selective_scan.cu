// The selective scan of the first Mamba mixer: a state vector per channel, with its state in the request's slot.
//
// Per channel c and state entry n, with dt_t[c] = softplus(step_t[c]) (the step projection's result with its bias) and
// A[c][n] = -exp(A_log[c][n]) formed once when the weights are loaded:
//
//     S[c][n] <- exp(dt_t[c] A[c][n]) S[c][n] + dt_t[c] x_t[c] B_t[n]
//     y_t[c]  =  sum_n S[c][n] C_t[n] + D[c] x_t[c],        out_t[c] = y_t[c] * silu(z_t[c])
//
// SL lanes share a channel and hold NR state entries each; a block owns SCAN_CHANNELS channels of one request and
// walks the request's new tokens in order; a token's B and C are staged once for all of the block's channels, and the
// next tile's inputs are loaded into registers while the current one is worked on.  The
// step size, the decay, the state and the sums are float32 whatever the activation dtype.  State row of a slot:
// [inner][state] (state fastest) at the row's start.
//
// A long portion is cut into chunks that run side by side (the recurrence is diagonal): a first pass runs every chunk
// from a zero state and leaves its end state L_c and the sum of its steps in a workspace; `selective_combine` walks a
// request's chunks in order, S <- exp(A sum_c dt) S + L_c, leaves in the workspace the state each chunk starts from
// and writes the slot; a second pass runs every chunk from there and writes the outputs.
#include "common.cuh"

namespace lily {

constexpr int SL = 8;                   // lanes that share a channel
constexpr int SCAN_TOKENS = 16;         // tokens staged at a time
constexpr int SCAN_THREADS = 128;
constexpr int SCAN_CHANNELS = SCAN_THREADS / SL;

struct SelectiveArgs {
    const void* x;            // [tokens, inner]: the convolved and activated inputs
    const void* low;          // [tokens, low_stride]: B at b_col, C at c_col (n_state columns each)
    int low_stride, b_col, c_col;
    const float* step;        // [tokens, inner]: W_dt . + bias, before softplus
    const void* z;            // [tokens, z_stride]: the gate's columns start at z_col
    int z_stride, z_col;
    const float* A;           // [inner, n_state]
    const float* D;           // [inner]
    float* state;             // [slots, state_stride]
    size_t state_stride;
    void* out;                // [tokens, inner]
    const int* cu_seqlens;
    const int* slots;
    int inner, n_state;
    // the work of block x: request work_req[x] (null: request x), its tokens [work_start[x], + work_len[x]) (null: all)
    const int* work_req;
    const int* work_start;
    const int* work_len;
    int mode;                 // 0: from and to the slot; 1: chunk x from zero, end state and sum of steps to the workspace,
                              // no outputs; 2: chunk x from the workspace's state, outputs, no state written
    float* ws_state;          // [chunks][inner][n_state]
    float* ws_steps;          // [chunks][inner]
};

// grid (requests, ceil(inner / SCAN_CHANNELS)), block SCAN_THREADS; n_state <= SL * NR
// AHEAD: a tile's inputs are loaded one tile ahead (portions of prompts); without it they are loaded when their turn
// comes, which keeps fewer registers alive (steps in which every request brings one token).
template <typename T, int NR, bool AHEAD>
__global__ void __launch_bounds__(SCAN_THREADS) selective_scan_kernel(const SelectiveArgs a) {
    constexpr int SP = SL * NR;
    __shared__ float Bs[SCAN_TOKENS][SP], Cs[SCAN_TOKENS][SP];
    __shared__ float dts[SCAN_TOKENS][SCAN_CHANNELS], xs[SCAN_TOKENS][SCAN_CHANNELS], zs[SCAN_TOKENS][SCAN_CHANNELS],
        ys[SCAN_TOKENS][SCAN_CHANNELS];
    pdl_enter_small();
    const int req = a.work_req ? a.work_req[blockIdx.x] : blockIdx.x, ch0 = blockIdx.y * SCAN_CHANNELS;
    const int l = threadIdx.x % SL, cg = threadIdx.x / SL;
    const int ch = ch0 + cg, inner = a.inner, ns = a.n_state;
    const bool ch_ok = ch < inner;
    const int first = a.work_start ? a.work_start[blockIdx.x] : 0;
    const int tok0 = a.cu_seqlens[req] + first, len = a.work_len ? a.work_len[blockIdx.x] : a.cu_seqlens[req + 1] - tok0;
    if (len <= 0) return;
    const int mode = a.mode;
    float* st = mode == 0 ? a.state + (size_t)a.slots[req] * a.state_stride + (size_t)(ch_ok ? ch : 0) * ns
                          : a.ws_state + ((size_t)blockIdx.x * inner + (ch_ok ? ch : 0)) * ns;
    float S[NR], A[NR], steps = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int n = l + SL * r;
        const bool ok = ch_ok && n < ns;
        S[r] = ok && mode != 1 ? st[n] : 0.f;
        A[r] = ok ? a.A[(size_t)ch * ns + n] * 1.4426950408889634f : 0.f;      // in units of log2: the decay is one exp2 an entry
    }
    const float skip = ch_ok ? a.D[ch] : 0.f;
    const T* x = (const T*)a.x;
    const T* low = (const T*)a.low;
    const T* z = (const T*)a.z;
    T* out = (T*)a.out;

    // A tile's inputs are asked for into registers one tile ahead, so that they travel while the tile before is worked on.
    constexpr int PER = SCAN_TOKENS * SP / SCAN_THREADS;                    // B (and C) entries a thread stages: NR
    constexpr int CPER = SCAN_TOKENS * SCAN_CHANNELS / SCAN_THREADS;        // step, x and z entries a thread stages: 2
    float rB[PER], rC[PER], rs[CPER], rx[CPER], rz[CPER];
    auto fetch = [&](int t0) {
        const int n = min(SCAN_TOKENS, len - t0);
#pragma unroll
        for (int it = 0; it < PER; ++it) {
            const int e = it * SCAN_THREADS + threadIdx.x, t = e / SP, i = e % SP;
            const bool ok = t < n && i < ns;
            const T* row = low + (size_t)(tok0 + t0 + (ok ? t : 0)) * a.low_stride + (ok ? i : 0);
            rB[it] = ok ? to_float(row[a.b_col]) : 0.f;
            rC[it] = ok ? to_float(row[a.c_col]) : 0.f;
        }
#pragma unroll
        for (int it = 0; it < CPER; ++it) {
            const int e = it * SCAN_THREADS + threadIdx.x, t = e / SCAN_CHANNELS, c = e % SCAN_CHANNELS;
            const bool ok = t < n && ch0 + c < inner;
            const size_t tok = tok0 + t0 + (ok ? t : 0);
            rs[it] = ok ? a.step[tok * inner + ch0 + c] : 0.f;
            rx[it] = ok ? to_float(x[tok * inner + ch0 + c]) : 0.f;
            rz[it] = ok ? to_float(z[tok * a.z_stride + a.z_col + ch0 + c]) : 0.f;
        }
    };
    if (AHEAD) fetch(0);

    for (int t0 = 0; t0 < len; t0 += SCAN_TOKENS) {
        const int n = min(SCAN_TOKENS, len - t0);
        if (!AHEAD) fetch(t0);
        __syncthreads();
#pragma unroll
        for (int it = 0; it < PER; ++it) {
            const int e = it * SCAN_THREADS + threadIdx.x;
            Bs[e / SP][e % SP] = rB[it];
            Cs[e / SP][e % SP] = rC[it];
        }
#pragma unroll
        for (int it = 0; it < CPER; ++it) {
            const int e = it * SCAN_THREADS + threadIdx.x, t = e / SCAN_CHANNELS, c = e % SCAN_CHANNELS;
            dts[t][c] = rs[it] > 20.f ? rs[it] : log1pf(expf(rs[it]));
            xs[t][c] = rx[it];
            zs[t][c] = rz[it];
        }
        __syncthreads();
        if (AHEAD && t0 + SCAN_TOKENS < len) fetch(t0 + SCAN_TOKENS);
#pragma unroll 4
        for (int t = 0; t < n; ++t) {                 // the exponentials and the lane sums of neighbouring tokens overlap
            const float dt = dts[t][cg], xv = xs[t][cg], dx = dt * xv;
            steps += dt;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                S[r] = fmaf(exp2f(dt * A[r]), S[r], dx * Bs[t][l + SL * r]);
                acc = fmaf(S[r], Cs[t][l + SL * r], acc);
            }
#pragma unroll
            for (int o = SL / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);      // every thread of the block is in this turn
            if (l == 0) {
                const float zv = zs[t][cg];
                ys[t][cg] = fmaf(skip, xv, acc) * (zv / (1.f + expf(-zv)));
            }
        }
        __syncthreads();
        if (mode != 1)
            for (int e = threadIdx.x; e < n * SCAN_CHANNELS; e += SCAN_THREADS) {
                const int t = e / SCAN_CHANNELS, c = e % SCAN_CHANNELS;
                if (ch0 + c < inner) out[(size_t)(tok0 + t0 + t) * inner + ch0 + c] = from_float<T>(ys[t][c]);
            }
    }
    if (ch_ok && mode != 2) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int n = l + SL * r;
            if (n < ns) st[n] = S[r];
        }
        if (mode == 1 && l == 0) a.ws_steps[(size_t)blockIdx.x * inner + ch] = steps;
    }
}

// grid (long requests, ceil(inner * n_state / 256)): a thread an entry of a request's state, its chunks in order.
__global__ void selective_combine_kernel(float* __restrict__ state, size_t state_stride, const int* __restrict__ slots,
                                         const int* __restrict__ long_req, const int* __restrict__ long_first,
                                         const int* __restrict__ long_count, const float* __restrict__ A,
                                         float* __restrict__ ws_state, const float* __restrict__ ws_steps, int inner, int ns) {
    pdl_enter_small();
    const int e = blockIdx.y * blockDim.x + threadIdx.x;
    if (e >= inner * ns) return;
    const int ch = e / ns;
    float* slot = state + (size_t)slots[long_req[blockIdx.x]] * state_stride + e;
    const float rate = A[e];
    float S = *slot;
    const int c0 = long_first[blockIdx.x], c1 = c0 + long_count[blockIdx.x];
    for (int c = c0; c < c1; ++c) {
        float* at = ws_state + (size_t)c * inner * ns + e;
        const float own = *at;
        *at = S;                                                     // what chunk c starts from
        S = fmaf(expf(rate * ws_steps[(size_t)c * inner + ch]), S, own);
    }
    *slot = S;
}

}  // namespace lily

using namespace lily;

LILY_API int lily_selective_scan_max_state() { return SL * 32; }

LILY_API int lily_selective_scan(const void* x, const void* low, int low_stride, int b_col, int c_col, const float* step,
                                 const void* z, int z_stride, int z_col, const float* A, const float* D, float* state,
                                 size_t state_stride, void* out, const int* cu_seqlens, const int* slots, int requests, int tokens,
                                 int inner, int n_state, int dtype, const int* work_req, const int* work_start,
                                 const int* work_len, int mode, float* ws_state, float* ws_steps, cudaStream_t stream) {
    // `requests`: the blocks along x (requests, or the entries of the work lists)
    if (requests == 0) return 0;
    LILY_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || (work_req && work_start && work_len && ws_state && ws_steps)),
                 "selective_scan: chunks come with their lists and a workspace");
    LILY_REQUIRE(inner > 0 && n_state > 0 && n_state <= SL * 32, "selective_scan: %d channels of %d state entries (up to %d)", inner, n_state, SL * 32);
    LILY_REQUIRE((size_t)inner * n_state <= state_stride, "selective_scan: the state row is shorter than %d x %d", inner, n_state);
    LILY_REQUIRE((inner + SCAN_CHANNELS - 1) / SCAN_CHANNELS <= 65535, "selective_scan: %d channels", inner);
    SelectiveArgs a{};
    a.x = x; a.low = low; a.low_stride = low_stride; a.b_col = b_col; a.c_col = c_col; a.step = step;
    a.z = z; a.z_stride = z_stride; a.z_col = z_col; a.A = A; a.D = D; a.state = state; a.state_stride = state_stride;
    a.out = out; a.cu_seqlens = cu_seqlens; a.slots = slots; a.inner = inner; a.n_state = n_state;
    a.work_req = work_req; a.work_start = work_start; a.work_len = work_len; a.mode = mode; a.ws_state = ws_state; a.ws_steps = ws_steps;
    dim3 grid(requests, (inner + SCAN_CHANNELS - 1) / SCAN_CHANNELS), block(SCAN_THREADS);
    const int per = (n_state + SL - 1) / SL;
    const bool ahead = mode != 0 || tokens > requests;  // some request brings more than one token
#define GO(NR)                                                                                                            \
    do {                                                                                                                  \
        if (dtype == kBF16) {                                                                                             \
            if (ahead) launch_pdl(selective_scan_kernel<__nv_bfloat16, NR, true>, grid, block, 0, stream, a);             \
            else launch_pdl(selective_scan_kernel<__nv_bfloat16, NR, false>, grid, block, 0, stream, a);                  \
        } else {                                                                                                          \
            if (ahead) launch_pdl(selective_scan_kernel<float, NR, true>, grid, block, 0, stream, a);                     \
            else launch_pdl(selective_scan_kernel<float, NR, false>, grid, block, 0, stream, a);                          \
        }                                                                                                                 \
    } while (0)
    if (per <= 1) GO(1);
    else if (per <= 2) GO(2);
    else if (per <= 4) GO(4);
    else if (per <= 8) GO(8);
    else if (per <= 16) GO(16);
    else GO(32);
#undef GO
    LILY_CHECK_LAUNCH("selective_scan");
    return 0;
}

LILY_API int lily_selective_combine(float* state, size_t state_stride, const int* slots, const int* long_req, const int* long_first,
                                    const int* long_count, int num_long, const float* A, float* ws_state, const float* ws_steps,
                                    int inner, int n_state, cudaStream_t stream) {
    if (num_long == 0) return 0;
    const int entries = inner * n_state;
    launch_pdl(selective_combine_kernel, dim3(num_long, (entries + 255) / 256), dim3(256), 0, stream, state, state_stride, slots,
               long_req, long_first, long_count, A, ws_state, ws_steps, inner, n_state);
    LILY_CHECK_LAUNCH("selective_combine");
    return 0;
}
