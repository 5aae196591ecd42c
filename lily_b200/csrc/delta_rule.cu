// The recurrence of the gated delta-rule mixer, with its state in the request's slot.
//
// Per value head h (query/key head g = h / (heads / kv_heads)), with S a d x dv matrix that is zero when the request
// starts, a_t = exp(-exp(A_log_h) softplus(alpha_t + dt_bias_h)) and b_t = sigmoid(beta_t):
//
//     S <- a_t S;   u = b_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// with q_t and k_t made unit vectors per head first (x / sqrt(sum x^2 + eps); q also times `q_scale`).  The columns of
// S never meet: column j needs (S^T k)_j and (S^T q)_j only, so a block owns a few columns of one head of one request
// and walks the request's new tokens in order.  DL lanes share a column and hold R of its rows each; a token costs one
// pass over the lane's rows for three sums at once, (S^T k)_j, (S^T q)_j and k . q, taken over the old S:
//
//     u_j = b (v_j - a (S^T k)_j),    o_j = a (S^T q)_j + (k . q) u_j,    S_ij <- a S_ij + k_i u_j
//
// then one exchange over the DL lanes and one pass that updates the rows.  The tokens come in tiles of DELTA_TOKENS
// through shared memory; the next tile's inputs are loaded into registers while the current one is worked on.  Decay, gate, unit vectors, state and sums are
// float32 whatever the activation dtype.  State row of a slot: [heads][dv][d] (d fastest) at the row's start.
#include "common.cuh"

namespace lily {

constexpr int DL = 16;                 // lanes that share a column
constexpr int DELTA_TOKENS = 16;       // tokens staged at a time
constexpr int DELTA_THREADS = 128;
constexpr int DELTA_COLS = DELTA_THREADS / DL;

struct DeltaArgs {
    const void* qkv;          // [tokens, qkv_stride]: convolved and activated q (kv_heads x d), k (kv_heads x d), v (heads x dv)
    int qkv_stride, q_col, k_col, v_col;
    const void* proj;         // [tokens, proj_stride]: the projection that holds beta and alpha (heads columns each)
    int proj_stride, b_col, a_col;
    const float* a_log;       // [heads]
    const float* dt_bias;     // [heads]
    float* state;             // [slots, state_stride]
    size_t state_stride;
    float* y;                 // [tokens, heads * dv]
    const int* cu_seqlens;
    const int* slots;
    int heads, kv_heads, d, dv;
    float unit_eps, q_scale;
};

// Sum over the DL lanes of a column.  The mask names those lanes only: the two groups of a warp may stand in
// different turns of a loop (a tile whose tokens do not divide among the groups).
__device__ __forceinline__ float sum_over_lanes(float v) {
    const unsigned mask = (DL == 32 ? 0xffffffffu : ((1u << DL) - 1u)) << ((threadIdx.x & 31) / DL * DL);
#pragma unroll
    for (int o = DL / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
    return v;
}

// grid (requests, heads, ceil(dv / DELTA_COLS)), block DELTA_THREADS; d <= DL * R
// AHEAD: a tile's inputs are loaded one tile ahead (portions of prompts); without it they are loaded when their turn
// comes, which keeps fewer registers alive and more blocks on a SM (steps in which every request brings one token).
template <typename T, int R, bool AHEAD>
__global__ void __launch_bounds__(DELTA_THREADS) delta_rule_kernel(const DeltaArgs a) {
    constexpr int DP = DL * R;
    __shared__ float qs[DELTA_TOKENS][DP], ks[DELTA_TOKENS][DP];
    __shared__ float vs[DELTA_TOKENS][DELTA_COLS], os[DELTA_TOKENS][DELTA_COLS], as[DELTA_TOKENS], bs[DELTA_TOKENS];
    pdl_enter_small();
    const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * DELTA_COLS;
    const int l = threadIdx.x % DL, cg = threadIdx.x / DL;
    const int j = col0 + cg, d = a.d, dv = a.dv;
    const bool col_ok = j < dv;
    const int kvh = head / (a.heads / a.kv_heads);
    const int tok0 = a.cu_seqlens[req], len = a.cu_seqlens[req + 1] - tok0;
    if (len <= 0) return;
    float* st = a.state + (size_t)a.slots[req] * a.state_stride + ((size_t)head * dv + (col_ok ? j : 0)) * d;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = l + DL * r;
        S[r] = col_ok && i < d ? st[i] : 0.f;
    }
    const float rate = expf(a.a_log[head]), dt_bias = a.dt_bias[head];
    const T* qkv = (const T*)a.qkv;
    const T* proj = (const T*)a.proj;
    const int out_stride = a.heads * dv;

    // A tile's inputs are asked for into registers one tile ahead, so that they travel while the tile before is worked on.
    constexpr int PER = DELTA_TOKENS * DP / DELTA_THREADS;          // q (and k) entries a thread stages: 2 R
    float rq[PER], rk[PER], rv = 0.f, rb = 0.f, ra = 0.f;
    auto fetch = [&](int t0) {
        const int n = min(DELTA_TOKENS, len - t0);
#pragma unroll
        for (int it = 0; it < PER; ++it) {
            const int e = it * DELTA_THREADS + threadIdx.x, t = e / DP, i = e % DP;
            const bool ok = t < n && i < d;
            const T* row = qkv + (size_t)(tok0 + t0 + (ok ? t : 0)) * a.qkv_stride + (size_t)kvh * d + (ok ? i : 0);
            rq[it] = ok ? to_float(row[a.q_col]) : 0.f;
            rk[it] = ok ? to_float(row[a.k_col]) : 0.f;
        }
        {
            const int t = threadIdx.x / DELTA_COLS, c = threadIdx.x % DELTA_COLS;       // DELTA_TOKENS * DELTA_COLS == DELTA_THREADS
            rv = t < n && col0 + c < dv ? to_float(qkv[(size_t)(tok0 + t0 + t) * a.qkv_stride + a.v_col + (size_t)head * dv + col0 + c]) : 0.f;
        }
        if (threadIdx.x < n) {
            const T* row = proj + (size_t)(tok0 + t0 + threadIdx.x) * a.proj_stride + head;
            rb = to_float(row[a.b_col]);
            ra = to_float(row[a.a_col]);
        }
    };
    static_assert(DELTA_TOKENS * DELTA_COLS == DELTA_THREADS, "a thread stages one value of a tile");
    if (AHEAD) fetch(0);

    for (int t0 = 0; t0 < len; t0 += DELTA_TOKENS) {
        const int n = min(DELTA_TOKENS, len - t0);
        if (!AHEAD) fetch(t0);
        __syncthreads();
#pragma unroll
        for (int it = 0; it < PER; ++it) {
            const int e = it * DELTA_THREADS + threadIdx.x;
            qs[e / DP][e % DP] = rq[it];
            ks[e / DP][e % DP] = rk[it];
        }
        vs[threadIdx.x / DELTA_COLS][threadIdx.x % DELTA_COLS] = rv;
        if (threadIdx.x < n) {
            const float alpha = ra + dt_bias;
            bs[threadIdx.x] = 1.f / (1.f + expf(-rb));
            as[threadIdx.x] = expf(-rate * (alpha > 20.f ? alpha : log1pf(expf(alpha))));
        }
        __syncthreads();
        if (AHEAD && t0 + DELTA_TOKENS < len) fetch(t0 + DELTA_TOKENS);
        // q and k of the head as unit vectors: a group of lanes a token
        for (int t = cg; t < n; t += DELTA_COLS) {
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float x = qs[t][l + DL * r], z = ks[t][l + DL * r];
                sq = fmaf(x, x, sq);
                sk = fmaf(z, z, sk);
            }
            const float fq = a.q_scale / sqrtf(sum_over_lanes(sq) + a.unit_eps), fk = 1.f / sqrtf(sum_over_lanes(sk) + a.unit_eps);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                qs[t][l + DL * r] *= fq;
                ks[t][l + DL * r] *= fk;
            }
        }
        __syncthreads();
#pragma unroll 2
        for (int t = 0; t < n; ++t) {
            float sk = 0.f, sq = 0.f, kq = 0.f, kk[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                kk[r] = ks[t][l + DL * r];
                const float qq = qs[t][l + DL * r];
                sk = fmaf(S[r], kk[r], sk);
                sq = fmaf(S[r], qq, sq);
                kq = fmaf(kk[r], qq, kq);
            }
            sk = sum_over_lanes(sk);
            sq = sum_over_lanes(sq);
            kq = sum_over_lanes(kq);
            const float decay = as[t];
            const float u = bs[t] * (vs[t][cg] - decay * sk);
#pragma unroll
            for (int r = 0; r < R; ++r) S[r] = fmaf(kk[r], u, decay * S[r]);
            if (l == 0) os[t][cg] = fmaf(decay, sq, kq * u);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * DELTA_COLS; e += DELTA_THREADS) {
            const int t = e / DELTA_COLS, c = e % DELTA_COLS;
            if (col0 + c < dv) a.y[(size_t)(tok0 + t0 + t) * out_stride + (size_t)head * dv + col0 + c] = os[t][c];
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = l + DL * r;
            if (i < d) st[i] = S[r];
        }
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_delta_rule_max_head_dim() { return DL * 16; }

LILY_API int lily_delta_rule(const void* qkv, int qkv_stride, int q_col, int k_col, int v_col, const void* proj, int proj_stride,
                             int b_col, int a_col, const float* a_log, const float* dt_bias, float* state, size_t state_stride,
                             float* y, const int* cu_seqlens, const int* slots, int requests, int tokens, int heads, int kv_heads,
                             int d, int dv, float unit_eps, float q_scale, int dtype, cudaStream_t stream) {
    if (requests == 0) return 0;
    LILY_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "delta_rule: %d heads over %d query/key heads", heads, kv_heads);
    LILY_REQUIRE(d > 0 && d <= DL * 16 && dv > 0, "delta_rule: head sizes %d / %d (keys up to %d)", d, dv, DL * 16);
    LILY_REQUIRE((size_t)heads * d * dv <= state_stride, "delta_rule: the state row is shorter than %d matrices of %d x %d", heads, d, dv);
    LILY_REQUIRE(heads <= 65535 && (dv + DELTA_COLS - 1) / DELTA_COLS <= 65535, "delta_rule: grid too large");
    DeltaArgs a{};
    a.qkv = qkv; a.qkv_stride = qkv_stride; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col;
    a.proj = proj; a.proj_stride = proj_stride; a.b_col = b_col; a.a_col = a_col; a.a_log = a_log; a.dt_bias = dt_bias;
    a.state = state; a.state_stride = state_stride; a.y = y; a.cu_seqlens = cu_seqlens; a.slots = slots;
    a.heads = heads; a.kv_heads = kv_heads; a.d = d; a.dv = dv; a.unit_eps = unit_eps; a.q_scale = q_scale;
    dim3 grid(requests, heads, (dv + DELTA_COLS - 1) / DELTA_COLS), block(DELTA_THREADS);
    const int rows = (d + DL - 1) / DL;
    const bool ahead = tokens > requests;               // some request brings more than one token
#define GO(R)                                                                                                         \
    do {                                                                                                              \
        if (dtype == kBF16) {                                                                                         \
            if (ahead) launch_pdl(delta_rule_kernel<__nv_bfloat16, R, true>, grid, block, 0, stream, a);              \
            else launch_pdl(delta_rule_kernel<__nv_bfloat16, R, false>, grid, block, 0, stream, a);                   \
        } else {                                                                                                      \
            if (ahead) launch_pdl(delta_rule_kernel<float, R, true>, grid, block, 0, stream, a);                      \
            else launch_pdl(delta_rule_kernel<float, R, false>, grid, block, 0, stream, a);                           \
        }                                                                                                             \
    } while (0)
    if (rows <= 1) GO(1);
    else if (rows <= 2) GO(2);
    else if (rows <= 4) GO(4);
    else if (rows <= 8) GO(8);
    else GO(16);
#undef GO
    LILY_CHECK_LAUNCH("delta_rule");
    return 0;
}
