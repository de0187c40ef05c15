// Recurrent mixers whose per-request state is a matrix per head: the gated delta rule and the matrix
// memory of xLSTM (mLSTM).  The state is float32, lives in the request's state slot and is carried from
// step to step; a step may bring any number of tokens of any number of requests (a prompt's portion
// beside single decoded tokens), each request walking its own tokens in order from its own state.
//
// Both rules update every COLUMN of the state matrix S [d, e] independently of the other columns:
//
//   gated delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                      column j:  r = S_j . k;  u_j = beta (v_j - g r);  S_j <- g S_j + u_j k;
//                                 o_j = g (S_j . q) + u_j (k . q)          (S_j . q taken before the update)
//   matrix memory      m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m')
//                      S <- a S + b k v^T;  n <- a n + b k;  o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//                      column j:  S_j <- a S_j + (b v_j) k;  o_j = (S_j . q) / den
//
// so the work is spread over (request, head, block of columns): a block owns SANDY_MATRIX_STATE_COLS
// columns, a warp four of them, a lane the rows lane, lane + 32, ... of each; the dot products are warp
// reductions.  The tokens' inputs are staged through shared memory a chunk at a time, the next chunk's
// loads in flight while the current one is computed.  The state is stored transposed, [head][column][row],
// so that a lane's rows of a column are consecutive lanes' consecutive floats.  The matrix memory's n and m
// are advanced by every column block for itself and therefore kept once per column block.  That is the token-by-token
// form, which decode steps and short portions take; requests that bring many tokens go through the chunked kernels
// further down, which treat 32 tokens at once.
//
// Everything here is float32 arithmetic whatever the engine's compute type: gates, decays, exponentials,
// unit norms, the state.  Inputs that come from a projection are read in the projection's type.
#include "common.cuh"
#include "matrix_state.h"

namespace {

constexpr int WARPS = 4;
constexpr int CPW = 4;                                   // columns per warp
constexpr int COLS = SANDY_MATRIX_STATE_COLS;            // columns per block
static_assert(COLS == WARPS * CPW, "a block's columns are its warps' columns");
constexpr int THREADS = WARPS * 32;
constexpr int CHUNK = 8;                                 // tokens staged at a time
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ---- gated delta rule: what comes before the recurrence ---------------------------------------------------
// Per token: the short causal convolution of the q, k and v channels (taps from the step's earlier tokens
// or, before the step's start, from the tail kept in the state), silu, unit vectors per q/k head (q also
// times q_scale), and the two gates.  One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ taps, int n_taps,
                     const float* __restrict__ gates, int ld_gates, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const float* __restrict__ state, long long state_stride,
                     long long tail_off, const int* __restrict__ token_seq, const int* __restrict__ q_start,
                     const int* __restrict__ seq_slots, float* __restrict__ qkv, int ld_qkv, float* __restrict__ bg,
                     int n_heads, int n_qk_heads, int qk_dim, int v_dim, float q_scale) {
    extern __shared__ float act[];                    // [channels]
    const int t = blockIdx.x;
    const int qk = n_qk_heads * qk_dim;
    const int channels = 2 * qk + n_heads * v_dim;
    const int s = token_seq[t];
    const int i_in_step = t - q_start[s];
    const float* tail = state + (long long)seq_slots[s] * state_stride + tail_off;      // [n_taps - 1][channels]
    pdl_wait();
    pdl_launch_dependents();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.0f;
        for (int j = 0; j < n_taps; j++) {
            const int lag = n_taps - 1 - j;
            const int src = i_in_step - lag;
            const float x = src >= 0 ? to_f32(proj[(size_t)(t - lag) * ld + c]) : tail[(size_t)(n_taps - 1 + src) * channels + c];
            y = fmaf(taps[(size_t)c * n_taps + j], x, y);
        }
        act[c] = silu_f(y);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    float* out = qkv + (size_t)t * ld_qkv;
    for (int head = warp; head < 2 * n_qk_heads; head += n_warps) {                      // q heads, then k heads
        const float* x = act + head * qk_dim;
        float ss = 0.0f;
        for (int i = lane; i < qk_dim; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float inv = (head < n_qk_heads ? q_scale : 1.0f) / sqrtf(ss + 1e-6f);
        for (int i = lane; i < qk_dim; i += 32) out[head * qk_dim + i] = x[i] * inv;
    }
    for (int c = 2 * qk + threadIdx.x; c < channels; c += blockDim.x) out[c] = act[c];
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        const float b = gates[(size_t)t * ld_gates + h], a = gates[(size_t)t * ld_gates + n_heads + h];
        bg[(size_t)t * 2 * n_heads + h] = 1.0f / (1.0f + expf(-b));
        bg[(size_t)t * 2 * n_heads + n_heads + h] = -expf(a_log[h]) * softplus_f(a + dt_bias[h]);      // log of the decay
    }
}

// The convolution's tail after the step: the last n_taps - 1 inputs of every request.  One block per request;
// a thread reads all it needs of the old tail before it writes.
template <typename T>
__global__ void __launch_bounds__(256)
conv_tail_kernel(const T* __restrict__ proj, int ld, int channels, int n_taps, float* __restrict__ state,
                 long long state_stride, long long tail_off, const int* __restrict__ q_start,
                 const int* __restrict__ seq_slots) {
    const int s = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int t0 = q_start[s], n = q_start[s + 1] - t0;
    float* tail = state + (long long)seq_slots[s] * state_stride + tail_off;
    const int keep = n_taps - 1;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float v[MAX_TAPS];
#pragma unroll
        for (int j = 0; j < MAX_TAPS; j++) {
            if (j < keep) {
                const int r = n - keep + j;           // position among the step's tokens; negative: in the old tail
                v[j] = r >= 0 ? to_f32(proj[(size_t)(t0 + r) * ld + c]) : tail[(size_t)(keep + r) * channels + c];
            }
        }
#pragma unroll
        for (int j = 0; j < MAX_TAPS; j++)
            if (j < keep) tail[(size_t)j * channels + c] = v[j];
    }
}

// Sum of each of N values over the warp; every lane gets all sums.
template <int N>
__device__ __forceinline__ void warp_sum_all(float (&v)[N]) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < N; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
}

// What one token brings to a block of columns, as it lies in shared memory:
// k [d], q [d], v [COLS], two scalars (delta: beta, g;  matrix memory: log i, log f).
__device__ __forceinline__ int per_token(int d) { return 2 * d + COLS + 2; }

// ---- gated delta rule: the recurrence ---------------------------------------------------------------------
// qkv: float32 [T, ld] rows of (q [Hqk * d], k [Hqk * d], v [H * e]) as delta_prepare left them; bg: [T, 2H]
// (beta, then the logarithm of the decay).  Requests that bring `long_from` tokens or more are left to the chunked
// kernel below (0: none are).
template <int R>
__global__ void __launch_bounds__(THREADS)
delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ bg, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                  float* __restrict__ out, int ld_out, int n_heads, int n_qk_heads, int d, int e, int long_from) {
    extern __shared__ float stage[];                  // [CHUNK][per_token]
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qh = h / (n_heads / n_qk_heads);
    const int per = per_token(d);
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (long_from > 0 && t1 - t0 >= long_from) return;
    float* S = state + (long long)seq_slots[s] * state_stride + (long long)h * e * d;    // [e][d]
    pdl_wait();
    float st[R][CPW];
#pragma unroll
    for (int c = 0; c < CPW; c++) {
        const int col = col0 + warp * CPW + c;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = lane + 32 * r;
            st[r][c] = (col < e && i < d) ? S[(size_t)col * d + i] : 0.0f;
        }
    }
    constexpr int NL = (CHUNK * (2 * 32 * R + COLS + 2) + THREADS - 1) / THREADS;
    float pre[NL];
    auto fetch = [&](int tc) {
        const int n_tok = min(CHUNK, t1 - tc);
#pragma unroll
        for (int x = 0; x < NL; x++) {
            const int f = threadIdx.x + x * THREADS;
            const int tok = f / per, j = f % per;
            float v = 0.0f;
            if (tok < n_tok) {
                const float* row = qkv + (size_t)(tc + tok) * ld;
                if (j < d) v = row[(n_qk_heads + qh) * d + j];
                else if (j < 2 * d) v = row[qh * d + (j - d)];
                else if (j < 2 * d + COLS) {
                    const int col = col0 + j - 2 * d;
                    v = col < e ? row[2 * n_qk_heads * d + h * e + col] : 0.0f;
                } else {
                    v = bg[(size_t)(tc + tok) * 2 * n_heads + (j - 2 * d - COLS) * n_heads + h];
                    if (j == 2 * d + COLS + 1) v = expf(v);       // bg holds the decay's logarithm
                }
            }
            pre[x] = v;
        }
    };
    if (t0 < t1) fetch(t0);
    for (int tc = t0; tc < t1; tc += CHUNK) {
        __syncthreads();
#pragma unroll
        for (int x = 0; x < NL; x++) {
            const int f = threadIdx.x + x * THREADS;
            if (f < CHUNK * per) stage[f] = pre[x];
        }
        __syncthreads();
        if (tc + CHUNK < t1) fetch(tc + CHUNK);
        const int n_tok = min(CHUNK, t1 - tc);
        for (int tok = 0; tok < n_tok; tok++) {
            const float* in = stage + tok * per;
            float k[R], q[R];
            float red[2 * CPW + 1];
#pragma unroll
            for (int x = 0; x < 2 * CPW + 1; x++) red[x] = 0.0f;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int i = lane + 32 * r;
                k[r] = i < d ? in[i] : 0.0f;
                q[r] = i < d ? in[d + i] : 0.0f;
                red[2 * CPW] = fmaf(k[r], q[r], red[2 * CPW]);
#pragma unroll
                for (int c = 0; c < CPW; c++) {
                    red[c] = fmaf(st[r][c], k[r], red[c]);
                    red[CPW + c] = fmaf(st[r][c], q[r], red[CPW + c]);
                }
            }
            warp_sum_all(red);
            const float beta = in[2 * d + COLS], g = in[2 * d + COLS + 1];
            float o_mine = 0.0f;
#pragma unroll
            for (int c = 0; c < CPW; c++) {
                const float v = in[2 * d + warp * CPW + c];
                const float u = beta * (v - g * red[c]);
                const float o = g * red[CPW + c] + u * red[2 * CPW];
                if (lane == c) o_mine = o;
#pragma unroll
                for (int r = 0; r < R; r++) st[r][c] = fmaf(k[r], u, g * st[r][c]);
            }
            const int col = col0 + warp * CPW + lane;
            if (lane < CPW && col < e) out[(size_t)(tc + tok) * ld_out + h * e + col] = o_mine;
        }
    }
    pdl_launch_dependents();
    if (t0 < t1) {
#pragma unroll
        for (int c = 0; c < CPW; c++) {
            const int col = col0 + warp * CPW + c;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int i = lane + 32 * r;
                if (col < e && i < d) S[(size_t)col * d + i] = st[r][c];
            }
        }
    }
}

// ---- matrix memory: the recurrence ------------------------------------------------------------------------
// proj: [T, ld] of T with q at q_off + h * d, k at k_off + h * d, v at v_off + h * e; gates: float32 [T, ld_gates]
// with the input gate's pre-activation at column h and the forget gate's at n_heads + h; their biases gate_bias
// [2H].  log i = cap tanh((x + b) / cap), log f = logsigmoid(cap tanh((y + b') / cap)).  q is scaled by q_scale.
// State of a slot: S [H][e][d], then n [H][Z][d], then m [H][Z], Z = ceil(e / COLS).
template <typename T, int R>
__global__ void __launch_bounds__(THREADS)
mlstm_scan_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                  int ld_gates, const float* __restrict__ gate_bias, float cap, float q_scale, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                  float* __restrict__ out, int ld_out, int n_heads, int d, int e, int long_from) {
    extern __shared__ float stage[];
    const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, col0 = z * COLS, Z = gridDim.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per = per_token(d);
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (long_from > 0 && t1 - t0 >= long_from) return;
    float* base = state + (long long)seq_slots[s] * state_stride;
    float* S = base + (long long)h * e * d;
    float* n_st = base + (long long)n_heads * e * d + ((long long)h * Z + z) * d;
    float* m_st = base + (long long)n_heads * e * d + (long long)n_heads * Z * d + (long long)h * Z + z;
    const float bias_i = gate_bias[h], bias_f = gate_bias[n_heads + h];
    pdl_wait();
    float st[R][CPW], nv[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = lane + 32 * r;
        nv[r] = i < d ? n_st[i] : 0.0f;
#pragma unroll
        for (int c = 0; c < CPW; c++) {
            const int col = col0 + warp * CPW + c;
            st[r][c] = (col < e && i < d) ? S[(size_t)col * d + i] : 0.0f;
        }
    }
    float m = *m_st;
    constexpr int NL = (CHUNK * (2 * 32 * R + COLS + 2) + THREADS - 1) / THREADS;
    float pre[NL];
    auto fetch = [&](int tc) {
        const int n_tok = min(CHUNK, t1 - tc);
#pragma unroll
        for (int x = 0; x < NL; x++) {
            const int f = threadIdx.x + x * THREADS;
            const int tok = f / per, j = f % per;
            float v = 0.0f;
            if (tok < n_tok) {
                const T* row = proj + (size_t)(tc + tok) * ld;
                if (j < d) v = to_f32(row[k_off + h * d + j]);
                else if (j < 2 * d) v = to_f32(row[q_off + h * d + (j - d)]) * q_scale;
                else if (j < 2 * d + COLS) {
                    const int col = col0 + j - 2 * d;
                    v = col < e ? to_f32(row[v_off + h * e + col]) : 0.0f;
                } else if (j == 2 * d + COLS) {
                    v = cap * tanhf((gates[(size_t)(tc + tok) * ld_gates + h] + bias_i) / cap);
                } else {
                    v = log_sigmoid_f(cap * tanhf((gates[(size_t)(tc + tok) * ld_gates + n_heads + h] + bias_f) / cap));
                }
            }
            pre[x] = v;
        }
    };
    if (t0 < t1) fetch(t0);
    for (int tc = t0; tc < t1; tc += CHUNK) {
        __syncthreads();
#pragma unroll
        for (int x = 0; x < NL; x++) {
            const int f = threadIdx.x + x * THREADS;
            if (f < CHUNK * per) stage[f] = pre[x];
        }
        __syncthreads();
        if (tc + CHUNK < t1) fetch(tc + CHUNK);
        const int n_tok = min(CHUNK, t1 - tc);
        for (int tok = 0; tok < n_tok; tok++) {
            const float* in = stage + tok * per;
            const float li = in[2 * d + COLS], lf = in[2 * d + COLS + 1];
            const float m_new = fmaxf(lf + m, li);
            const float a = expf(lf + m - m_new), b = expf(li - m_new);
            m = m_new;
            float red[CPW + 1];
#pragma unroll
            for (int x = 0; x < CPW + 1; x++) red[x] = 0.0f;
            float bv[CPW];
#pragma unroll
            for (int c = 0; c < CPW; c++) bv[c] = b * in[2 * d + warp * CPW + c];
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int i = lane + 32 * r;
                const float k = i < d ? in[i] : 0.0f, q = i < d ? in[d + i] : 0.0f;
                nv[r] = fmaf(b, k, a * nv[r]);
                red[CPW] = fmaf(nv[r], q, red[CPW]);
#pragma unroll
                for (int c = 0; c < CPW; c++) {
                    st[r][c] = fmaf(bv[c], k, a * st[r][c]);
                    red[c] = fmaf(st[r][c], q, red[c]);
                }
            }
            warp_sum_all(red);
            const float den = fmaxf(fabsf(red[CPW]), expf(-m)) + 1e-6f;
            float o_mine = 0.0f;
#pragma unroll
            for (int c = 0; c < CPW; c++)
                if (lane == c) o_mine = red[c] / den;
            const int col = col0 + warp * CPW + lane;
            if (lane < CPW && col < e) out[(size_t)(tc + tok) * ld_out + h * e + col] = o_mine;
        }
    }
    pdl_launch_dependents();
    if (t0 < t1) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = lane + 32 * r;
            if (warp == 0 && i < d) n_st[i] = nv[r];
#pragma unroll
            for (int c = 0; c < CPW; c++) {
                const int col = col0 + warp * CPW + c;
                if (col < e && i < d) S[(size_t)col * d + i] = st[r][c];
            }
        }
        if (threadIdx.x == 0) *m_st = m;
    }
}

// ---- the same recurrences, a chunk of tokens at a time ----------------------------------------------------
// Walking a prompt token by token leaves a warp one short dependent chain per token (measured: 240 instructions
// at 6 cycles each), so a request that brings many tokens is taken CC tokens at a time instead.  Inside a chunk
// everything is a small matrix product in float32 (FFMA; the design wants the recurrences in 32-bit, so no tensor
// cores), parallel over the chunk's tokens; only the state goes from chunk to chunk.  With S0 the state before the
// chunk, tokens 1..CC, and sums over j <= t unless said otherwise:
//
//   matrix memory   F_t = sum_{l<=t} log f_l;  a_j = log i_j - F_j;  M_t = max(m0, max_{j<=t} a_j);  m_t = F_t + M_t
//                   w(t, j) = exp(a_j - M_t) (never above one);  c_t = exp(m0 - M_t)
//                   S_t = c_t S0 + sum_j w(t, j) k_j v_j^T;   n_t likewise
//                   o_t = (c_t S0^T q_t + sum_j w(t, j) (q_t . k_j) v_j) / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//   delta rule      G_t = sum_{l<=t} log g_l;  r(t, j) = exp(G_t - G_j)
//                   u_t = beta_t (v_t - exp(G_t) S0^T k_t - sum_{j<t} r(t, j) (k_t . k_j) u_j)      a triangular system,
//                                                                                                   solved row by row
//                   o_t = exp(G_t) S0^T q_t + sum_j r(t, j) (q_t . k_j) u_j
//                   S_CC = exp(G_CC) S0 + sum_j r(CC, j) k_j u_j^T
//
// A block owns COLS columns of one head's state, as in the kernels above (and recomputes the products that do not
// depend on the column: q . k, k . k).  Tokens beyond a request's last are given weights of zero (log i = -inf,
// beta = 0) and decays of one, so that a partly filled chunk leaves the state where its last token left it.
constexpr int CC = 32;                 // tokens per chunk
constexpr int CT = 256;                // threads: a token row of q k^T, two columns of a read-out each
constexpr int LA = CC + 4;             // row pitch of the CC x CC matrices

// x . y_b for one row x and 4 rows y_b of Y that lie 8 rows apart, rows of `len` floats (a multiple of 4) at pitch
// ld.  A warp's threads then read neighbouring rows of Y, which lie in different banks (the pitch is 4 mod 32).
__device__ __forceinline__ void tile_1x4(const float* __restrict__ X, const float* __restrict__ Y, int ld, int len,
                                         float (&acc)[4]) {
#pragma unroll
    for (int b = 0; b < 4; b++) acc[b] = 0.0f;
    for (int i = 0; i < len; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(X + i);
        float4 y[4];
#pragma unroll
        for (int b = 0; b < 4; b++) y[b] = *reinterpret_cast<const float4*>(Y + b * 8 * ld + i);
#pragma unroll
        for (int b = 0; b < 4; b++) {
            acc[b] = fmaf(x.x, y[b].x, acc[b]);
            acc[b] = fmaf(x.y, y[b].y, acc[b]);
            acc[b] = fmaf(x.z, y[b].z, acc[b]);
            acc[b] = fmaf(x.w, y[b].w, acc[b]);
        }
    }
}

struct ChunkSmem {
    float *q, *k, *v, *qk, *kk, *s0, *n0, *v1, *v2, *v3, *v4;
};
__device__ __forceinline__ ChunkSmem carve(float* base, int dp, bool two) {
    ChunkSmem m;
    const int ld = dp + 4;
    m.q = base;
    m.k = m.q + CC * ld;
    m.v = m.k + CC * ld;                 // [CC][COLS]
    m.qk = m.v + CC * COLS;              // [CC][LA]
    m.kk = m.qk + CC * LA;               // [CC][LA] (delta rule only)
    m.s0 = m.kk + (two ? CC * LA : 0);   // [dp][COLS]
    m.n0 = m.s0 + dp * COLS;             // [dp]
    m.v1 = m.n0 + dp;                    // four vectors of CC
    m.v2 = m.v1 + CC;
    m.v3 = m.v2 + CC;
    m.v4 = m.v3 + CC;
    return m;
}
size_t chunk_smem_bytes(int d, bool two) {
    const int dp = (d + 3) / 4 * 4;
    return (size_t)(2 * CC * (dp + 4) + CC * COLS + (two ? 2 : 1) * CC * LA + dp * COLS + dp + 4 * CC) * sizeof(float);
}

// Inclusive running sum / maximum over the 32 lanes of a warp.
__device__ __forceinline__ float warp_scan_sum(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}
__device__ __forceinline__ float warp_scan_max(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v = fmaxf(v, u);
    }
    return v;
}
static_assert(CC == 32, "the running sums of a chunk are one warp's scan");

// DPMAX: the head's query/key size rounded up to 32, 64, 128 or 256.  Up to 128 a thread holds its share of the next
// chunk's queries and keys in registers while this chunk is computed (NPRE of them: 2 * CC * dp <= NPRE * CT); wider
// heads are staged when their chunk begins.  MAXR: rows of the state a thread owns.
template <typename T, int DPMAX>
__global__ void __launch_bounds__(CT)          // all registers: capped at 128 it ran at half the speed (343 against 190 us)
mlstm_chunk_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                   int ld_gates, const float* __restrict__ gate_bias, float cap, float q_scale, float* __restrict__ state,
                   long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                   float* __restrict__ out, int ld_out, int n_heads, int d, int e, int long_from) {
    extern __shared__ __align__(16) float chunk_raw[];
    constexpr int NPRE = DPMAX <= 128 ? 2 * CC * DPMAX / CT : 0;
    constexpr int MAXR = DPMAX / 32;
    const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, col0 = z * COLS, Z = gridDim.z;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 - t0 < long_from) return;
    const int dp = (d + 3) / 4 * 4, ldq = dp + 4;
    const ChunkSmem m = carve(chunk_raw, dp, false);
    float* li = m.v1;     // a_j
    float* Ms = m.v2;     // M_t
    float* cw = m.v3;     // c_t
    float* Fs = m.v4;     // F_t
    __shared__ float m0_s;
    const int tid = threadIdx.x;
    float* base = state + (long long)seq_slots[s] * state_stride;
    float* S = base + (long long)h * e * d;
    float* n_st = base + (long long)n_heads * e * d + ((long long)h * Z + z) * d;
    float* m_st = base + (long long)n_heads * e * d + (long long)n_heads * Z * d + (long long)h * Z + z;
    const float bias_i = gate_bias[h], bias_f = gate_bias[n_heads + h];
    pdl_wait();
    for (int x = tid; x < dp * COLS; x += CT) {
        const int c = x / dp, i = x % dp;                // consecutive threads read consecutive rows of a column
        m.s0[i * COLS + c] = (i < d && col0 + c < e) ? S[(size_t)(col0 + c) * d + i] : 0.0f;
    }
    for (int i = tid; i < dp; i += CT) m.n0[i] = i < d ? n_st[i] : 0.0f;
    if (tid == 0) m0_s = *m_st;
    const int tr = tid / 8, tc4 = tid % 8;               // this thread's row and four columns of q k^T
    const int ot = tid / 8, oc = (tid % 8) * 2;          // this thread's token and two columns of the read-out
    // the next chunk's inputs wait in registers while this chunk is computed
    // (as loaded: an instruction that used a value here would make the warp wait for it)
    T pre_qk[NPRE > 0 ? NPRE : 1], pre_v[CC * COLS / CT];
    float pre_g[2];
    auto fetch = [&](int tcn) {
        const int n_tok = min(CC, t1 - tcn);              // <= 0 behind the last chunk: nothing is read
#pragma unroll
        for (int u = 0; u < NPRE; u++) {
            const int x = tid + u * CT;
            const int which = x / (CC * dp), rem = x % (CC * dp);
            const int t = rem / dp, i = rem % dp;
            T v = from_f32<T>(0.0f);
            if (which < 2 && t < n_tok && i < d) v = proj[(size_t)(tcn + t) * ld + (which == 0 ? q_off : k_off) + h * d + i];
            pre_qk[u] = v;
        }
#pragma unroll
        for (int u = 0; u < CC * COLS / CT; u++) {
            const int x = tid + u * CT;
            const int t = x / COLS, c = x % COLS;
            T v = from_f32<T>(0.0f);
            if (t < n_tok && col0 + c < e) v = proj[(size_t)(tcn + t) * ld + v_off + h * e + col0 + c];
            pre_v[u] = v;
        }
        pre_g[0] = pre_g[1] = 0.0f;
        if (tid < CC && tid < n_tok) {
            const float* g = gates + (size_t)(tcn + tid) * ld_gates;
            pre_g[0] = g[h];
            pre_g[1] = g[n_heads + h];
        }
    };
    fetch(t0);
    for (int tc = t0; tc < t1; tc += CC) {
        const int n_tok = min(CC, t1 - tc);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < NPRE; u++) {
            const int x = tid + u * CT;
            const int which = x / (CC * dp), rem = x % (CC * dp);
            if (which < 2) (which == 0 ? m.q : m.k)[(rem / dp) * ldq + rem % dp] = to_f32(pre_qk[u]) * (which == 0 ? q_scale : 1.0f);
        }
        if (NPRE == 0)
            for (int x = tid; x < CC * dp; x += CT) {
                const int t = x / dp, i = x % dp;
                const bool live = t < n_tok && i < d;
                const T* row = proj + (size_t)(tc + t) * ld;
                m.q[t * ldq + i] = live ? to_f32(row[q_off + h * d + i]) * q_scale : 0.0f;
                m.k[t * ldq + i] = live ? to_f32(row[k_off + h * d + i]) : 0.0f;
            }
#pragma unroll
        for (int u = 0; u < CC * COLS / CT; u++) m.v[tid + u * CT] = to_f32(pre_v[u]);
        if (tid < CC) {
            const bool live = tid < n_tok;
            li[tid] = live ? cap * tanhf((pre_g[0] + bias_i) / cap) : -INFINITY;
            Fs[tid] = live ? log_sigmoid_f(cap * tanhf((pre_g[1] + bias_f) / cap)) : 0.0f;
        }
        __syncthreads();
        fetch(tc + CC);
        if (tid < CC) {                                   // the running sums and maxima: one warp's scans
            const float F = warp_scan_sum(Fs[tid], tid);
            const float a = li[tid] - F;
            const float M = fmaxf(warp_scan_max(a, tid), m0_s);
            li[tid] = a;
            Fs[tid] = F;
            Ms[tid] = M;
            cw[tid] = expf(m0_s - M);
        }
        {
            float acc[4];
            tile_1x4(m.q + tr * ldq, m.k + tc4 * ldq, ldq, dp, acc);
#pragma unroll
            for (int b = 0; b < 4; b++) m.qk[tr * LA + tc4 + 8 * b] = acc[b];
        }
        __syncthreads();
        for (int x = tid; x < CC * CC; x += CT) {         // weights: w(t, j) (q_t . k_j), zero above the diagonal
            const int t = x / CC, j = x % CC;
            m.qk[t * LA + j] = j <= t ? m.qk[t * LA + j] * expf(li[j] - Ms[t]) : 0.0f;
        }
        __syncthreads();
        // read-out of token ot, columns oc and oc + 1
        float o[2] = {0.0f, 0.0f}, nq = 0.0f;
        {
            const float* qrow = m.q + ot * ldq;
            for (int i = 0; i < dp; i++) {
                const float qi = qrow[i];
                const float2 sv = *reinterpret_cast<const float2*>(m.s0 + i * COLS + oc);
                o[0] = fmaf(qi, sv.x, o[0]); o[1] = fmaf(qi, sv.y, o[1]);
                nq = fmaf(qi, m.n0[i], nq);
            }
            const float c = cw[ot];
            o[0] *= c; o[1] *= c; nq *= c;
            const float* prow = m.qk + ot * LA;
            for (int j = 0; j <= ot; j++) {
                const float p = prow[j];
                const float2 vv = *reinterpret_cast<const float2*>(m.v + j * COLS + oc);
                o[0] = fmaf(p, vv.x, o[0]); o[1] = fmaf(p, vv.y, o[1]);
                nq += p;
            }
            if (ot < n_tok) {
                const float den = fmaxf(fabsf(nq), expf(-(Fs[ot] + Ms[ot]))) + 1e-6f;
#pragma unroll
                for (int c2 = 0; c2 < 2; c2++)
                    if (col0 + oc + c2 < e) out[(size_t)(tc + ot) * ld_out + h * e + col0 + oc + c2] = o[c2] / den;
            }
        }
        // the state after the chunk: rows i = ot, ot + 32, ..., columns oc .. oc + 3 (kept in registers until everyone has read S0)
        float sn[MAXR][2], nn[MAXR];
        const float c_last = cw[CC - 1], M_last = Ms[CC - 1];
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
            const int i = ot + 32 * r;
            if (i < dp) {
                const float2 sv = *reinterpret_cast<const float2*>(m.s0 + i * COLS + oc);
                sn[r][0] = c_last * sv.x; sn[r][1] = c_last * sv.y;
                nn[r] = c_last * m.n0[i];
            }
        }
        for (int j = 0; j < CC; j++) {
            const float w = expf(li[j] - M_last);
            const float2 vv = *reinterpret_cast<const float2*>(m.v + j * COLS + oc);
#pragma unroll
            for (int r = 0; r < MAXR; r++) {
                const int i = ot + 32 * r;
                if (i < dp) {
                    const float wk = w * m.k[j * ldq + i];
                    sn[r][0] = fmaf(wk, vv.x, sn[r][0]); sn[r][1] = fmaf(wk, vv.y, sn[r][1]);
                    nn[r] += wk;
                }
            }
        }
        const float m_new = Fs[CC - 1] + M_last;
        __syncthreads();
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
            const int i = ot + 32 * r;
            if (i < dp) {
                *reinterpret_cast<float2*>(m.s0 + i * COLS + oc) = make_float2(sn[r][0], sn[r][1]);
                if (oc == 0) m.n0[i] = nn[r];
            }
        }
        if (tid == 0) m0_s = m_new;
    }
    __syncthreads();
    pdl_launch_dependents();
    for (int x = tid; x < dp * COLS; x += CT) {
        const int c = x / dp, i = x % dp;
        if (i < d && col0 + c < e) S[(size_t)(col0 + c) * d + i] = m.s0[i * COLS + c];
    }
    for (int i = tid; i < d; i += CT) n_st[i] = m.n0[i];
    if (tid == 0) *m_st = m0_s;
}

template <int DPMAX>
__global__ void __launch_bounds__(CT, 2)       // two blocks an SM: wide models have more blocks than SMs (1,000 -> 408 us at 24 heads)
delta_chunk_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ bg, float* __restrict__ state,
                   long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                   float* __restrict__ out, int ld_out, int n_heads, int n_qk_heads, int d, int e, int long_from) {
    extern __shared__ __align__(16) float chunk_raw[];
    constexpr int NPRE = DPMAX <= 128 ? 2 * CC * DPMAX / CT : 0;
    constexpr int MAXR = DPMAX / 32;
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 - t0 < long_from) return;
    const int qh = h / (n_heads / n_qk_heads);
    const int dp = (d + 3) / 4 * 4, ldq = dp + 4;
    const ChunkSmem m = carve(chunk_raw, dp, true);
    float* beta = m.v1;
    float* G = m.v2;      // running sum of the decays' logarithms
    const int tid = threadIdx.x;
    float* S = state + (long long)seq_slots[s] * state_stride + (long long)h * e * d;
    pdl_wait();
    for (int x = tid; x < dp * COLS; x += CT) {
        const int c = x / dp, i = x % dp;
        m.s0[i * COLS + c] = (i < d && col0 + c < e) ? S[(size_t)(col0 + c) * d + i] : 0.0f;
    }
    const int tr = tid / 8, tc4 = tid % 8;
    const int ot = tid / 8, oc = (tid % 8) * 2;
    float pre_qk[NPRE > 0 ? NPRE : 1], pre_v[CC * COLS / CT], pre_g[2];
    auto fetch = [&](int tcn) {
        const int n_tok = min(CC, t1 - tcn);
#pragma unroll
        for (int u = 0; u < NPRE; u++) {
            const int x = tid + u * CT;
            const int which = x / (CC * dp), rem = x % (CC * dp);
            const int t = rem / dp, i = rem % dp;
            float v = 0.0f;
            if (which < 2 && t < n_tok && i < d) v = qkv[(size_t)(tcn + t) * ld + (which * n_qk_heads + qh) * d + i];
            pre_qk[u] = v;
        }
#pragma unroll
        for (int u = 0; u < CC * COLS / CT; u++) {
            const int x = tid + u * CT;
            const int t = x / COLS, c = x % COLS;
            pre_v[u] = (t < n_tok && col0 + c < e) ? qkv[(size_t)(tcn + t) * ld + 2 * n_qk_heads * d + h * e + col0 + c] : 0.0f;
        }
        pre_g[0] = pre_g[1] = 0.0f;
        if (tid < CC && tid < n_tok) {
            pre_g[0] = bg[(size_t)(tcn + tid) * 2 * n_heads + h];
            pre_g[1] = bg[(size_t)(tcn + tid) * 2 * n_heads + n_heads + h];
        }
    };
    fetch(t0);
    for (int tc = t0; tc < t1; tc += CC) {
        const int n_tok = min(CC, t1 - tc);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < NPRE; u++) {
            const int x = tid + u * CT;
            const int which = x / (CC * dp), rem = x % (CC * dp);
            if (which < 2) (which == 0 ? m.q : m.k)[(rem / dp) * ldq + rem % dp] = pre_qk[u];
        }
        if (NPRE == 0)
            for (int x = tid; x < CC * dp; x += CT) {
                const int t = x / dp, i = x % dp;
                const bool live = t < n_tok && i < d;
                const float* row = qkv + (size_t)(tc + t) * ld;
                m.q[t * ldq + i] = live ? row[qh * d + i] : 0.0f;
                m.k[t * ldq + i] = live ? row[(n_qk_heads + qh) * d + i] : 0.0f;
            }
#pragma unroll
        for (int u = 0; u < CC * COLS / CT; u++) m.v[tid + u * CT] = pre_v[u];
        if (tid < CC) {
            beta[tid] = pre_g[0];
            G[tid] = warp_scan_sum(pre_g[1], tid);        // running sum of the decays' logarithms
        }
        __syncthreads();
        fetch(tc + CC);
        {
            float acc[4];
            tile_1x4(m.q + tr * ldq, m.k + tc4 * ldq, ldq, dp, acc);
#pragma unroll
            for (int b = 0; b < 4; b++) m.qk[tr * LA + tc4 + 8 * b] = acc[b];
            tile_1x4(m.k + tr * ldq, m.k + tc4 * ldq, ldq, dp, acc);
#pragma unroll
            for (int b = 0; b < 4; b++) m.kk[tr * LA + tc4 + 8 * b] = acc[b];
        }
        __syncthreads();
        for (int x = tid; x < CC * CC; x += CT) {
            const int t = x / CC, j = x % CC;
            const float r = j <= t ? expf(G[t] - G[j]) : 0.0f;
            m.qk[t * LA + j] = m.qk[t * LA + j] * r;                             // r(t, j) (q_t . k_j), j <= t
            m.kk[t * LA + j] = j < t ? beta[t] * r * m.kk[t * LA + j] : 0.0f;    // beta_t r(t, j) (k_t . k_j), j < t
        }
        // what S0 gives token ot, columns oc and oc + 1: to the right-hand side of the system and to the read-out
        float o[2] = {0.0f, 0.0f}, bk[2] = {0.0f, 0.0f};
        {
            const float* qrow = m.q + ot * ldq;
            const float* krow = m.k + ot * ldq;
            for (int i = 0; i < dp; i++) {
                const float qi = qrow[i], ki = krow[i];
                const float2 sv = *reinterpret_cast<const float2*>(m.s0 + i * COLS + oc);
                o[0] = fmaf(qi, sv.x, o[0]); o[1] = fmaf(qi, sv.y, o[1]);
                bk[0] = fmaf(ki, sv.x, bk[0]); bk[1] = fmaf(ki, sv.y, bk[1]);
            }
            const float gt = expf(G[ot]);
            float2 vv = *reinterpret_cast<const float2*>(m.v + ot * COLS + oc);
            vv.x = beta[ot] * (vv.x - gt * bk[0]); vv.y = beta[ot] * (vv.y - gt * bk[1]);
            o[0] *= gt; o[1] *= gt;
            *reinterpret_cast<float2*>(m.v + ot * COLS + oc) = vv;              // each thread reads and writes its own two
        }
        __syncthreads();
        // The triangular system u_t = b_t - sum_{j<t} L(t, j) u_j, eight rows at a time: what the rows solved so far
        // give the next eight is subtracted by 128 threads at once; inside the eight, a column a thread, rows in order.
        for (int r0 = 0; r0 < CC; r0 += 8) {
            if (r0 > 0) {
                if (tid < 8 * COLS) {
                    const int t = r0 + tid / COLS, c = tid % COLS;
                    const float* lrow = m.kk + t * LA;
                    float a0 = 0.0f, a1 = 0.0f;
                    for (int j = 0; j < r0; j += 2) {
                        a0 = fmaf(lrow[j], m.v[j * COLS + c], a0);
                        a1 = fmaf(lrow[j + 1], m.v[(j + 1) * COLS + c], a1);
                    }
                    m.v[t * COLS + c] -= a0 + a1;
                }
                __syncthreads();
            }
            if (tid < COLS) {
                float u[8];
                u[0] = m.v[r0 * COLS + tid];
#pragma unroll
                for (int a = 1; a < 8; a++) {
                    const float* lrow = m.kk + (r0 + a) * LA + r0;
                    float acc = 0.0f;
#pragma unroll
                    for (int b = 0; b < a; b++) acc = fmaf(lrow[b], u[b], acc);
                    u[a] = m.v[(r0 + a) * COLS + tid] - acc;
                    m.v[(r0 + a) * COLS + tid] = u[a];
                }
            }
            __syncthreads();
        }
        {
            const float* prow = m.qk + ot * LA;
            for (int j = 0; j <= ot; j++) {
                const float p = prow[j];
                const float2 uu = *reinterpret_cast<const float2*>(m.v + j * COLS + oc);
                o[0] = fmaf(p, uu.x, o[0]); o[1] = fmaf(p, uu.y, o[1]);
            }
            if (ot < n_tok)
#pragma unroll
                for (int c2 = 0; c2 < 2; c2++)
                    if (col0 + oc + c2 < e) out[(size_t)(tc + ot) * ld_out + h * e + col0 + oc + c2] = o[c2];
        }
        float sn[MAXR][2];
        const float G_last = G[CC - 1], g_all = expf(G_last);
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
            const int i = ot + 32 * r;
            if (i < dp) {
                const float2 sv = *reinterpret_cast<const float2*>(m.s0 + i * COLS + oc);
                sn[r][0] = g_all * sv.x; sn[r][1] = g_all * sv.y;
            }
        }
        for (int j = 0; j < CC; j++) {
            const float w = expf(G_last - G[j]);
            const float2 uu = *reinterpret_cast<const float2*>(m.v + j * COLS + oc);
#pragma unroll
            for (int r = 0; r < MAXR; r++) {
                const int i = ot + 32 * r;
                if (i < dp) {
                    const float wk = w * m.k[j * ldq + i];
                    sn[r][0] = fmaf(wk, uu.x, sn[r][0]); sn[r][1] = fmaf(wk, uu.y, sn[r][1]);
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
            const int i = ot + 32 * r;
            if (i < dp) *reinterpret_cast<float2*>(m.s0 + i * COLS + oc) = make_float2(sn[r][0], sn[r][1]);
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    for (int x = tid; x < dp * COLS; x += CT) {
        const int c = x / dp, i = x % dp;
        if (i < d && col0 + c < e) S[(size_t)(col0 + c) * d + i] = m.s0[i * COLS + c];
    }
}

size_t stage_bytes(int d) { return (size_t)CHUNK * (2 * d + COLS + 2) * sizeof(float); }

}  // namespace

// Floats of one request's matrix-memory state: S [H][e][d], n and m once per block of columns.
SANDY_API long long sandy_mlstm_state_floats(int n_heads, int qk_dim, int v_dim) {
    const long long Z = (v_dim + COLS - 1) / COLS;
    return (long long)n_heads * v_dim * qk_dim + (long long)n_heads * Z * qk_dim + (long long)n_heads * Z;
}

SANDY_API int sandy_delta_prepare(const void* proj, int ld, int dtype, const float* taps, int n_taps, const float* gates,
                                  int ld_gates, const float* a_log, const float* dt_bias, const float* state,
                                  long long state_stride, long long tail_off, const int* token_seq, const int* q_start,
                                  const int* seq_slots, float* qkv, int ld_qkv, float* bg, int n_tokens, int n_heads,
                                  int n_qk_heads, int qk_dim, int v_dim, float q_scale, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!proj || !taps || !gates || !a_log || !dt_bias || !state || !qkv || !bg) return SANDY_ERR_ARGUMENT;
    if (n_taps < 1 || n_taps > MAX_TAPS || n_qk_heads <= 0 || n_heads % n_qk_heads) return SANDY_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(2 * n_qk_heads * qk_dim + n_heads * v_dim) * sizeof(float);
    if (smem > 200 * 1024) return SANDY_ERR_UNSUPPORTED;
#define GO(TT)                                                                                                          \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            cudaError_t err = cudaFuncSetAttribute(delta_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return (int)err;                                                                    \
        }                                                                                                               \
        return sandy_launch(delta_prepare_kernel<TT>, dim3(n_tokens), dim3(256), smem, stream, (const TT*)proj, ld, taps, \
                            n_taps, gates, ld_gates, a_log, dt_bias, state, state_stride, tail_off, token_seq, q_start,  \
                            seq_slots, qkv, ld_qkv, bg, n_heads, n_qk_heads, qk_dim, v_dim, q_scale);                   \
    } while (0)
    if (dtype == SANDY_F32) GO(float);
    if (dtype == SANDY_BF16) GO(bf16);
#undef GO
    return SANDY_ERR_UNSUPPORTED;
}

SANDY_API int sandy_conv_tail(const void* proj, int ld, int dtype, int channels, int n_taps, float* state,
                              long long state_stride, long long tail_off, const int* q_start, const int* seq_slots,
                              int n_seqs, cudaStream_t stream) {
    if (n_seqs == 0 || n_taps <= 1) return SANDY_OK;
    if (!proj || !state || !q_start || !seq_slots) return SANDY_ERR_ARGUMENT;
    if (n_taps > MAX_TAPS) return SANDY_ERR_UNSUPPORTED;
    if (dtype == SANDY_F32)
        return sandy_launch(conv_tail_kernel<float>, dim3(n_seqs), dim3(256), 0, stream, (const float*)proj, ld, channels,
                            n_taps, state, state_stride, tail_off, q_start, seq_slots);
    if (dtype == SANDY_BF16)
        return sandy_launch(conv_tail_kernel<bf16>, dim3(n_seqs), dim3(256), 0, stream, (const bf16*)proj, ld, channels,
                            n_taps, state, state_stride, tail_off, q_start, seq_slots);
    return SANDY_ERR_UNSUPPORTED;
}

SANDY_API int sandy_delta_scan(const float* qkv, int ld, const float* bg, float* state, long long state_stride,
                               const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads,
                               int n_qk_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!qkv || !bg || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || n_qk_heads <= 0 || n_heads % n_qk_heads) return SANDY_ERR_UNSUPPORTED;
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
    const size_t smem = stage_bytes(qk_dim);
#define CASE(RR)                                                                                                       \
    if (qk_dim <= 32 * RR)                                                                                             \
        return sandy_launch(delta_scan_kernel<RR>, grid, dim3(THREADS), smem, stream, qkv, ld, bg, state, state_stride, \
                            q_start, seq_slots, out, ld_out, n_heads, n_qk_heads, qk_dim, v_dim, long_from)
    CASE(1); CASE(2); CASE(3); CASE(4); CASE(6); CASE(8);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

SANDY_API int sandy_mlstm_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off, const float* gates,
                               int ld_gates, const float* gate_bias, float cap, float q_scale, float* state,
                               long long state_stride, const int* q_start, const int* seq_slots, float* out, int ld_out,
                               int n_seqs, int n_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!proj || !gates || !gate_bias || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || !(cap > 0.0f)) return SANDY_ERR_UNSUPPORTED;
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
    const size_t smem = stage_bytes(qk_dim);
#define CASE(TT, RR)                                                                                                     \
    if (qk_dim <= 32 * RR)                                                                                               \
        return sandy_launch(mlstm_scan_kernel<TT, RR>, grid, dim3(THREADS), smem, stream, (const TT*)proj, ld, q_off,    \
                            k_off, v_off, gates, ld_gates, gate_bias, cap, q_scale, state, state_stride, q_start,        \
                            seq_slots, out, ld_out, n_heads, qk_dim, v_dim, long_from)
    if (dtype == SANDY_F32) { CASE(float, 1); CASE(float, 2); CASE(float, 3); CASE(float, 4); CASE(float, 6); CASE(float, 8); }
    if (dtype == SANDY_BF16) { CASE(bf16, 1); CASE(bf16, 2); CASE(bf16, 3); CASE(bf16, 4); CASE(bf16, 6); CASE(bf16, 8); }
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

// The chunked forms: only requests that bring at least `long_from` tokens (the token-by-token kernels above, given
// the same number, take the others).  Arguments as sandy_delta_scan / sandy_mlstm_scan.
SANDY_API int sandy_delta_chunk_scan(const float* qkv, int ld, const float* bg, float* state, long long state_stride,
                                     const int* q_start, const int* seq_slots, float* out, int ld_out, int n_seqs, int n_heads,
                                     int n_qk_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!qkv || !bg || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || n_qk_heads <= 0 || n_heads % n_qk_heads || long_from < 1) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(qkv) & 3) || (reinterpret_cast<uintptr_t>(state) & 3)) return SANDY_ERR_UNSUPPORTED;
    const size_t smem = chunk_smem_bytes(qk_dim, true);
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
#define GO(DPMAX)                                                                                                         \
    do {                                                                                                                  \
        auto kern = delta_chunk_kernel<DPMAX>;                                                              \
        static size_t configured = 0;                                                                                     \
        if (smem > 48 * 1024 && smem > configured) {                                                                      \
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (err != cudaSuccess) return (int)err;                                                                      \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        return sandy_launch(kern, grid, dim3(CT), smem, stream, qkv, ld, bg, state, state_stride, q_start, seq_slots, out, \
                            ld_out, n_heads, n_qk_heads, qk_dim, v_dim, long_from);                                       \
    } while (0)
    if (qk_dim <= 32) GO(32);
    if (qk_dim <= 64) GO(64);
    if (qk_dim <= 128) GO(128);
    GO(256);
#undef GO
}

SANDY_API int sandy_mlstm_chunk_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off, const float* gates,
                                     int ld_gates, const float* gate_bias, float cap, float q_scale, float* state,
                                     long long state_stride, const int* q_start, const int* seq_slots, float* out, int ld_out,
                                     int n_seqs, int n_heads, int qk_dim, int v_dim, int long_from, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!proj || !gates || !gate_bias || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || !(cap > 0.0f) || long_from < 1) return SANDY_ERR_UNSUPPORTED;
    const size_t smem = chunk_smem_bytes(qk_dim, false);
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
#define GO(TT, DPMAX)                                                                                                     \
    do {                                                                                                                  \
        auto kern = mlstm_chunk_kernel<TT, DPMAX>;                                                          \
        static size_t configured = 0;                                                                                     \
        if (smem > 48 * 1024 && smem > configured) {                                                                      \
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (err != cudaSuccess) return (int)err;                                                                      \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        return sandy_launch(kern, grid, dim3(CT), smem, stream, (const TT*)proj, ld, q_off, k_off, v_off, gates, ld_gates, \
                            gate_bias, cap, q_scale, state, state_stride, q_start, seq_slots, out, ld_out, n_heads, qk_dim, \
                            v_dim, long_from);                                                                            \
    } while (0)
#define SIZES(TT)                                                                                                         \
    do {                                                                                                                  \
        if (qk_dim <= 32) GO(TT, 32);                                                                                     \
        if (qk_dim <= 64) GO(TT, 64);                                                                                     \
        if (qk_dim <= 128) GO(TT, 128);                                                                                   \
        GO(TT, 256);                                                                                                      \
    } while (0)
    if (dtype == SANDY_F32) SIZES(float);
    if (dtype == SANDY_BF16) SIZES(bf16);
#undef SIZES
#undef GO
    return SANDY_ERR_UNSUPPORTED;
}
