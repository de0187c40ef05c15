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
// are advanced by every column block for itself and therefore kept once per column block.
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
        bg[(size_t)t * 2 * n_heads + n_heads + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
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
// qkv: float32 [T, ld] rows of (q [Hqk * d], k [Hqk * d], v [H * e]) as delta_prepare left them; bg: [T, 2H].
template <int R>
__global__ void __launch_bounds__(THREADS)
delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ bg, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ seq_slots,
                  float* __restrict__ out, int ld_out, int n_heads, int n_qk_heads, int d, int e) {
    extern __shared__ float stage[];                  // [CHUNK][per_token]
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qh = h / (n_heads / n_qk_heads);
    const int per = per_token(d);
    const int t0 = q_start[s], t1 = q_start[s + 1];
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
                } else v = bg[(size_t)(tc + tok) * 2 * n_heads + (j - 2 * d - COLS) * n_heads + h];
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
                  float* __restrict__ out, int ld_out, int n_heads, int d, int e) {
    extern __shared__ float stage[];
    const int s = blockIdx.x, h = blockIdx.y, z = blockIdx.z, col0 = z * COLS, Z = gridDim.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per = per_token(d);
    const int t0 = q_start[s], t1 = q_start[s + 1];
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
                               int n_qk_heads, int qk_dim, int v_dim, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!qkv || !bg || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || n_qk_heads <= 0 || n_heads % n_qk_heads) return SANDY_ERR_UNSUPPORTED;
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
    const size_t smem = stage_bytes(qk_dim);
#define CASE(RR)                                                                                                       \
    if (qk_dim <= 32 * RR)                                                                                             \
        return sandy_launch(delta_scan_kernel<RR>, grid, dim3(THREADS), smem, stream, qkv, ld, bg, state, state_stride, \
                            q_start, seq_slots, out, ld_out, n_heads, n_qk_heads, qk_dim, v_dim)
    CASE(1); CASE(2); CASE(3); CASE(4); CASE(6); CASE(8);
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}

SANDY_API int sandy_mlstm_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off, const float* gates,
                               int ld_gates, const float* gate_bias, float cap, float q_scale, float* state,
                               long long state_stride, const int* q_start, const int* seq_slots, float* out, int ld_out,
                               int n_seqs, int n_heads, int qk_dim, int v_dim, cudaStream_t stream) {
    if (n_seqs == 0) return SANDY_OK;
    if (!proj || !gates || !gate_bias || !state || !q_start || !seq_slots || !out) return SANDY_ERR_ARGUMENT;
    if (qk_dim <= 0 || qk_dim > 256 || v_dim <= 0 || !(cap > 0.0f)) return SANDY_ERR_UNSUPPORTED;
    const dim3 grid(n_seqs, n_heads, (v_dim + COLS - 1) / COLS);
    const size_t smem = stage_bytes(qk_dim);
#define CASE(TT, RR)                                                                                                     \
    if (qk_dim <= 32 * RR)                                                                                               \
        return sandy_launch(mlstm_scan_kernel<TT, RR>, grid, dim3(THREADS), smem, stream, (const TT*)proj, ld, q_off,    \
                            k_off, v_off, gates, ld_gates, gate_bias, cap, q_scale, state, state_stride, q_start,        \
                            seq_slots, out, ld_out, n_heads, qk_dim, v_dim)
    if (dtype == SANDY_F32) { CASE(float, 1); CASE(float, 2); CASE(float, 3); CASE(float, 4); CASE(float, 6); CASE(float, 8); }
    if (dtype == SANDY_BF16) { CASE(bf16, 1); CASE(bf16, 2); CASE(bf16, 3); CASE(bf16, 4); CASE(bf16, 6); CASE(bf16, 8); }
#undef CASE
    return SANDY_ERR_UNSUPPORTED;
}
