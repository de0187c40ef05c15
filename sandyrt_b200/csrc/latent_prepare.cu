// What lies between the down-projections of attention over a latent and the attention itself, one pass per token.
//
// Attention over a latent keeps, per token, one short vector c (the RMS-normed down-projection of the layer's
// input) and, where the layer has positions, one rotated key part that all heads share.  Keys and values of
// every head are linear in c, so the scores and the weighted sums can be taken in the latent's own space:
//   score_h(i, j) = (U_k,h^T q_h(i)) . c(j) + q_rot,h(i) . k_rot(j),      out_h(i) = U_v,h sum_j p_h(i, j) c(j).
// The cache therefore holds ONE row per token, [c | k_rot | zeros up to the padded size], which is key and
// value at once (a one-plane page), and every query head is an "absorbed" query [U_k,h^T q_h | q_rot,h | zeros].
//
// This kernel does, for one token per block:
//   1. RMS norm of the key/value latent (eps inside the root, a plain gain) in 32-bit;
//   2. rotary positions on the shared key part and on the rotated part of every query head: entries 2i and
//      2i+1 are one pair (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq[i], positions
//      and angles in 32-bit; of `rot_dim` entries the first `rot_dims` turn, the rest pass unchanged;
//   3. the cache row into the request's page (token -> request -> block table -> page);
//   4. the rotated query parts into columns [kv_rank, kv_rank + rot_dim) of every absorbed query head and
//      zeros behind them (the latent columns are written by the per-head product that follows);
//   5. where queries pass a latent of their own: its RMS norm, written in the compute type.
#include "common.cuh"

namespace {

constexpr int THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_prepare_kernel(const float* __restrict__ down, int ld_down, int q_rank, int kv_rank, int rot_dim,
                      const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                      const float* __restrict__ freq, int rot_dims, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                      T* __restrict__ cache, long long page_stride, int page_size, int num_pages, int pad_dim,
                      int write_cache, T* __restrict__ q_latent, int ld_ql, const T* __restrict__ q, int ld_q,
                      int n_heads, int qk_dim, T* __restrict__ q_abs, int ld_qa, int* __restrict__ status) {
    __shared__ float scratch[32];
    extern __shared__ float cs[];                    // cos [rot_dims / 2], sin [rot_dims / 2]
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const int pos = positions[t];                    // the step's index arrays were staged before the step
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float a = (float)pos * freq[i];
        float s, c;
        sincosf(a, &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    long long dst = -1;
    if (write_cache) {
        const int s = token_seq[t];
        const int page = (pos >= 0 && pos / page_size < max_blocks) ? block_table[(size_t)s * max_blocks + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && status) atomicOr(status, 8);
        } else {
            dst = (long long)page * page_stride + (long long)(pos % page_size) * pad_dim;
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    const float* row = down + (size_t)t * ld_down;

    // the query latent's norm
    if (q_rank > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            q_latent[(size_t)t * ld_ql + i] = from_f32<T>(row[i] * inv * q_gain[i]);
    }
    // the key/value latent's norm
    const float* lat = row + q_rank;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(lat[i], lat[i], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);      // its barriers also publish cs

    // entry i of a rotated part whose entries are read through `at`
    auto turned = [&](auto at, int i) -> float {
        if (i >= rot_dims) return at(i);
        const int p = i >> 1;
        const float u = at(i & ~1), v = at(i | 1);
        return (i & 1) ? v * cs[p] + u * cs[half + p] : u * cs[p] - v * cs[half + p];
    };

    if (dst >= 0) {
        const float* kr = lat + kv_rank;
        for (int i = threadIdx.x; i < pad_dim; i += blockDim.x) {
            float v = 0.0f;
            if (i < kv_rank) v = lat[i] * inv * kv_gain[i];
            else if (i < kv_rank + rot_dim) v = turned([&](int j) { return kr[j]; }, i - kv_rank);
            cache[dst + i] = from_f32<T>(v);
        }
    }
    // rotated query parts and the padding of the absorbed queries
    const int tail = pad_dim - kv_rank;              // columns behind the latent part of a head
    if (tail > 0) {
        for (int idx = threadIdx.x; idx < n_heads * tail; idx += blockDim.x) {
            const int h = idx / tail, i = idx % tail;
            float v = 0.0f;
            if (i < rot_dim) {
                const T* qr = q + (size_t)t * ld_q + (size_t)h * (qk_dim + rot_dim) + qk_dim;
                v = turned([&](int j) { return to_f32(qr[j]); }, i);
            }
            q_abs[(size_t)t * ld_qa + (size_t)h * pad_dim + kv_rank + i] = from_f32<T>(v);
        }
    }
}

}  // namespace

// down: float32 [n_tokens, >= q_rank + kv_rank + rot_dim] with pitch ld_down: the query latent (q_rank columns, may
// be 0), the key/value latent, the shared rotated key part (rot_dim columns, may be 0).  Gains float32.  freq: float32
// [rot_dims / 2], rot_dims <= rot_dim and even.  cache: one-plane pages [page][page_size][pad_dim] of dtype, pad_dim >=
// kv_rank + rot_dim.  q_latent: [n_tokens, q_rank] of dtype (q_rank > 0).  q: the query projection [n_tokens, n_heads *
// (qk_dim + rot_dim)] of dtype (read only where rot_dim > 0).  q_abs: [n_tokens, n_heads * pad_dim] of dtype.
SANDY_API int sandy_latent_prepare(const float* down, int ld_down, int n_tokens, int q_rank, int kv_rank, int rot_dim,
                                   const float* q_gain, const float* kv_gain, float eps, const float* freq, int rot_dims,
                                   const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                                   void* cache, long long page_stride, int page_size, int num_pages, int pad_dim,
                                   int write_cache, void* q_latent, int ld_ql, const void* q, int ld_q, int n_heads,
                                   int qk_dim, void* q_abs, int ld_qa, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return SANDY_OK;
    if (!down || !positions || !token_seq || !kv_gain || !q_abs || (write_cache && (!block_table || !cache)) ||
        (q_rank > 0 && (!q_gain || !q_latent)) || (rot_dim > 0 && !q) || (rot_dims > 0 && !freq))
        return SANDY_ERR_ARGUMENT;
    if (kv_rank <= 0 || q_rank < 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) ||
        pad_dim < kv_rank + rot_dim)
        return SANDY_ERR_UNSUPPORTED;
    const size_t smem = (size_t)rot_dims * sizeof(float);
    if (smem > 32 * 1024) return SANDY_ERR_UNSUPPORTED;
    if (dtype == SANDY_F32)
        return sandy_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(THREADS), smem, stream, down, ld_down, q_rank,
                            kv_rank, rot_dim, q_gain, kv_gain, eps, freq, rot_dims, positions, token_seq, block_table,
                            max_blocks, (float*)cache, page_stride, page_size, num_pages, pad_dim, write_cache,
                            (float*)q_latent, ld_ql, (const float*)q, ld_q, n_heads, qk_dim, (float*)q_abs, ld_qa, status);
    if (dtype == SANDY_BF16)
        return sandy_launch(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(THREADS), smem, stream, down, ld_down, q_rank,
                            kv_rank, rot_dim, q_gain, kv_gain, eps, freq, rot_dims, positions, token_seq, block_table,
                            max_blocks, (bf16*)cache, page_stride, page_size, num_pages, pad_dim, write_cache,
                            (bf16*)q_latent, ld_ql, (const bf16*)q, ld_q, n_heads, qk_dim, (bf16*)q_abs, ld_qa, status);
    return SANDY_ERR_UNSUPPORTED;
}
