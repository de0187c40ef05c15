// Products with one small weight matrix per GROUP of rows or columns:
//
//   per head     out[t, g * o_gcols + n] = sum_k W_g[n, k] * a[t, g * a_gcols + k]        every group sees every row;
//                a head's slice of the columns goes through the head's own matrix (the up-projections of attention
//                over a latent: U_k,h^T on the queries, U_v,h on the weighted sums of latents)
//   per expert   out[s, n] = act(sum_k W_g[n, k] * a[row(s), k])  for the slots s of group g     a mixture of experts:
//                slots group_start[g] .. group_start[g+1]-1 belong to expert g (device data: the routing of this
//                step), a slot reads the row a_row[s] / a_row_div of `a` (or row s) and writes row s of `out`
//
// One kernel serves both: a block computes a 32 x 64 tile of one group's output, operands staged through shared
// memory as floats 32 k at a time, every sum carried in 32-bit in a fixed order of k (so a row's result does not
// depend on which rows share its tile).  The weight is [N, K] row-major per group.  A grid of the per-expert form
// covers the worst case of tiles (slots / 32 + groups) and blocks beyond the step's tiles leave at once, so a
// recorded launch serves every routing.
//
// These are FFMA tiles, not tensor-core tiles: K and N here are a head's or an expert's sizes (tens to a few
// hundred), and both compute types share the code.
#include "common.cuh"

namespace {

constexpr int TM = 32, TN = 64, TK = 32, THREADS = 256;

struct GroupedArgs {
    const void* a; int lda; int a_gcols;
    const void* w; long long w_gstride; int ldw;
    void* out; int ldo; int o_gcols;
    int N, K, G, rows;
    const int* group_start;
    const int* a_row; int a_row_div;
    int act;                                        // 0 none, 1 the square of relu
};

template <typename TA, typename TO>
__global__ void __launch_bounds__(THREADS) grouped_tile_kernel(GroupedArgs p) {
    __shared__ float sA[TK][TM + 1];
    __shared__ float sW[TK][TN + 1];
    __shared__ int s_rows[TM];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    int g, row0, row_end;
    if (p.group_start) {
        // which group and which of its tiles this block is
        int tile = blockIdx.y;
        g = 0;
        int start = p.group_start[0], end = start;
        for (; g < p.G; g++) {
            end = p.group_start[g + 1];
            const int tiles = (end - start + TM - 1) / TM;
            if (tile < tiles) break;
            tile -= tiles;
            start = end;
        }
        if (g >= p.G) return;
        row0 = start + tile * TM;
        row_end = end;
    } else {
        g = blockIdx.z;
        row0 = blockIdx.y * TM;
        row_end = p.rows;
    }
    const int n0 = blockIdx.x * TN;
    if (tid < TM) {
        const int s = row0 + tid;
        int r = -1;
        if (s < row_end) r = p.a_row ? p.a_row[s] / p.a_row_div : s;
        s_rows[tid] = r;
    }
    __syncthreads();
    const TA* A = (const TA*)p.a + (size_t)g * p.a_gcols;
    const TA* W = (const TA*)p.w + (size_t)g * p.w_gstride;
    const int tx = tid % 16, ty = tid / 16;
    float acc[2][4] = {};
    const int ar = tid / 8, ak = (tid % 8) * 4;     // this thread's piece of the A tile: row ar, 4 k from ak
    const int wn = tid / 4, wk = (tid % 4) * 8;     // of the W tile: row wn, 8 k from wk
    const int a_row = s_rows[ar];
    for (int k0 = 0; k0 < p.K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + ak + j;
            sA[ak + j][ar] = (a_row >= 0 && k < p.K) ? to_f32(A[(size_t)a_row * p.lda + k]) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int k = k0 + wk + j, n = n0 + wn;
            sW[wk + j][wn] = (n < p.N && k < p.K) ? to_f32(W[(size_t)n * p.ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; k++) {
            const float a0 = sA[k][ty * 2], a1 = sA[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float w = sW[k][tx * 4 + j];
                acc[0][j] = fmaf(a0, w, acc[0][j]);
                acc[1][j] = fmaf(a1, w, acc[1][j]);
            }
        }
        __syncthreads();
    }
    TO* O = (TO*)p.out + (size_t)g * p.o_gcols;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int s = row0 + ty * 2 + i;
        if (s >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (p.act == 1) {
                v = fmaxf(v, 0.0f);
                v = v * v;
            }
            O[(size_t)s * p.ldo + n] = from_f32<TO>(v);
        }
    }
}

template <typename TA, typename TO>
int launch(const GroupedArgs& p, dim3 grid, cudaStream_t stream) {
    return sandy_launch(grouped_tile_kernel<TA, TO>, grid, dim3(THREADS), 0, stream, p);
}

int dispatch(const GroupedArgs& p, dim3 grid, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (in_dtype == SANDY_F32 && out_dtype == SANDY_F32) return launch<float, float>(p, grid, stream);
    if (in_dtype == SANDY_BF16 && out_dtype == SANDY_BF16) return launch<bf16, bf16>(p, grid, stream);
    if (in_dtype == SANDY_BF16 && out_dtype == SANDY_F32) return launch<bf16, float>(p, grid, stream);
    return SANDY_ERR_UNSUPPORTED;
}

}  // namespace

// Per head: a [rows, >= G * a_gcols] and w [G][N, K] (pitch ldw, w_gstride elements between groups) of in_dtype; out
// [rows, >= G * o_gcols] of out_dtype.
SANDY_API int sandy_head_product(const void* a, int lda, int a_gcols, const void* w, long long w_gstride, int ldw, void* out,
                                 int ldo, int o_gcols, int rows, int n_groups, int N, int K, int in_dtype, int out_dtype,
                                 cudaStream_t stream) {
    if (rows == 0 || n_groups == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out) return SANDY_ERR_ARGUMENT;
    if (n_groups > 65535 || (rows + TM - 1) / TM > 65535) return SANDY_ERR_UNSUPPORTED;
    GroupedArgs p = {a, lda, a_gcols, w, w_gstride, ldw, out, ldo, o_gcols, N, K, n_groups, rows, nullptr, nullptr, 1, 0};
    return dispatch(p, dim3((N + TN - 1) / TN, (rows + TM - 1) / TM, n_groups), in_dtype, out_dtype, stream);
}

// Per expert: `n_slots` bounds the slots (tokens x experts per token); group_start int32 [G + 1] on the device; a_row
// int32 [n_slots] or null; a slot reads row a_row[s] / a_row_div of a.  act: 0 none, 1 relu squared.
SANDY_API int sandy_expert_product(const void* a, int lda, const void* w, long long w_gstride, int ldw, void* out, int ldo,
                                   int n_slots, int n_groups, int N, int K, const int* group_start, const int* a_row,
                                   int a_row_div, int act, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (n_slots == 0 || n_groups == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || !group_start || a_row_div < 1) return SANDY_ERR_ARGUMENT;
    const int tiles = (n_slots + TM - 1) / TM + n_groups;
    if (tiles > 65535) return SANDY_ERR_UNSUPPORTED;
    GroupedArgs p = {a, lda, 0, w, w_gstride, ldw, out, ldo, 0, N, K, n_groups, 0, group_start, a_row, a_row_div, act};
    return dispatch(p, dim3((N + TN - 1) / TN, tiles, 1), in_dtype, out_dtype, stream);
}
