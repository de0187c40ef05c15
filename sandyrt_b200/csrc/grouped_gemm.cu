// Products with one small weight matrix per GROUP of rows or columns:
//
//   per head     out[t, g * o_gcols + n] = sum_k W_g[n, k] * a[t, g * a_gcols + k]        every group sees every row;
//                a head's slice of the columns goes through the head's own matrix (the up-projections of attention
//                over a latent: U_k,h^T on the queries, U_v,h on the weighted sums of latents)
//   per expert   out[s, n] = act(sum_k W_g[n, k] * a[row(s), k])  for the slots s of group g     a mixture of experts:
//                slots group_start[g] .. group_start[g+1]-1 belong to expert g (device data: the routing of this
//                step), a slot reads the row a_row[s] / a_row_div of `a` (or row s) and writes row s of `out`
//
// Both forms share their kernels: a block computes one tile of one group's output, every sum carried in 32-bit in
// a fixed order of k (so a row's result does not depend on which rows share its tile).  The weight is [N, K]
// row-major per group.  A grid of the per-expert form covers the worst case of tiles (slots / tile rows + groups)
// and blocks beyond the step's tiles leave at once, so a recorded launch serves every routing.
//
// Two kernels.  bfloat16 operands whose rows start on 16-byte boundaries go through tensor cores (mma.sync
// m16n8k16; tiles of 64 x 64, or 128 x 64 where the groups are long; operands staged by cp.async in a ring of
// stages and read with ldmatrix; rows a tile does not have are zero-filled, so a decode step's one or two rows per
// expert cost a tile's weight traffic and nothing else).  float32 operands and odd sizes take FFMA tiles.  Which kernel runs is a matter of the model's
// sizes alone, never of a step's rows.
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

// ---- tensor-core tiles (bfloat16) ---------------------------------------------------------------------------------
constexpr int MN = 64, MK = 32, MPITCH = MK + 8, MTHREADS = 128;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;               // 0: nothing is read and the 16 bytes become zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void store_pair(float* dst, float a, float b) { *reinterpret_cast<float2*>(dst) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* dst, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b); }

// MT: row tiles of 16 a warp owns (2: blocks of 64 rows behind a ring of four stages; 4: blocks of 128 rows, which
// feed twice the products from the same weight fragments, behind a ring of three).
template <typename TO, int MT>
__global__ void __launch_bounds__(MTHREADS) grouped_mma_kernel(GroupedArgs p) {
    constexpr int MM = 32 * MT, MSTAGES = MT == 2 ? 4 : 3;
    __shared__ __align__(16) bf16 sA[MSTAGES][MM][MPITCH];
    __shared__ __align__(16) bf16 sB[MSTAGES][MN][MPITCH];
    __shared__ int s_rows[MM];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    int g, row0, row_end;
    if (p.group_start) {
        int tile = blockIdx.y;
        g = 0;
        int start = p.group_start[0], end = start;
        for (; g < p.G; g++) {
            end = p.group_start[g + 1];
            const int tiles = (end - start + MM - 1) / MM;
            if (tile < tiles) break;
            tile -= tiles;
            start = end;
        }
        if (g >= p.G) return;
        row0 = start + tile * MM;
        row_end = end;
    } else {
        g = blockIdx.z;
        row0 = blockIdx.y * MM;
        row_end = p.rows;
    }
    const int n0 = blockIdx.x * MN;
    for (int i = tid; i < MM; i += MTHREADS) {
        const int s = row0 + i;
        int r = -1;
        if (s < row_end) r = p.a_row ? p.a_row[s] / p.a_row_div : s;
        s_rows[i] = r;
    }
    __syncthreads();
    const bf16* A = (const bf16*)p.a + (size_t)g * p.a_gcols;
    const bf16* W = (const bf16*)p.w + (size_t)g * p.w_gstride;
    // a stage: rows x 4 pieces of 8 for each operand
    auto load_stage = [&](int stage, int k0) {
#pragma unroll
        for (int i = 0; i < MM * 4 / MTHREADS; i++) {
            const int c = tid + i * MTHREADS, r = c >> 2, kc = (c & 3) * 8;
            const int ar = s_rows[r];
            const bool va = ar >= 0 && k0 + kc < p.K;
            cp_async_16(&sA[stage][r][kc], va ? (const void*)(A + (size_t)ar * p.lda + k0 + kc) : (const void*)A, va);
        }
#pragma unroll
        for (int i = 0; i < MN * 4 / MTHREADS; i++) {
            const int c = tid + i * MTHREADS, r = c >> 2, kc = (c & 3) * 8;
            const int n = n0 + r;
            const bool vb = n < p.N && k0 + kc < p.K;
            cp_async_16(&sB[stage][r][kc], vb ? (const void*)(W + (size_t)n * p.ldw + k0 + kc) : (const void*)W, vb);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_k = (p.K + MK - 1) / MK;
#pragma unroll
    for (int s = 0; s < MSTAGES - 1; s++) {
        if (s < n_k) load_stage(s, s * MK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 1) * (16 * MT), wn = (warp & 1) * 32;
    float acc[MT][4][4] = {};
    for (int kt = 0; kt < n_k; kt++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MSTAGES - 2) : "memory");
        __syncthreads();                             // stage kt has landed for everyone, stage kt - 1 has been read by everyone
        if (kt + MSTAGES - 1 < n_k) load_stage((kt + MSTAGES - 1) % MSTAGES, (kt + MSTAGES - 1) * MK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = kt % MSTAGES;
#pragma unroll
        for (int kk = 0; kk < MK; kk += 16) {
            unsigned a[MT][4], b[2][4];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                ldmatrix_x4(a[mt], &sA[st][wm + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < 2; np++)
                ldmatrix_x4(b[np], &sB[st][wn + np * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nt = 0; nt < 4; nt++) mma_bf16(acc[mt][nt], a[mt], b[nt >> 1][(nt & 1) * 2], b[nt >> 1][(nt & 1) * 2 + 1]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    TO* O = (TO*)p.out + (size_t)g * p.o_gcols;
    const int gq = lane >> 2, tq = lane & 3;
    // a thread holds pairs of neighbouring columns: one store a pair where every pair starts on a pair's boundary
    const bool pairs = !(p.ldo & 1) && !(p.o_gcols & 1) && !((uintptr_t)p.out % (2 * sizeof(TO)));
    auto finish = [&](float v) {
        if (p.act == 1) {
            v = fmaxf(v, 0.0f);
            v = v * v;
        }
        return v;
    };
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int s = row0 + wm + mt * 16 + gq + half * 8;
            if (s >= row_end) continue;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int n = n0 + wn + nt * 8 + tq * 2;
                const float v0 = finish(acc[mt][nt][half * 2]), v1 = finish(acc[mt][nt][half * 2 + 1]);
                TO* dst = O + (size_t)s * p.ldo + n;
                if (pairs && n + 1 < p.N) {
                    store_pair(dst, v0, v1);
                } else {
                    if (n < p.N) dst[0] = from_f32<TO>(v0);
                    if (n + 1 < p.N) dst[1] = from_f32<TO>(v1);
                }
            }
        }
}

// Whether the tensor-core kernel can take a problem: every row piece a cp.async fetches starts on a 16-byte boundary.
bool mma_takes(const GroupedArgs& p) {
    return p.K % 8 == 0 && p.lda % 8 == 0 && p.ldw % 8 == 0 && p.a_gcols % 8 == 0 && p.w_gstride % 8 == 0 &&
           !((uintptr_t)p.a & 15) && !((uintptr_t)p.w & 15);
}

template <typename TA, typename TO>
int launch(const GroupedArgs& p, dim3 grid, cudaStream_t stream) {
    return sandy_launch(grouped_tile_kernel<TA, TO>, grid, dim3(THREADS), 0, stream, p);
}

// `row_tiles(tile rows)` gives the grid's second dimension for a kernel's tile height.
template <typename F>
int dispatch(const GroupedArgs& p, F row_tiles, int groups_z, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (in_dtype == SANDY_BF16 && mma_takes(p)) {
        // Blocks of 128 rows where the groups are long (a prompt step), of 64 otherwise.  Both add an element's
        // products in the same order, so the choice never changes a result.
        const bool tall = row_tiles(1) / (p.group_start ? p.G : 1) >= 96;
        const dim3 grid((p.N + MN - 1) / MN, row_tiles(tall ? 128 : 64), groups_z);
        if (grid.y > 65535) return SANDY_ERR_UNSUPPORTED;
        if (out_dtype == SANDY_BF16)
            return tall ? sandy_launch(grouped_mma_kernel<bf16, 4>, grid, dim3(MTHREADS), 0, stream, p)
                        : sandy_launch(grouped_mma_kernel<bf16, 2>, grid, dim3(MTHREADS), 0, stream, p);
        if (out_dtype == SANDY_F32)
            return tall ? sandy_launch(grouped_mma_kernel<float, 4>, grid, dim3(MTHREADS), 0, stream, p)
                        : sandy_launch(grouped_mma_kernel<float, 2>, grid, dim3(MTHREADS), 0, stream, p);
        return SANDY_ERR_UNSUPPORTED;
    }
    const dim3 grid((p.N + TN - 1) / TN, row_tiles(TM), groups_z);
    if (grid.y > 65535) return SANDY_ERR_UNSUPPORTED;
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
    if (n_groups > 65535) return SANDY_ERR_UNSUPPORTED;
    GroupedArgs p = {a, lda, a_gcols, w, w_gstride, ldw, out, ldo, o_gcols, N, K, n_groups, rows, nullptr, nullptr, 1, 0};
    return dispatch(p, [&](int tile) { return (rows + tile - 1) / tile; }, n_groups, in_dtype, out_dtype, stream);
}

// Per expert: `n_slots` bounds the slots (tokens x experts per token); group_start int32 [G + 1] on the device; a_row
// int32 [n_slots] or null; a slot reads row a_row[s] / a_row_div of a.  act: 0 none, 1 relu squared.
SANDY_API int sandy_expert_product(const void* a, int lda, const void* w, long long w_gstride, int ldw, void* out, int ldo,
                                   int n_slots, int n_groups, int N, int K, const int* group_start, const int* a_row,
                                   int a_row_div, int act, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (n_slots == 0 || n_groups == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || !group_start || a_row_div < 1) return SANDY_ERR_ARGUMENT;
    GroupedArgs p = {a, lda, 0, w, w_gstride, ldw, out, ldo, 0, N, K, n_groups, 0, group_start, a_row, a_row_div, act};
    // the worst case of tiles: every group's last tile partly filled
    return dispatch(p, [&](int tile) { return (n_slots + tile - 1) / tile + n_groups; }, 1, in_dtype, out_dtype, stream);
}
