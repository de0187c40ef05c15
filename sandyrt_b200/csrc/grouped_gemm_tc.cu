// The product with one matrix per expert on the 5th-generation tensor cores (tcgen05), for steps with many rows:
//
//   out[s, n] = act( sum_k a[s, k] * w[g * N + n, k] )      for the slots s of group g, group_start[g] <= s < group_start[g+1]
//
// a: [slots, K] bfloat16 with the rows of a group one after another (the routing's sorted order; the caller gathers
// them there), w: [G * N, K] bfloat16, out bfloat16 or float.  The groups' borders are device data, so a recorded
// launch serves every routing: the grid covers the worst case of tiles (slots / 128 + groups), every block finds its
// group and its first row by walking group_start, and blocks beyond the step's tiles leave at once.
//
// A block computes one 128 x BN tile as csrc/gemm_tc.cu does: one lane issues the TMA loads of the A tile (rows row0 ..
// row0 + 127 of a, wherever a group starts: TMA's row coordinate has no alignment rule) and of the W tile (rows g * N +
// n0 ..) into a ring of stages, one lane issues tcgen05.mma into tensor memory, four warps read the accumulator with
// tcgen05.ld and store from their registers.  A tile's rows behind its group's end hold the next group's rows times
// this group's matrix: they are computed and not stored; the same goes for columns behind N (the next expert's rows of
// w).  For a given output element the k-steps are added in ascending order, so a row's result depends on nothing else
// in the step.  Every wait on an mbarrier is bounded: on expiry the kernel raises `*status`, stops issuing, frees its
// tensor memory and returns.
#include "tcgen05.cuh"

namespace {

constexpr int NUM_THREADS = 192;

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct GroupTile { int g, row0, row_end; };

// The group and the first row of a block's tile; g < 0 if the step has fewer tiles.
__device__ __forceinline__ GroupTile find_tile(const int* __restrict__ group_start, int G, int tile) {
    int start = group_start[0];
    for (int g = 0; g < G; g++) {
        const int end = group_start[g + 1];
        const int tiles = (end - start + BM - 1) / BM;
        if (tile < tiles) return {g, start + tile * BM, end};
        tile -= tiles;
        start = end;
    }
    return {-1, 0, 0};
}

template <int BN, int STAGES, int ACT>
__global__ void __launch_bounds__(NUM_THREADS, 2)
grouped_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, EpilogueArgs ep,
                  const int* __restrict__ group_start, int G, int N, int K, int* __restrict__ status) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_base = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    const int k_tiles = (K + BK - 1) / BK;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    // Every role finds the tile itself, after its own wait for the kernel before (which wrote group_start): the
    // three agree, so a block without a tile issues nothing and waits for nothing.
    if (warp == 0) {
        if (elect_one()) {
            pdl_wait();
            const GroupTile t = find_tile(group_start, G, blockIdx.y);
            for (int kt = 0; kt < k_tiles && t.g >= 0; kt++) {
                const int s = kt % STAGES;
                const uint32_t round = kt / STAGES;
                if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1)) {
                    if (status) atomicOr(status, 1);
                    break;
                }
                uint8_t* sa = stage_base + s * L::STAGE_BYTES;
                uint8_t* sb = sa + L::A_BYTES;
                mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                tma_load_2d(sa, &map_a, kt * BK, t.row0, &full_bar[s]);
                tma_load_2d(sb, &map_w, kt * BK, t.g * N + n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            pdl_wait();
            const GroupTile t = find_tile(group_start, G, blockIdx.y);
            if (t.g >= 0) {
                constexpr uint32_t idesc = make_instr_desc(BN);
                bool ok = true;
                for (int kt = 0; kt < k_tiles && ok; kt++) {
                    const int s = kt % STAGES;
                    const uint32_t round = kt / STAGES;
                    if (!mbar_wait(&full_bar[s], round & 1)) {
                        if (status) atomicOr(status, 2);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stage_base + s * L::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + L::A_BYTES;
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                umma_commit(accum_bar);
            }
        }
    } else {
        const int quarter = warp & 3;
        float bias[BN / 32];
        load_bias(bias, ep, n0, N);
        pdl_wait();
        const GroupTile t = find_tile(group_start, G, blockIdx.y);
        if (t.g >= 0) {
            const bool ready = mbar_wait(accum_bar, 0);
            if (!ready && lane == 0 && status) atomicOr(status, 4);
            tc_fence_after();
            if (ready)      // rows are clipped at the group's end, columns at N; stores from the registers
                write_back_warp_as<BN / 32, 2, ACT, false>(tmem_base + ((uint32_t)(quarter * 32) << 16), stage_base,
                                                           t.row0 + quarter * 32, n0, ep, nullptr, t.row_end, N, -1, 0, status, bias, [] {});
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

template <int BN, int STAGES, int ACT>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, const EpilogueArgs& ep, const int* group_start, int G, int n_slots, int N,
           int K, int* status, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(grouped_tc_kernel<BN, STAGES, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = (n_slots + BM - 1) / BM + G;
    if (tiles > 65535) return SANDY_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, tiles);
    return sandy_launch(grouped_tc_kernel<BN, STAGES, ACT>, grid, dim3(NUM_THREADS), L::TOTAL, stream, ma, mw, ep, group_start, G, N, K,
                        status);
}

template <int ACT>
int launch_width(const CUtensorMap& ma, const void* w, int ldw, const EpilogueArgs& ep, const int* group_start, int G, int n_slots,
                 int N, int K, int* status, cudaStream_t stream) {
    CUtensorMap mw;
    const int bn = N >= 128 ? 128 : 64;
    if (!get_map(w, (long long)G * N, K, ldw, bn, &mw)) return SANDY_ERR_UNSUPPORTED;
    if (bn == 128) return launch<128, 3, ACT>(ma, mw, ep, group_start, G, n_slots, N, K, status, stream);
    return launch<64, 4, ACT>(ma, mw, ep, group_start, G, n_slots, N, K, status, stream);
}

}  // namespace

// a: bfloat16 [n_slots, K] (pitch lda), rows sorted by group; w: bfloat16 [n_groups * N, K] (pitch ldw); out: [n_slots, N]
// (pitch ldo) of out_dtype; group_start: int32 [n_groups + 1] on the device.  act: 0 none, 1 relu squared.  Pitches of a
// and w multiples of 8 elements, both 16-byte aligned.
SANDY_API int sandy_expert_product_tc(const void* a, int lda, const void* w, int ldw, void* out, int ldo, int n_slots,
                                      int n_groups, int N, int K, const int* group_start, int act, int out_dtype, int* status,
                                      cudaStream_t stream) {
    if (n_slots == 0 || n_groups == 0 || N == 0) return SANDY_OK;
    if (!a || !w || !out || !group_start || K <= 0) return SANDY_ERR_ARGUMENT;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return SANDY_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return SANDY_ERR_UNSUPPORTED;
    if (out_dtype != SANDY_F32 && out_dtype != SANDY_BF16) return SANDY_ERR_UNSUPPORTED;
    CUtensorMap ma;
    if (!get_map(a, n_slots, K, lda, BM, &ma)) return SANDY_ERR_UNSUPPORTED;
    KVWrite kv{};
    EpilogueArgs ep{nullptr, nullptr, out, 0, ldo, act == 1 ? SANDY_ACT_RELU_SQUARED : SANDY_ACT_NONE, out_dtype == SANDY_F32 ? 1 : 0, kv, 0};
    if (act == 1) return launch_width<SANDY_ACT_RELU_SQUARED>(ma, w, ldw, ep, group_start, n_groups, n_slots, N, K, status, stream);
    if (act == 0) return launch_width<SANDY_ACT_NONE>(ma, w, ldw, ep, group_start, n_groups, n_slots, N, K, status, stream);
    return SANDY_ERR_UNSUPPORTED;
}
