// SPDX-License-Identifier: Apache-2.0
// bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with fp32 accumulators in TMEM,
// persistent warp-specialised CTAs (one per SM) and a double-buffered accumulator so that the epilogue
// of tile i overlaps the main loop of tile i+1.
//
//   C[M, N] = op(A) * op(B)^T      A: [M, K] (K contiguous) or [K, M] (M contiguous, "MN-major")
//                                  B: [N, K] (K contiguous) or [K, N] (N contiguous, "MN-major")
//
// so one kernel serves the forward (x W^T), the data gradient (dY W) and the weight gradient (dY^T X)
// of a linear layer.  Epilogues: plain store, accumulate into C, SwiGLU on block-interleaved gate/up
// columns (64 gate columns followed by their 64 up columns).
//
// Roles inside a CTA of 192 threads: warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer
// (one elected lane; also owns TMEM allocation), warps 2..5 = epilogue (TMEM -> registers -> global).
// Every barrier wait is bounded; on a timeout the CTA records an error code, drains, frees TMEM and
// returns, so a logic error can not hang the device.
//
// The reference has no GEMM of its own: dense layers go to cuBLAS through nn.Linear and the grouped
// expert GEMM is a Triton kernel (arctic_training/model/moe/moe_gemm.py:36-166).

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>

namespace atb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
constexpr int kMaxGroups = 1024;

enum Epilogue : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_PUSH_HEADS = 3 };

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOffset = STAGES * kStageBytes;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem slot, abort flag, group offsets
    static constexpr int kOffsetsOffset = kBarrierOffset + (2 * STAGES + 4) * 8 + 16;
    static constexpr int kTotal = kOffsetsOffset + (kMaxGroups + 1) * 4;
};

enum GroupMode : int { GROUP_NONE = 0, GROUP_RAGGED_M = 1, GROUP_RAGGED_K = 2 };

struct GemmParams {
    bf16* C;
    const bf16* R;  // EPI_ACCUM: C = A B + R (R may be C itself: in-place accumulation, or a residual stream)
    int M, N, K;  // per-group extents in the grouped modes (M is unused for GROUP_RAGGED_M)
    int64_t ldc, ldr;
    int* error_flag;  // device int: 0 ok, otherwise (role << 8) | reason
    // grouped GEMM: `group_offsets[g]` is the first row of group g in the ragged operand(s); every group
    // starts at a multiple of 128 rows.  GROUP_RAGGED_M: A rows are ragged, B holds one matrix per group.
    // GROUP_RAGGED_K: the contraction runs over the rows of group g; C holds one [M, N] block per group.
    const int* group_offsets;
    int num_groups;
    int group_mode;
    // A operand assembled from several tensors along K (CTA-pair kernel, K-major A): k in [j * a_seg_len, (j + 1) *
    // a_seg_len) comes from tensor map j of `SegMaps`, rows a_seg_row0 + m.  0 = A is the single tensor of tmap_a.
    int a_seg_len;
    int a_seg_row0;
    // Staged gather of A (CTA-pair kernel): the last `stage_ctas` CTAs of the grid do not compute; they copy the K
    // segments of A from `stage_src[j]` (peer memory) into the local matrix that tmap_a describes and count finished
    // segments per 256-row tile in `stage_flags`; a computing pair starts a tile once its rows have all arrived.
    int stage_ctas;
    int stage_segs;
    // stage_mode 0: gather of A as described above.  stage_mode 1: gather of B (a weight [N, K] stored K-major inside a
    // flat parameter buffer that is sharded contiguously over the ranks, `stage_shard_elems` elements each): the
    // staging CTAs copy the element range [stage_flat_off + 256 n K, +256 K) of N tile n from the shards that hold it
    // (stage_src[p] = rank p's shard) into the local full buffer `stage_dst` and then count the tile in
    // stage_flags[n]; a computing pair starts a tile once the rows of its B tile have arrived.
    int stage_mode;
    int64_t stage_flat_off;
    int64_t stage_shard_elems;
    const bf16* stage_src[8];
    int64_t stage_src_ld;
    bf16* stage_dst;
    int64_t stage_dst_ld;
    int* stage_flags;
    // EPI_PUSH_HEADS (CTA-pair kernel): the output is a fused q|k|v projection [rows, (Hq + 2 Hkv) D] that is not
    // stored here: every 32-column piece goes to the rank that owns its head, into that rank's buffer
    // [P * rows_per_rank, Hlq + 2 Hlkv, D] at row push_rank * rows_per_rank + row (sequence -> head exchange of Ulysses
    // done by the epilogue stores).  KV heads are replicated when there are fewer of them than ranks.
    bf16* push_dst[8];
    int push_ranks, push_rank, push_hq, push_hkv, push_d, push_rows;
    // Cache behaviour of the CTA-pair kernel (bit 0: the epilogue writes the output with streaming stores and reads
    // the accumulate operand with streaming loads; bit 1: operand tiles are loaded with an evict-last L2 policy).
    int cache_flags;
};

constexpr int kMaxSegs = 8;
// Tensor maps of the K segments of A.  They may describe other GPUs' memory (peer mappings): the loads are plain
// per-CTA-pair TMA tile loads, each tile is fetched by the one pair that needs it.
struct SegMaps {
    CUtensorMap m[kMaxSegs];
};

// What one output tile reads and writes.
struct TileInfo {
    int a_m0, a_k0;  // A: first M coordinate and first contraction coordinate
    int b_n0, b_k0;  // B: first N coordinate and first contraction coordinate
    int k_blocks;
    int c_row0, c_row_limit, c_col0;
};


template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024 bytes that the
    // 128-byte swizzle pattern needs (the launch reserves the slack).
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    int* s_offsets = reinterpret_cast<int*>(smem + L::kOffsetsOffset);
    constexpr int GROUP_M = 8;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // 512 for BN=256, 256 for BN=128

    if (p.group_mode != GROUP_NONE) {
        for (int g = threadIdx.x; g <= p.num_groups; g += blockDim.x) s_offsets[g] = p.group_offsets[g];
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_rows = p.group_mode == GROUP_NONE ? p.M : s_offsets[p.num_groups];
    const int tiles_m = p.group_mode == GROUP_RAGGED_K ? (p.M + BM - 1) / BM : (total_rows + BM - 1) / BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int tiles_per_group = tiles_m * tiles_n;  // GROUP_RAGGED_K only
    const int num_tiles = p.group_mode == GROUP_RAGGED_K ? tiles_per_group * p.num_groups : tiles_m * tiles_n;

    // Maps a linear tile index to its coordinates; returns false for tiles that have no work (empty group).
    auto get_tile = [&](int t, TileInfo& ti) -> bool {
        if (p.group_mode == GROUP_RAGGED_K) {
            const int g = t / tiles_per_group;
            const int r = t - g * tiles_per_group;
            const int tm = r % tiles_m, tn = r / tiles_m;
            const int row0 = s_offsets[g], rows = s_offsets[g + 1] - row0;
            if (rows <= 0) return false;
            ti.a_m0 = tm * BM; ti.a_k0 = row0; ti.b_n0 = tn * BN; ti.b_k0 = row0;
            ti.k_blocks = (rows + BK - 1) / BK;
            ti.c_row0 = g * p.M + tm * BM; ti.c_row_limit = g * p.M + p.M; ti.c_col0 = tn * BN;
            return true;
        }
        const int per_group = GROUP_M * tiles_n;
        const int grp = t / per_group;
        const int first_m = grp * GROUP_M;
        const int gsz = min(GROUP_M, tiles_m - first_m);
        const int r = t - grp * per_group;
        const int tm = first_m + (r % gsz), tn = r / gsz;
        ti.a_m0 = tm * BM; ti.a_k0 = 0; ti.b_n0 = tn * BN; ti.b_k0 = 0;
        ti.k_blocks = (p.K + BK - 1) / BK;
        ti.c_row0 = tm * BM; ti.c_row_limit = total_rows; ti.c_col0 = tn * BN;
        if (p.group_mode == GROUP_RAGGED_M) {
            // binary search for the group that owns row tm * BM (segments are tile aligned)
            int lo = 0, hi = p.num_groups - 1;
            const int row = tm * BM;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_offsets[mid] <= row) lo = mid; else hi = mid - 1;
            }
            if constexpr (B_MN) ti.b_k0 = lo * p.K; else ti.b_n0 = lo * p.N + tn * BN;
        }
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::tma_prefetch_desc(&tmap_a);
            ptx::tma_prefetch_desc(&tmap_b);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                TileInfo ti;
                if (!get_tile(t, ti)) continue;
                for (int kb = 0; kb < ti.k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, kWaitLimitNs)) {
                        atomicCAS(p.error_flag, 0, (1 << 8) | 1);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * L::kStageBytes;
                    uint8_t* sb = sa + L::kABytes;
                    ptx::mbar_expect_tx(&full_bar[stage], L::kStageBytes);
                    if constexpr (!A_MN) {
                        ptx::tma_load_2d(sa, &tmap_a, ti.a_k0 + kb * BK, ti.a_m0, &full_bar[stage]);
                    } else {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            ptx::tma_load_2d(sa + c * (BK * 128), &tmap_a, ti.a_m0 + c * 64, ti.a_k0 + kb * BK,
                                             &full_bar[stage]);
                    }
                    if constexpr (!B_MN) {
                        ptx::tma_load_2d(sb, &tmap_b, ti.b_k0 + kb * BK, ti.b_n0, &full_bar[stage]);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            ptx::tma_load_2d(sb + c * (BK * 128), &tmap_b, ti.b_n0 + c * 64, ti.b_k0 + kb * BK,
                                             &full_bar[stage]);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: wait for them (bounded)
                // before the CTA is allowed to retire.
                for (int s = 0; s < STAGES; ++s) {
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(&full_bar[s], 0) && !ptx::mbar_try_wait(&full_bar[s], 1)) {
                        if (ptx::globaltimer_ns() - t0 > 100000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(BM, BN, A_MN, B_MN);
            // K-major operand: rows of 128 bytes, 8-row groups 1024 bytes apart; one UMMA_K step = 32 bytes.
            // MN-major operand: chunks of 64 (MN) x BK (K) elements, 128 bytes per K row, 8-K groups 1024
            // bytes apart, chunks BK*128 bytes apart; one UMMA_K step = 16 rows = 2048 bytes.
            constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, B_LBO = B_MN ? BK * 128 : 16;
            constexpr uint32_t A_KSTEP = A_MN ? UMMA_K * 128 : UMMA_K * 2, B_KSTEP = B_MN ? UMMA_K * 128 : UMMA_K * 2;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                TileInfo ti;
                if (!get_tile(t, ti)) continue;
                const int k_blocks = ti.k_blocks;
                const int acc = it & 1;
                ++it;
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase[acc] ^ 1u, abort_flag, kWaitLimitNs)) {
                    atomicCAS(p.error_flag, 0, (2 << 8) | 1);
                    ok = false;
                    break;
                }
                acc_phase[acc] ^= 1u;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag, kWaitLimitNs)) {
                        atomicCAS(p.error_flag, 0, (2 << 8) | 2);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + stage * L::kStageBytes);
                    const uint32_t sb = sa + L::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = ptx::make_smem_desc_sw128(sa + k * A_KSTEP, A_LBO, 1024);
                        const uint64_t db = ptx::make_smem_desc_sw128(sb + k * B_KSTEP, B_LBO, 1024);
                        ptx::mma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::mma_commit(&empty_bar[stage]);  // releases the smem slot once these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::mma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) are visible to this warp
        uint32_t acc_phase[2] = {0, 0};
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile(t, ti)) continue;
            const int acc = it & 1;
            ++it;
            if (!ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase[acc], abort_flag, kWaitLimitNs)) {
                if (lane == 0) atomicCAS(p.error_flag, 0, (3 << 8) | 1);
                ok = false;
                break;
            }
            acc_phase[acc] ^= 1u;
            ptx::tc_fence_after();
            const int row = ti.c_row0 + quarter * 32 + lane;
            const bool row_ok = row < ti.c_row_limit;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            if constexpr (EPI == EPI_SWIGLU) {
                // columns [128g, 128g+64) gate, [128g+64, 128g+128) up  ->  output columns [64g, 64g+64)
                bf16* crow = p.C + (int64_t)row * p.ldc + (int64_t)(ti.c_col0 / 2);
#pragma unroll 1
                for (int g = 0; g < BN / 128; ++g) {
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        uint32_t rg[32], ru[32];
                        ptx::tmem_ld_32x32b_x32(taddr + g * 128 + h * 32, rg);
                        ptx::tmem_ld_32x32b_x32(taddr + g * 128 + 64 + h * 32, ru);
                        ptx::tmem_ld_wait();
                        const int col0 = ti.c_col0 / 2 + g * 64 + h * 32;
                        if (row_ok && col0 < p.N / 2) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                float o[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const float gg = __uint_as_float(rg[v * 8 + j]);
                                    const float uu = __uint_as_float(ru[v * 8 + j]);
                                    o[j] = gg / (1.f + __expf(-gg)) * uu;
                                }
                                *reinterpret_cast<bf16x8*>(crow + g * 64 + h * 32 + v * 8) = pack8(o);
                            }
                        }
                    }
                }
            } else {
                bf16* crow = p.C + (int64_t)row * p.ldc + (int64_t)ti.c_col0;
                const bf16* rrow = p.R + (int64_t)row * p.ldr + (int64_t)ti.c_col0;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                    ptx::tmem_ld_wait();
                    const int col0 = ti.c_col0 + c * 32;
                    if (row_ok) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col0 + v * 8 < p.N) {  // N is a multiple of 8 (checked on the host)
                                float o[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(r[v * 8 + j]);
                                bf16x8* dst = reinterpret_cast<bf16x8*>(crow + c * 32 + v * 8);
                                if constexpr (EPI == EPI_ACCUM) {
                                    float old[8];
                                    unpack8(*reinterpret_cast<const bf16x8*>(rrow + c * 32 + v * 8), old);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) o[j] += old[j];
                                }
                                *dst = pack8(o);
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
        }
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- CTA-pair variant ---------------------------------------------------------------------------------
// One 256 x 256 output tile per cluster of two CTAs (`tcgen05.mma.cta_group::2`).  Each CTA stages its own 128 rows
// of A and its own 128 rows of B (half of the N extent), so the shared-memory traffic per tensor-core cycle drops by a
// third compared with the single-CTA 128 x 256 tile; the leader CTA (cluster rank 0) issues the MMAs for both, each
// CTA keeps its 128 accumulator rows in its own TMEM and writes them out itself.  Dense GEMM only (no grouping).
//
// Barriers: `full[s]` lives in the leader and counts one expect-tx arrival per CTA plus the bytes of both CTAs'
// copies; `empty[s]` and `tmem_full[a]` exist in both CTAs and are signalled by the leader's commits (one commit per
// CTA, addressed through the cluster window); `tmem_empty[a]` lives in the leader and collects the arrivals of the
// eight epilogue warps of the pair.
template <int STAGES>
struct PairSmemLayout {
    static constexpr int kABytes = 128 * BK * 2;
    static constexpr int kBBytes = 128 * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOffset = STAGES * kStageBytes;
    static constexpr int kTotal = kBarrierOffset + (2 * STAGES + 4) * 8 + 16;
};

template <int STAGES, bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const GemmParams p, const __grid_constant__ SegMaps segs) {
    using L = PairSmemLayout<STAGES>;
    constexpr int TM = 256, TN = 256;  // tile of the pair
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();  // 0 = leader
    const bool leader = cta == 0;
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 2);   // one expect-tx arrival from each CTA of the pair (used in the leader)
            ptx::mbar_init(&empty_bar[s], 1);  // leader's commit
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 8);  // four epilogue warps in each CTA (used in the leader)
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // the peer's barriers are initialised before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + TM - 1) / TM;
    const int tiles_n = (p.N + TN - 1) / TN;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int cluster_id = blockIdx.x >> 1, num_clusters = (gridDim.x - p.stage_ctas) >> 1;
    const bool is_stager = cluster_id >= num_clusters;
    constexpr int GROUP_M = 8;
    auto tile_coords = [&](int t, int& tm, int& tn) {
        const int per_group = GROUP_M * tiles_n;
        const int g = t / per_group;
        const int first_m = g * GROUP_M;
        const int gsz = min(GROUP_M, tiles_m - first_m);
        const int r = t - g * per_group;
        tm = first_m + (r % gsz);
        tn = r / gsz;
    };

    if (is_stager) {
        // ------------------------------------------------------------------ gather of A from the peers
        // One thread streams the segments through this CTA's (otherwise idle) tile buffers with bulk copies: a chunk of
        // rows is contiguous at the owner, lands in shared memory, and is written row by row into the local matrix.
        // Several chunks are in flight; the only waits are on this CTA's own copies (bounded).
        if (threadIdx.x == 0 && p.stage_mode == 1) {
            // ---- gather of B: contiguous element ranges of the sharded flat buffer, 32 KB chunks through shared memory
            constexpr int NBUF = STAGES < 6 ? STAGES : 6;
            constexpr int LEAD = NBUF / 2;
            constexpr int64_t CHUNK = 16384;  // elements (32 KB)
            const int sidx = (int)blockIdx.x - 2 * num_clusters;
            uint32_t ph[NBUF];
            for (int i = 0; i < NBUF; ++i) ph[i] = 0;
            bool ok = true;
            const int64_t w_end = p.stage_flat_off + (int64_t)p.N * p.K;
            for (int nt = sidx; nt < tiles_n && ok; nt += p.stage_ctas) {
                const int64_t e0 = p.stage_flat_off + (int64_t)nt * TN * p.K;
                const int64_t e1 = min(e0 + (int64_t)TN * p.K, w_end);
                // a chunk never crosses a shard boundary: count the chunks of this tile first
                int n_chunks = 0;
                for (int64_t e = e0; e < e1; ++n_chunks) {
                    const int64_t off = e % p.stage_shard_elems;
                    e += min(min(CHUNK, e1 - e), p.stage_shard_elems - off);
                }
                int64_t load_e = e0, store_e = e0;
                int64_t lens[NBUF];
                // software pipeline: loads run LEAD chunks ahead of the stores; one bulk group is committed per step
                for (int c = 0; c < n_chunks + LEAD && ok; ++c) {
                    if (c < n_chunks) {
                        const int b = c % NBUF;
                        ptx::bulk_wait_read<NBUF - LEAD - 1>();  // the stores that last read buffer b have drained it
                        const int64_t owner = load_e / p.stage_shard_elems;
                        const int64_t off = load_e - owner * p.stage_shard_elems;
                        const int64_t len = min(min(CHUNK, e1 - load_e), p.stage_shard_elems - off);
                        lens[b] = len;
                        ptx::mbar_expect_tx(&empty_bar[b], (uint32_t)(len * 2));
                        ptx::bulk_load(smem + b * 32768, p.stage_src[owner] + off, (uint32_t)(len * 2), &empty_bar[b]);
                        load_e += len;
                    }
                    const int d = c - LEAD;
                    if (d >= 0) {
                        const int b = d % NBUF;
                        if (!ptx::mbar_wait_bounded(&empty_bar[b], ph[b], abort_flag, kWaitLimitNs)) {
                            atomicCAS(p.error_flag, 0, (0x16 << 8) | 1);
                            ok = false;
                            break;
                        }
                        ph[b] ^= 1u;
                        ptx::bulk_store(p.stage_dst + store_e, smem + b * 32768, (uint32_t)(lens[b] * 2));
                        store_e += lens[b];
                    }
                    ptx::bulk_commit();
                }
                ptx::bulk_wait<0>();  // the rows of this tile are written
                ptx::fence_proxy_async_all();
                __threadfence();
                if (ok) atomicAdd(&p.stage_flags[nt], 1);
            }
            ptx::bulk_wait<0>();
        } else if (threadIdx.x == 0) {
            constexpr int NBUF = STAGES < 6 ? STAGES : 6;
            constexpr uint32_t BUF_BYTES = 32768;
            const int sidx = (int)blockIdx.x - 2 * num_clusters;
            const int P = p.stage_segs;
            const uint32_t seg_bytes = (uint32_t)p.a_seg_len * 2;
            const int rows_per_chunk = max(1, (int)(BUF_BYTES / seg_bytes));
            uint32_t ph[NBUF];
            for (int i = 0; i < NBUF; ++i) ph[i] = 0;
            bool ok = true;
            for (int item = sidx; item < tiles_m * P && ok; item += p.stage_ctas) {
                const int mt = item / P;
                const int j = (item - mt * P + mt) % P;  // consecutive tiles start at different peers
                const int r0 = mt * TM, nrows = min(TM, p.M - r0);
                const uint8_t* src = reinterpret_cast<const uint8_t*>(p.stage_src[j] + (int64_t)(p.a_seg_row0 + r0) * p.stage_src_ld);
                bf16* dst = p.stage_dst + (int64_t)r0 * p.stage_dst_ld + (int64_t)j * p.a_seg_len;
                const int nchunks = (nrows + rows_per_chunk - 1) / rows_per_chunk;
                // software pipeline: loads run LEAD chunks ahead of the stores; one bulk group is committed per step
                constexpr int LEAD = NBUF / 2;
                for (int c = 0; c < nchunks + LEAD && ok; ++c) {
                    if (c < nchunks) {
                        const int b = c % NBUF;
                        // buffer b was last read by the stores of chunk c - NBUF, committed at step c - NBUF + LEAD:
                        // NBUF - LEAD - 1 groups have been committed since
                        ptx::bulk_wait_read<NBUF - LEAD - 1>();
                        const int rows = min(rows_per_chunk, nrows - c * rows_per_chunk);
                        const uint32_t bytes = (uint32_t)rows * seg_bytes;
                        ptx::mbar_expect_tx(&empty_bar[b], bytes);
                        ptx::bulk_load(smem + b * BUF_BYTES, src + (int64_t)c * rows_per_chunk * seg_bytes, bytes, &empty_bar[b]);
                    }
                    const int d = c - LEAD;
                    if (d >= 0) {
                        const int b = d % NBUF;
                        if (!ptx::mbar_wait_bounded(&empty_bar[b], ph[b], abort_flag, kWaitLimitNs)) {
                            atomicCAS(p.error_flag, 0, (0x15 << 8) | 1);
                            ok = false;
                            break;
                        }
                        ph[b] ^= 1u;
                        const int rows = min(rows_per_chunk, nrows - d * rows_per_chunk);
                        for (int rr = 0; rr < rows; ++rr)
                            ptx::bulk_store(dst + (int64_t)(d * rows_per_chunk + rr) * p.stage_dst_ld,
                                            smem + b * BUF_BYTES + rr * seg_bytes, seg_bytes);
                    }
                    ptx::bulk_commit();  // one group per step (possibly empty) keeps the wait arithmetic uniform
                }
                ptx::bulk_wait<0>();      // the rows of this item are written
                ptx::fence_proxy_async_all();
                __threadfence();
                atomicAdd(&p.stage_flags[mt], 1);
            }
            ptx::bulk_wait<0>();
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (in both CTAs)
        if (lane == 0) {
            ptx::tma_prefetch_desc(&tmap_a);
            ptx::tma_prefetch_desc(&tmap_b);
            const bool keep_operands = (p.cache_flags & 2) != 0;
            const uint64_t keep_policy = keep_operands ? ptx::make_l2_policy_evict_last() : 0;
            auto load = [&](void* dst, const CUtensorMap* tm_, int x, int y, uint64_t* bar) {
                if (keep_operands) ptx::tma_load_2d_pair_hint(dst, tm_, x, y, bar, keep_policy);
                else ptx::tma_load_2d_pair(dst, tm_, x, y, bar);
            };
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                int tm, tn;
                tile_coords(t, tm, tn);
                const int a_m0 = tm * TM + (int)cta * 128, b_n0 = tn * TN + (int)cta * 128;
                if (p.stage_ctas > 0) {
                    // rows of this tile (of A, or of B in mode 1) are being gathered by the staging CTAs: wait (bounded)
                    // until they have all landed
                    const uint64_t t0 = ptx::globaltimer_ns();
                    const int fidx = p.stage_mode == 1 ? tn : tm;
                    while (ptx::ld_acquire_gpu(reinterpret_cast<const uint32_t*>(p.stage_flags) + fidx) < (uint32_t)p.stage_segs) {
                        if (*abort_flag || ptx::globaltimer_ns() - t0 > kWaitLimitNs) {
                            *abort_flag = 1;
                            atomicCAS(p.error_flag, 0, (0x14 << 8) | 1);
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                    ptx::fence_proxy_async_all();  // the gathered rows were written with ordinary stores; TMA reads them next
                }
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, kWaitLimitNs)) {
                        atomicCAS(p.error_flag, 0, (0x11 << 8) | 1);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * L::kStageBytes;
                    uint8_t* sb = sa + L::kABytes;
                    ptx::mbar_expect_tx_cluster(ptx::mapa_shared(ptx::smem_u32(&full_bar[stage]), 0), L::kStageBytes);
                    if constexpr (!A_MN) {
                        if (p.a_seg_len > 0 && p.stage_ctas == 0) {
                            const int seg = (kb * BK) / p.a_seg_len;
                            ptx::tma_load_2d_pair(sa, &segs.m[seg], kb * BK - seg * p.a_seg_len, p.a_seg_row0 + a_m0,
                                                  &full_bar[stage]);
                        } else {
                            load(sa, &tmap_a, kb * BK, a_m0, &full_bar[stage]);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 2; ++c)
                            load(sa + c * (BK * 128), &tmap_a, a_m0 + c * 64, kb * BK, &full_bar[stage]);
                    }
                    if constexpr (!B_MN) {
                        load(sb, &tmap_b, kb * BK, b_n0, &full_bar[stage]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 2; ++c)
                            load(sb + c * (BK * 128), &tmap_b, b_n0 + c * 64, kb * BK, &full_bar[stage]);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(TM, TN, A_MN, B_MN);
            constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, B_LBO = B_MN ? BK * 128 : 16;
            constexpr uint32_t A_KSTEP = A_MN ? UMMA_K * 128 : UMMA_K * 2, B_KSTEP = B_MN ? UMMA_K * 128 : UMMA_K * 2;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int it = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
                const int acc = it & 1;
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase[acc] ^ 1u, abort_flag, kWaitLimitNs)) {
                    atomicCAS(p.error_flag, 0, (0x12 << 8) | 1);
                    ok = false;
                    break;
                }
                acc_phase[acc] ^= 1u;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag, kWaitLimitNs)) {
                        atomicCAS(p.error_flag, 0, (0x12 << 8) | 2);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = ptx::smem_u32(smem + stage * L::kStageBytes);
                    const uint32_t sb = sa + L::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = ptx::make_smem_desc_sw128(sa + k * A_KSTEP, A_LBO, 1024);
                        const uint64_t db = ptx::make_smem_desc_sw128(sb + k * B_KSTEP, B_LBO, 1024);
                        ptx::mma_bf16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    const uint32_t eb = ptx::smem_u32(&empty_bar[stage]);
                    ptx::mma_commit_pair(ptx::mapa_shared(eb, 0));  // frees the slot in both CTAs
                    ptx::mma_commit_pair(ptx::mapa_shared(eb, 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    const uint32_t fb = ptx::smem_u32(&tmem_full[acc]);
                    ptx::mma_commit_pair(ptx::mapa_shared(fb, 0));
                    ptx::mma_commit_pair(ptx::mapa_shared(fb, 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const int quarter = warp & 3;
        uint32_t acc_phase[2] = {0, 0};
        int it = 0;
        bool ok = true;
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
            const int acc = it & 1;
            int tm, tn;
            tile_coords(t, tm, tn);
            if (!ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase[acc], abort_flag, kWaitLimitNs)) {
                if (lane == 0) atomicCAS(p.error_flag, 0, (0x13 << 8) | 1);
                ok = false;
                break;
            }
            acc_phase[acc] ^= 1u;
            ptx::tc_fence_after();
            const int row = tm * TM + (int)cta * 128 + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TN);
            if constexpr (EPI == EPI_PUSH_HEADS) {
                const int P = p.push_ranks, D = p.push_d, Hq = p.push_hq, Hkv = p.push_hkv;
                const int Hlq = Hq / P, rep = Hkv >= P ? 1 : P / Hkv, Hlkv = Hkv >= P ? Hkv / P : 1;
                const int W = (Hlq + 2 * Hlkv) * D;
                const int64_t drow = ((int64_t)p.push_rank * p.push_rows + row) * W;
#pragma unroll 1
                for (int c = 0; c < TN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                    ptx::tmem_ld_wait();
                    const int col0 = tn * TN + c * 32;
                    if (row_ok && col0 < p.N) {
                        // which head does this 32-column piece belong to, and who owns it
                        const int head = col0 / D, within = col0 - head * D;
                        int first_owner, owners, dcol;
                        if (head < Hq) {
                            first_owner = head / Hlq; owners = 1; dcol = (head - first_owner * Hlq) * D + within;
                        } else {
                            const int is_v = head >= Hq + Hkv;
                            const int kvh = head - Hq - is_v * Hkv;
                            first_owner = rep > 1 ? kvh * rep : kvh / Hlkv;
                            owners = rep;
                            dcol = (Hlq + is_v * Hlkv + (rep > 1 ? 0 : kvh - first_owner * Hlkv)) * D + within;
                        }
                        bf16x8 packed[4];
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            float o[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(r[v * 8 + j]);
                            packed[v] = pack8(o);
                        }
                        for (int o = first_owner; o < first_owner + owners; ++o) {
                            bf16x8* dst = reinterpret_cast<bf16x8*>(p.push_dst[o] + drow + dcol);
#pragma unroll
                            for (int v = 0; v < 4; ++v) dst[v] = packed[v];
                        }
                    }
                }
            } else
            if constexpr (EPI == EPI_SWIGLU) {
                bf16* crow = p.C + (int64_t)row * p.ldc + (int64_t)tn * (TN / 2);
#pragma unroll 1
                for (int g = 0; g < TN / 128; ++g) {
#pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        uint32_t rg[32], ru[32];
                        ptx::tmem_ld_32x32b_x32(taddr + g * 128 + h * 32, rg);
                        ptx::tmem_ld_32x32b_x32(taddr + g * 128 + 64 + h * 32, ru);
                        ptx::tmem_ld_wait();
                        const int col0 = tn * (TN / 2) + g * 64 + h * 32;
                        if (row_ok && col0 < p.N / 2) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                float o[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const float gg = __uint_as_float(rg[v * 8 + j]);
                                    const float uu = __uint_as_float(ru[v * 8 + j]);
                                    o[j] = gg / (1.f + __expf(-gg)) * uu;
                                }
                                *reinterpret_cast<bf16x8*>(crow + g * 64 + h * 32 + v * 8) = pack8(o);
                            }
                        }
                    }
                }
            } else {
                bf16* crow = p.C + (int64_t)row * p.ldc + (int64_t)tn * TN;
                const bf16* rrow = p.R + (int64_t)row * p.ldr + (int64_t)tn * TN;
                const bool streaming = (p.cache_flags & 1) != 0;
#pragma unroll 1
                for (int c = 0; c < TN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                    ptx::tmem_ld_wait();
                    const int col0 = tn * TN + c * 32;
                    if (row_ok) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col0 + v * 8 < p.N) {
                                float o[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(r[v * 8 + j]);
                                uint4* dst = reinterpret_cast<uint4*>(crow + c * 32 + v * 8);
                                if constexpr (EPI == EPI_ACCUM) {
                                    float old[8];
                                    const uint4* src = reinterpret_cast<const uint4*>(rrow + c * 32 + v * 8);
                                    const uint4 raw = streaming ? __ldcs(src) : *src;
                                    unpack8(*reinterpret_cast<const bf16x8*>(&raw), old);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) o[j] += old[j];
                                }
                                const bf16x8 packed = pack8(o);
                                if (streaming) __stcs(dst, *reinterpret_cast<const uint4*>(&packed));
                                else *dst = *reinterpret_cast<const uint4*>(&packed);
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&tmem_empty[acc]), 0));
        }
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // no CTA of the pair leaves while the other may still signal its barriers or read its tiles
    ptx::tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------------

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
        TORCH_CHECK(err == cudaSuccess && qres == cudaDriverEntryPointSuccess && ptr != nullptr,
                    "cuTensorMapEncodeTiled is not available from the driver");
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }();
    return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension `ld` (elements),
// box = [box_rows, 64 columns], 128-byte swizzle.
CUtensorMap make_tmap_bf16(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    TORCH_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA: base address must be 16-byte aligned");
    TORCH_CHECK((ld * 2) % 16 == 0, "TMA: row pitch must be a multiple of 16 bytes");
    // cuTensorMapEncodeTiled is a driver call and needs a context bound to this thread; a fresh thread (an autograd
    // worker on device 0, which never had to switch devices) has none until the first runtime call.
    static thread_local bool context_bound = false;
    if (!context_bound) {
        C10_CUDA_CHECK(cudaFree(nullptr));
        context_bound = true;
    }
    CUtensorMap tm;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = get_encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[256];
        snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with code %d (base %p, rows %lld, cols %lld, pitch %lld, box rows %d)",
                 (int)r, base, (long long)rows, (long long)cols, (long long)ld, box_rows);
        TORCH_CHECK(false, msg);
    }
    return tm;
}

at::Tensor& error_flag_for(const at::Device& dev) {
    static std::vector<at::Tensor> flags(64);
    auto& f = flags[dev.index() < 0 ? 0 : dev.index()];
    if (!f.defined()) f = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
    return f;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_ctas) {
    using L = SmemLayout<BN, STAGES>;
    auto kernel = gemm_bf16_tcgen05_kernel<BN, STAGES, A_MN, B_MN, EPI>;
    constexpr int smem_bytes = L::kTotal + 1024;  // slack for the 1024-byte round-up
    static bool attr_set = false;
    if (!attr_set) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        attr_set = true;
    }
    // the tile count of a grouped GEMM lives on the device: launch one persistent CTA per SM
    const int tiles = p.group_mode == GROUP_NONE ? (int)(ceil_div(p.M, BM) * ceil_div(p.N, BN)) : max_ctas;
    const int grid = std::max(1, std::min(tiles, max_ctas));
    kernel<<<grid, 192, smem_bytes, current_stream()>>>(ta, tb, p);
    ATB_LAUNCH_CHECK();
}

static const SegMaps kNoSegs = {};

template <int STAGES, bool A_MN, bool B_MN, int EPI>
void launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_ctas,
                      const SegMaps& segs = kNoSegs) {
    using L = PairSmemLayout<STAGES>;
    auto kernel = gemm_bf16_tcgen05_pair_kernel<STAGES, A_MN, B_MN, EPI>;
    constexpr int smem_bytes = L::kTotal + 1024;
    // The tile loop is static (cluster i takes tiles i, i + n, ...), so every cluster of the grid must be resident at
    // once: ask the runtime how many CTA pairs fit on the device (GPCs with an odd SM count leave one SM unpaired).
    static int max_clusters = 0;
    if (max_clusters == 0) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kNumSMs / 2 * 2);
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = smem_bytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        C10_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        max_clusters = std::max(1, n);
    }
    const int tiles = (int)(ceil_div(p.M, 256) * ceil_div(p.N, 256));
    const int stage_clusters = p.stage_ctas / 2;  // staging CTAs share the resident-cluster budget with the computing pairs
    TORCH_CHECK(p.stage_ctas % 2 == 0 && stage_clusters < max_clusters, "gemm: too many staging CTAs");
    const int clusters = std::max(1, std::min(tiles, std::min(max_ctas / 2, max_clusters - stage_clusters)));
    kernel<<<2 * (clusters + stage_clusters), 192, smem_bytes, current_stream()>>>(ta, tb, p, segs);
    ATB_LAUNCH_CHECK();
}

template <bool A_MN, bool B_MN>
void dispatch_epi_pair(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_ctas) {
    switch (epi) {
        case EPI_STORE: launch_gemm_pair<6, A_MN, B_MN, EPI_STORE>(ta, tb, p, max_ctas); break;
        case EPI_ACCUM: launch_gemm_pair<6, A_MN, B_MN, EPI_ACCUM>(ta, tb, p, max_ctas); break;
        case EPI_SWIGLU:
            if constexpr (!A_MN && !B_MN) { launch_gemm_pair<6, false, false, EPI_SWIGLU>(ta, tb, p, max_ctas); break; }
        default: TORCH_CHECK(false, "gemm: unsupported epilogue ", epi, " for this operand layout");
    }
}

static bool g_use_cta_pairs = true;  // dense GEMMs run on the CTA-pair kernel unless switched off

// ATB200_GEMM_CACHE: bit 0 streaming output stores / accumulate loads, bit 1 evict-last operand loads (read once)
static int gemm_cache_flags() {
    static const int flags = [] {
        const char* e = std::getenv("ATB200_GEMM_CACHE");
        return e ? std::atoi(e) : 0;
    }();
    return flags;
}

template <bool A_MN, bool B_MN>
void dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_ctas) {
    switch (epi) {
        case EPI_STORE: launch_gemm<256, 4, A_MN, B_MN, EPI_STORE>(ta, tb, p, max_ctas); break;
        case EPI_ACCUM: launch_gemm<256, 4, A_MN, B_MN, EPI_ACCUM>(ta, tb, p, max_ctas); break;
        case EPI_SWIGLU:
            if constexpr (!A_MN && !B_MN) { launch_gemm<256, 4, false, false, EPI_SWIGLU>(ta, tb, p, max_ctas); break; }
        default: TORCH_CHECK(false, "gemm: unsupported epilogue ", epi, " for this operand layout");
    }
}

}  // namespace

// out = gemm(a, b).  a_mn == false: a is [M, K]; true: a is [K, M].  b_mn == false: b is [N, K]; true: [K, N].
// epilogue: 0 store, 1 accumulate into `out`, 2 SwiGLU (out is [M, N/2]).
at::Tensor gemm_bf16(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, int64_t epilogue,
                     const c10::optional<at::Tensor>& out_opt, int64_t max_ctas,
                     const c10::optional<at::Tensor>& residual) {
    ATB_CHECK_CUDA(a); ATB_CHECK_CUDA(b);
    ATB_CHECK_DTYPE(a, at::kBFloat16); ATB_CHECK_DTYPE(b, at::kBFloat16);
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm: operands must be 2-D");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "gemm: operands must have a unit inner stride");
    const int64_t M = a_mn ? a.size(1) : a.size(0);
    const int64_t K = a_mn ? a.size(0) : a.size(1);
    const int64_t N = b_mn ? b.size(1) : b.size(0);
    const int64_t Kb = b_mn ? b.size(0) : b.size(1);
    TORCH_CHECK(K == Kb, "gemm: contraction sizes differ (", K, " vs ", Kb, ")");
    TORCH_CHECK(M > 0 && N > 0 && K > 0, "gemm: empty operand");
    TORCH_CHECK(N % 8 == 0, "gemm: N must be a multiple of 8");
    TORCH_CHECK(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "gemm: dimension too large");
    const int epi = (int)epilogue;
    if (epi == EPI_SWIGLU) TORCH_CHECK(N % 128 == 0, "gemm: SwiGLU epilogue needs N to be a multiple of 128");
    c10::cuda::CUDAGuard guard(a.device());

    const int64_t out_cols = epi == EPI_SWIGLU ? N / 2 : N;
    at::Tensor out;
    if (out_opt.has_value()) {
        out = *out_opt;
        ATB_CHECK_DTYPE(out, at::kBFloat16);
        TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == out_cols && out.stride(1) == 1,
                    "gemm: output has the wrong shape");
        TORCH_CHECK(out.stride(0) % 8 == 0, "gemm: output pitch must be a multiple of 8 elements");
    } else {
        TORCH_CHECK(epi != EPI_ACCUM || residual.has_value(), "gemm: accumulate epilogue needs an output or a residual tensor");
        out = at::empty({M, out_cols}, a.options());
    }
    ATB_CHECK_ALIGNED16(out);
    if (residual.has_value()) {
        TORCH_CHECK(epi == EPI_ACCUM, "gemm: a residual needs the accumulate epilogue");
        ATB_CHECK_DTYPE(*residual, at::kBFloat16); ATB_CHECK_ALIGNED16(*residual);
        TORCH_CHECK(residual->dim() == 2 && residual->size(0) == M && residual->size(1) == N && residual->stride(1) == 1 &&
                    residual->stride(0) % 8 == 0, "gemm: residual has the wrong shape");
    }

    // tensor maps: K-major operand [rows, K] -> box [tile rows, 64 k]; MN-major [K, rows] -> box [64 k, 64 rows]
    const CUtensorMap ta = a_mn ? make_tmap_bf16(a.data_ptr(), K, M, a.stride(0), BK)
                                : make_tmap_bf16(a.data_ptr(), M, K, a.stride(0), BM);
    const bool pairs = g_use_cta_pairs && max_ctas != 1;
    const CUtensorMap tb = b_mn ? make_tmap_bf16(b.data_ptr(), K, N, b.stride(0), BK)
                                : make_tmap_bf16(b.data_ptr(), N, K, b.stride(0), pairs ? 128 : 256);
    if (a_mn) TORCH_CHECK(M % 8 == 0, "gemm: MN-major A needs M to be a multiple of 8");

    GemmParams p;
    p.cache_flags = 0;
    p.C = (bf16*)out.data_ptr();
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.ldc = out.stride(0);
    p.R = residual.has_value() ? (const bf16*)residual->data_ptr() : p.C;
    p.ldr = residual.has_value() ? residual->stride(0) : p.ldc;
    p.a_seg_len = 0;
    p.a_seg_row0 = 0;
    p.stage_ctas = 0;
    p.stage_segs = 0;
    p.error_flag = error_flag_for(a.device()).data_ptr<int>();
    p.group_offsets = nullptr;
    p.num_groups = 0;
    p.group_mode = GROUP_NONE;
    p.cache_flags = gemm_cache_flags();
    const int ctas = max_ctas > 0 ? (int)max_ctas : kNumSMs;
    if (pairs) {
        if (!a_mn && !b_mn) dispatch_epi_pair<false, false>(epi, ta, tb, p, ctas);
        else if (!a_mn && b_mn) dispatch_epi_pair<false, true>(epi, ta, tb, p, ctas);
        else if (a_mn && !b_mn) dispatch_epi_pair<true, false>(epi, ta, tb, p, ctas);
        else dispatch_epi_pair<true, true>(epi, ta, tb, p, ctas);
        return out;
    }
    if (!a_mn && !b_mn) dispatch_epi<false, false>(epi, ta, tb, p, ctas);
    else if (!a_mn && b_mn) dispatch_epi<false, true>(epi, ta, tb, p, ctas);
    else if (a_mn && !b_mn) dispatch_epi<true, false>(epi, ta, tb, p, ctas);
    else dispatch_epi<true, true>(epi, ta, tb, p, ctas);
    return out;
}

// Grouped GEMM over ragged, tile-aligned segments (mixture-of-experts).  `offsets` is int32 [G + 1] on the device:
// first row of every group in the ragged operand, each a multiple of 128; rows up to offsets[G] are used.
//   mode 1 (ragged M):  out[r, :] = a[r, :] * B_g^T for r in group g.
//        a [R, K] (K contiguous); b_mn == false: b is [G * N, K] (forward);  b_mn == true: b is [G * K, N]
//        (data gradient: b holds the forward weights [G, K_c, N_out] and the contraction runs over their rows).
//   mode 2 (ragged K):  out_g [M, N] = a[rows_g, :M]^T * b[rows_g, :N]  (weight gradient), out is [G * M, N]
//        and must be zero-initialised by the caller when groups may be empty.
// epilogue as in gemm_bf16 (SwiGLU only for mode 1 with b_mn == false).
at::Tensor gemm_bf16_grouped(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets, int64_t mode,
                             bool b_mn, int64_t epilogue, const c10::optional<at::Tensor>& out_opt) {
    ATB_CHECK_CUDA(a); ATB_CHECK_CUDA(b); ATB_CHECK_CUDA(offsets);
    ATB_CHECK_DTYPE(a, at::kBFloat16); ATB_CHECK_DTYPE(b, at::kBFloat16); ATB_CHECK_DTYPE(offsets, at::kInt);
    ATB_CHECK_CONTIG(offsets);
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "grouped gemm: operands must be 2-D, unit inner stride");
    const int64_t G = offsets.numel() - 1;
    TORCH_CHECK(G >= 1 && G <= kMaxGroups, "grouped gemm: between 1 and 1024 groups");
    const int epi = (int)epilogue;
    c10::cuda::CUDAGuard guard(a.device());
    GemmParams p;
    p.cache_flags = 0;
    p.error_flag = error_flag_for(a.device()).data_ptr<int>();
    p.group_offsets = offsets.data_ptr<int>();
    p.num_groups = (int)G;
    p.group_mode = (int)mode;
    at::Tensor out;
    if (mode == GROUP_RAGGED_M) {
        const int64_t R = a.size(0), K = a.size(1);
        int64_t N;
        if (!b_mn) {
            TORCH_CHECK(b.size(0) % G == 0 && b.size(1) == K, "grouped gemm: b must be [G * N, K]");
            N = b.size(0) / G;
        } else {
            TORCH_CHECK(b.size(0) == G * K, "grouped gemm: b must be [G * K, N]");
            N = b.size(1);
        }
        TORCH_CHECK(R % BM == 0, "grouped gemm: the ragged operand must have a multiple of 128 rows");
        TORCH_CHECK(N % 8 == 0 && K % 8 == 0, "grouped gemm: N and K must be multiples of 8");
        if (epi == EPI_SWIGLU) TORCH_CHECK(N % 128 == 0 && !b_mn, "grouped gemm: SwiGLU epilogue needs K-major b and N % 128 == 0");
        const int64_t out_cols = epi == EPI_SWIGLU ? N / 2 : N;
        if (out_opt.has_value()) {
            out = *out_opt;
            TORCH_CHECK(out.dim() == 2 && out.size(0) == R && out.size(1) == out_cols && out.stride(1) == 1, "grouped gemm: bad output shape");
        } else {
            TORCH_CHECK(epi != EPI_ACCUM, "grouped gemm: accumulate needs an output tensor");
            out = at::zeros({R, out_cols}, a.options());  // rows past offsets[G] stay zero
        }
        p.M = (int)R; p.N = (int)N; p.K = (int)K;
        const CUtensorMap ta = make_tmap_bf16(a.data_ptr(), R, K, a.stride(0), BM);
        const CUtensorMap tb = b_mn ? make_tmap_bf16(b.data_ptr(), G * K, N, b.stride(0), BK)
                                    : make_tmap_bf16(b.data_ptr(), G * N, K, b.stride(0), 256);
        p.C = (bf16*)out.data_ptr();
        p.ldc = out.stride(0);
        p.R = p.C;
        p.ldr = p.ldc;
        p.a_seg_len = 0;
        p.a_seg_row0 = 0;
        p.stage_ctas = 0;
        p.stage_segs = 0;
        if (!b_mn) dispatch_epi<false, false>(epi, ta, tb, p, kNumSMs);
        else dispatch_epi<false, true>(epi, ta, tb, p, kNumSMs);
    } else if (mode == GROUP_RAGGED_K) {
        const int64_t R = a.size(0), M = a.size(1), N = b.size(1);
        TORCH_CHECK(b.size(0) == R, "grouped gemm: both operands must have the same ragged rows");
        TORCH_CHECK(R % BK == 0 && M % 8 == 0 && N % 8 == 0, "grouped gemm: rows % 64 == 0, M % 8 == 0, N % 8 == 0");
        TORCH_CHECK(epi == EPI_STORE || epi == EPI_ACCUM, "grouped gemm: weight-gradient mode supports store/accumulate");
        if (out_opt.has_value()) {
            out = *out_opt;
            TORCH_CHECK(out.dim() == 2 && out.size(0) == G * M && out.size(1) == N && out.stride(1) == 1, "grouped gemm: bad output shape");
        } else {
            TORCH_CHECK(epi != EPI_ACCUM, "grouped gemm: accumulate needs an output tensor");
            out = at::zeros({G * M, N}, a.options());
        }
        p.M = (int)M; p.N = (int)N; p.K = 0;
        const CUtensorMap ta = make_tmap_bf16(a.data_ptr(), R, M, a.stride(0), BK);
        const CUtensorMap tb = make_tmap_bf16(b.data_ptr(), R, N, b.stride(0), BK);
        p.C = (bf16*)out.data_ptr();
        p.ldc = out.stride(0);
        p.R = p.C;
        p.ldr = p.ldc;
        p.a_seg_len = 0;
        p.a_seg_row0 = 0;
        p.stage_ctas = 0;
        p.stage_segs = 0;
        dispatch_epi<true, true>(epi, ta, tb, p, kNumSMs);
    } else {
        TORCH_CHECK(false, "grouped gemm: mode must be 1 (ragged M) or 2 (ragged K)");
    }
    ATB_CHECK_ALIGNED16(out);
    return out;
}

// Selects the CTA-pair (cta_group::2, 256 x 256 tile) kernel for dense GEMMs; returns the previous setting.
// Fused q|k|v projection + Ulysses sequence -> head exchange: x [rows, K] times w [(Hq + 2 Hkv) D, K]^T, where the
// epilogue stores every head's columns into the owning rank's buffer (dst_ptrs[o] + dst_byte_offset, laid out
// [P * rows, Hlq + 2 Hlkv, D], this rank's rows at rank * rows).  Nothing is written locally.  The caller separates
// launches on different ranks from the consumers of the buffers with a device barrier.
void gemm_bf16_push_heads(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dst_ptrs, int64_t dst_byte_offset,
                          int64_t rank, int64_t Hq, int64_t Hkv, int64_t D) {
    ATB_CHECK_CUDA(x); ATB_CHECK_CUDA(w); ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_DTYPE(w, at::kBFloat16);
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && x.size(1) == w.size(1), "push_heads: x [rows, K], w [N, K]");
    TORCH_CHECK(dst_ptrs.device().is_cpu() && dst_ptrs.scalar_type() == at::kLong, "peer pointers: int64 CPU tensor");
    const int P = (int)dst_ptrs.numel();
    const int64_t M = x.size(0), N = w.size(0), K = x.size(1);
    TORCH_CHECK(P >= 1 && P <= 8 && Hq % P == 0 && (Hkv >= P ? Hkv % P == 0 : P % Hkv == 0), "push_heads: heads and ranks must divide");
    TORCH_CHECK(N == (Hq + 2 * Hkv) * D && D % 32 == 0 && K % 8 == 0 && dst_byte_offset % 16 == 0, "push_heads: shape mismatch");
    TORCH_CHECK(x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0, "push_heads: row pitches must be multiples of 8 elements");
    ATB_CHECK_ALIGNED16(x); ATB_CHECK_ALIGNED16(w);
    if (M == 0) return;
    c10::cuda::CUDAGuard guard(x.device());
    const CUtensorMap ta = make_tmap_bf16(x.data_ptr(), M, K, x.stride(0), 128);
    const CUtensorMap tb = make_tmap_bf16(w.data_ptr(), N, K, w.stride(0), 128);
    GemmParams p;
    p.cache_flags = 0;
    p.C = nullptr; p.R = nullptr; p.ldc = 0; p.ldr = 0;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.error_flag = error_flag_for(x.device()).data_ptr<int>();
    p.group_offsets = nullptr; p.num_groups = 0; p.group_mode = GROUP_NONE;
    p.a_seg_len = 0; p.a_seg_row0 = 0; p.stage_ctas = 0; p.stage_segs = 0;
    for (int o = 0; o < P; ++o) p.push_dst[o] = reinterpret_cast<bf16*>(dst_ptrs.data_ptr<int64_t>()[o] + dst_byte_offset);
    p.push_ranks = P; p.push_rank = (int)rank; p.push_hq = (int)Hq; p.push_hkv = (int)Hkv; p.push_d = (int)D; p.push_rows = (int)M;
    launch_gemm_pair<6, false, false, EPI_PUSH_HEADS>(ta, tb, p, kNumSMs);
}

// out = A b^T (+ residual) where K segment j of A [M, P * seg_cols] is rows [row0, row0 + M) of the [rows_total,
// seg_cols] bf16 tensor at a_ptrs[j] + a_byte_offset, which may be another GPU's memory mapped into this process (the
// head-sharded attention outputs of the Ulysses peers: the head -> sequence all-to-all happens inside the GEMM).
// b is [N, P * seg_cols].  Returns (out, a_local).
//   stage_ctas > 0: that many CTAs of the same launch copy the segments into a_local [M, K] (each remote byte crosses
//     NVLink once) while the other CTAs multiply tiles whose rows have arrived; a_local is the gathered operand, which
//     a caller needs again for the weight gradient.
//   stage_ctas == 0: every CTA pair fetches its A tiles from the owners directly with TMA; nothing is materialised
//     (a_local is empty), but a tile crosses the link once per column tile of the output.
std::tuple<at::Tensor, at::Tensor> gemm_bf16_peer_a(const at::Tensor& a_ptrs, int64_t a_byte_offset, int64_t rows_total,
                                                    int64_t seg_cols, int64_t row0, int64_t M, const at::Tensor& b,
                                                    const c10::optional<at::Tensor>& residual, int64_t stage_ctas) {
    ATB_CHECK_CUDA(b); ATB_CHECK_DTYPE(b, at::kBFloat16);
    TORCH_CHECK(a_ptrs.device().is_cpu() && a_ptrs.scalar_type() == at::kLong, "peer pointers: int64 CPU tensor");
    const int P = (int)a_ptrs.numel();
    TORCH_CHECK(P >= 1 && P <= kMaxSegs, "gemm_peer_a: 1..8 segments");
    TORCH_CHECK(seg_cols % BK == 0 && a_byte_offset % 16 == 0, "gemm_peer_a: segment width must be a multiple of 64");
    TORCH_CHECK(b.dim() == 2 && b.stride(1) == 1 && b.size(1) == P * seg_cols && b.stride(0) % 8 == 0, "gemm_peer_a: b must be [N, P * seg_cols]");
    TORCH_CHECK(M > 0 && row0 >= 0 && row0 + M <= rows_total && M < (1ll << 31), "gemm_peer_a: row range outside the segment tensors");
    TORCH_CHECK(stage_ctas >= 0 && stage_ctas % 2 == 0 && stage_ctas <= 64, "gemm_peer_a: staging CTAs: even, at most 64");
    const int64_t N = b.size(0), K = P * seg_cols;
    TORCH_CHECK(N % 8 == 0, "gemm_peer_a: N must be a multiple of 8");
    c10::cuda::CUDAGuard guard(b.device());
    auto out = at::empty({M, N}, b.options());
    at::Tensor a_local = at::empty({stage_ctas > 0 ? M : 0, K}, b.options());
    at::Tensor flags;
    SegMaps segs = {};
    GemmParams p;
    p.cache_flags = 0;
    p.a_seg_len = (int)seg_cols;
    p.a_seg_row0 = (int)row0;
    p.stage_ctas = (int)stage_ctas;
    p.stage_segs = P;
    p.stage_mode = 0;
    CUtensorMap ta;
    if (stage_ctas > 0) {
        flags = at::zeros({(int64_t)ceil_div(M, 256)}, b.options().dtype(at::kInt));
        for (int j = 0; j < P; ++j)
            p.stage_src[j] = reinterpret_cast<const bf16*>(a_ptrs.data_ptr<int64_t>()[j] + a_byte_offset);
        p.stage_src_ld = seg_cols;
        p.stage_dst = (bf16*)a_local.data_ptr();
        p.stage_dst_ld = K;
        p.stage_flags = flags.data_ptr<int>();
        ta = make_tmap_bf16(a_local.data_ptr(), M, K, K, 128);
        p.a_seg_len = (int)seg_cols;  // the staging CTAs need the segment width; the TMA producer reads a_local
    } else {
        for (int j = 0; j < P; ++j)
            segs.m[j] = make_tmap_bf16(reinterpret_cast<void*>(a_ptrs.data_ptr<int64_t>()[j] + a_byte_offset), rows_total,
                                       seg_cols, seg_cols, 128);
        ta = segs.m[0];
    }
    const CUtensorMap tb = make_tmap_bf16(b.data_ptr(), N, K, b.stride(0), 128);
    p.C = (bf16*)out.data_ptr();
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.ldc = out.stride(0);
    p.R = p.C;
    p.ldr = p.ldc;
    int epi = EPI_STORE;
    if (residual.has_value()) {
        ATB_CHECK_DTYPE(*residual, at::kBFloat16); ATB_CHECK_ALIGNED16(*residual);
        TORCH_CHECK(residual->dim() == 2 && residual->size(0) == M && residual->size(1) == N && residual->stride(1) == 1 &&
                    residual->stride(0) % 8 == 0, "gemm_peer_a: residual has the wrong shape");
        p.R = (const bf16*)residual->data_ptr();
        p.ldr = residual->stride(0);
        epi = EPI_ACCUM;
    }
    p.error_flag = error_flag_for(b.device()).data_ptr<int>();
    p.group_offsets = nullptr;
    p.num_groups = 0;
    p.group_mode = GROUP_NONE;
    if (epi == EPI_STORE) launch_gemm_pair<6, false, false, EPI_STORE>(ta, tb, p, kNumSMs, segs);
    else launch_gemm_pair<6, false, false, EPI_ACCUM>(ta, tb, p, kNumSMs, segs);
    return {out, a_local};
}

// out [M, N] = x [M, K] * W^T where W [N, K] lives at element offset `w_elem_offset` of a flat parameter buffer that is
// sharded contiguously over the ranks (ZeRO-3): rank p holds elements [p * shard_elems, (p + 1) * shard_elems) at
// shard_ptrs[p] + shard_byte_offset.  Staging CTAs of the same launch copy W's element range from the owners' shards
// (peer memory: plain bulk copies, no multicast) into `flat` (this rank's full buffer of the unit) while the CTA pairs
// multiply the row tiles of W that have arrived.  When the call returns (in stream order) `flat` holds all of W.
at::Tensor gemm_bf16_gather_b(const at::Tensor& x, const at::Tensor& shard_ptrs, int64_t shard_byte_offset, int64_t shard_elems,
                              at::Tensor flat, int64_t w_elem_offset, int64_t N, int64_t stage_ctas) {
    ATB_CHECK_CUDA(x); ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_CUDA(flat); ATB_CHECK_DTYPE(flat, at::kBFloat16);
    ATB_CHECK_CONTIG(flat); ATB_CHECK_ALIGNED16(flat); ATB_CHECK_ALIGNED16(x);
    TORCH_CHECK(shard_ptrs.device().is_cpu() && shard_ptrs.scalar_type() == at::kLong, "peer pointers: int64 CPU tensor");
    const int P = (int)shard_ptrs.numel();
    TORCH_CHECK(P >= 1 && P <= kMaxSegs, "gemm_gather_b: 1..8 ranks");
    TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0, "gemm_gather_b: x must be [M, K], K contiguous");
    const int64_t M = x.size(0), K = x.size(1);
    TORCH_CHECK(M > 0 && M < (1ll << 31) && N % 8 == 0 && K % 64 == 0, "gemm_gather_b: N % 8 == 0 and K % 64 == 0 expected");
    TORCH_CHECK(shard_elems % 8 == 0 && w_elem_offset % 8 == 0 && shard_byte_offset % 16 == 0,
                "gemm_gather_b: shard size and offsets must be multiples of 16 bytes");
    TORCH_CHECK(w_elem_offset >= 0 && w_elem_offset + N * K <= std::min<int64_t>(flat.numel(), shard_elems * P),
                "gemm_gather_b: the weight lies outside the flat buffer");
    TORCH_CHECK(stage_ctas >= 2 && stage_ctas % 2 == 0 && stage_ctas <= 64, "gemm_gather_b: staging CTAs: even, 2..64");
    c10::cuda::CUDAGuard guard(x.device());
    auto out = at::empty({M, N}, x.options());
    auto flags = at::zeros({(int64_t)ceil_div(N, 256)}, x.options().dtype(at::kInt));
    SegMaps segs = {};
    GemmParams p;
    p.cache_flags = 0;
    p.a_seg_len = 0; p.a_seg_row0 = 0;
    p.stage_ctas = (int)stage_ctas;
    p.stage_segs = 1;
    p.stage_mode = 1;
    p.stage_flat_off = w_elem_offset;
    p.stage_shard_elems = shard_elems;
    for (int j = 0; j < P; ++j)
        p.stage_src[j] = reinterpret_cast<const bf16*>(shard_ptrs.data_ptr<int64_t>()[j] + shard_byte_offset);
    p.stage_src_ld = 0;
    p.stage_dst = (bf16*)flat.data_ptr();
    p.stage_dst_ld = 0;
    p.stage_flags = flags.data_ptr<int>();
    const CUtensorMap ta = make_tmap_bf16(x.data_ptr(), M, K, x.stride(0), 128);
    const CUtensorMap tb = make_tmap_bf16((bf16*)flat.data_ptr() + w_elem_offset, N, K, K, 128);
    p.C = (bf16*)out.data_ptr();
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.ldc = out.stride(0);
    p.R = p.C;
    p.ldr = p.ldc;
    p.error_flag = error_flag_for(x.device()).data_ptr<int>();
    p.group_offsets = nullptr;
    p.num_groups = 0;
    p.group_mode = GROUP_NONE;
    launch_gemm_pair<6, false, false, EPI_STORE>(ta, tb, p, kNumSMs, segs);
    return out;
}

bool set_gemm_cta_pairs(bool on) {
    const bool old = g_use_cta_pairs;
    g_use_cta_pairs = on;
    return old;
}

CUtensorMap make_tmap_bf16_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    return make_tmap_bf16(base, rows, cols, ld, box_rows);
}
// 2-D fp32 tensor map over a row-major [rows, cols] matrix (leading dimension `ld` elements), box = [box_rows, 32 columns]
// (128 bytes), 128-byte swizzle: the staging layout of reductions into an fp32 accumulator.
CUtensorMap make_tmap_f32_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    TORCH_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0 && (ld * 4) % 16 == 0, "TMA: fp32 base / pitch must be 16-byte aligned");
    C10_CUDA_CHECK(cudaFree(nullptr));  // binds a context to this thread (see make_tmap_bf16)
    CUtensorMap tm;
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = get_encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (fp32) failed with code ", (int)r);
    return tm;
}
at::Tensor& gemm_error_flag(const at::Device& dev) { return error_flag_for(dev); }

// Reads and clears the per-device error word written by kernels whose bounded waits gave up.
int64_t read_and_clear_error_flag(const at::Tensor& like) {
    auto& f = error_flag_for(like.device());
    const int64_t v = f.item<int>();
    if (v != 0) f.zero_();
    return v;
}

}  // namespace atb
