// SPDX-License-Identifier: Apache-2.0
// Causal flash-attention backward for sm_100a: packed (variable-length) sequences, grouped-query heads, head_dim 128.
//
// Given Q, K, V, the forward output O with its log-sum-exp L, and dO, it computes per packed sequence
//   P  = exp(Q K^T * scale - L)            (recomputed, never stored)
//   dV = P^T dO        dP = dO V^T        dS = P o (dP - D),  D = rowsum(dO o O)
//   dK = scale * dS^T Q                     dQ = scale * dS K
//
// One CTA owns a block of 128 keys of one KV head and walks over every query block at or after it, for each of the
// query heads that share the KV head, so dK and dV accumulate in tensor memory and are written once (no atomics,
// bit-reproducible).  The scores are computed transposed (S^T = K Q^T, dP^T = V dO^T: a thread owns a key row), which
// lets P^T go back into tensor memory as bf16 and feed the dV product as the A operand without a shared-memory copy;
// dS^T is written once to shared memory and serves both as the K-major A operand of dK and as the MN-major A operand
// of dQ.  Tensor memory (512 columns): S^T / P^T | dP^T / dQ | dV | dK.  dQ of one (query block, key block) pair is
// staged in shared memory and added to an fp32 accumulator in global memory by the TMA unit (bulk tensor reductions,
// which keep the load/store pipes of the SM free for the score warps; the order of these additions is not fixed, so
// dQ is reproducible to fp32 rounding only) and converted to bf16, times the softmax scale, by a small kernel.
//
// Roles: warp 0 loads K, V, the Q ring (two slots) and the L / D vectors, warp 2 the dO slot (TMA), warp 1 issues the
// tensor-core products, eight warps turn S^T into P^T and dP^T into dS^T (two groups, 64 query columns each), four
// warps drain dQ.  Issue order per query block i:
//   dQ(i) dK(i) | dP(i+1) dV(i+1) | S(i+2)
// so that the exponentials of block i+1 run under dQ / dK of block i, the drain of dQ(i) runs under dK(i), and dP(i+1),
// which the next dS waits for, does not queue behind the product that needs those exponentials.
// All barrier waits are bounded.
//
// The reference obtains the attention backward from the flash-attn package or PyTorch SDPA through Hugging Face
// (arctic_training/config/model.py:48,85-98).

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>

#include <cstdlib>
#include <vector>

namespace atb {

CUtensorMap make_tmap_bf16_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
CUtensorMap make_tmap_f32_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
at::Tensor& gemm_error_flag(const at::Device& dev);

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int CHUNK_BYTES = 128 * 128;       // [128 rows][64 bf16]
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;  // 128 x 128 bf16
constexpr int SMEM_K = 0;
constexpr int SMEM_V = TILE_BYTES;
constexpr int SMEM_Q = 2 * TILE_BYTES;    // two stages
constexpr int SMEM_DO = 4 * TILE_BYTES;   // one stage: dO(i) is read by dP(i) and dV(i), which are issued back to back
constexpr int SMEM_DS = 5 * TILE_BYTES;   // dS^T of the current query block
constexpr int SMEM_DQ = 6 * TILE_BYTES;   // two staging buffers [128 rows][32 fp32] for the dQ reductions
constexpr int DQ_BUF_BYTES = 128 * 128;
constexpr int SMEM_LD = 7 * TILE_BYTES;   // float [2 stages][2][128]: L * log2(e) and D of the stage's query block
constexpr int SMEM_BAR = SMEM_LD + 2 * 2 * 128 * 4;
constexpr int SMEM_TOTAL = SMEM_BAR + 32 * 8;
static_assert(SMEM_TOTAL <= 232448, "shared memory budget of one CTA");
constexpr uint64_t kWaitNs = 2000000000ull;
// warps: 0 Q loads, 1 tensor-core issue, 2 dO loads, 3 unused, 4-11 scores (two groups of four: query columns 0-63 and
// 64-127 of every block), 12-15 dQ drain
constexpr int kThreads = 512;
constexpr int kDoWarp = 2, kScoreWarp0 = 4, kDrainWarp0 = 12;
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 384;

struct BwdParams {
    const float* lse2;  // [Hq, T]  log-sum-exp in log2 units
    const float* dsum;  // [Hq, T]  rowsum(dO o O)
    bf16* dk;           // [T, Hkv, 128], dkv_row_stride elements between tokens
    bf16* dv;
    int64_t dkv_row_stride;
    const int* cu_seqlens;
    int nseq, T, Hq, Hkv;
    float scale, scale_log2;
    int* error_flag;
    long long* prof;  // optional [32] cycle counters of the first CTA (nullptr: off)
    int debug_flags;  // timing experiments only.  bit 0: leave out the dQ reductions
};

// Cycle accounting of one CTA: every role sums clock64 deltas of its waits and phases in registers and adds them to its
// own slots of the profile buffer when it is done.
#define BWD_PROF_T() (prof_on ? clock64() : 0ll)

__global__ void __launch_bounds__(kThreads, 1)
fmha_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                        const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
    uint64_t* kv_full = bars;         // 1
    uint64_t* q_full = bars + 1;      // [2]
    uint64_t* q_empty = bars + 3;     // [2]
    uint64_t* do_full = bars + 5;     // 1
    uint64_t* do_empty = bars + 7;    // 1
    uint64_t* ld_full = bars + 9;     // [2]  L and D of the stage are in shared memory
    uint64_t* s_full = bars + 11;     // S^T of the block is in tensor memory
    uint64_t* p_ready = bars + 12;    // P^T is back in tensor memory (8 warps)
    uint64_t* dp_full = bars + 13;    // dP^T is in tensor memory
    uint64_t* ds_ready = bars + 14;   // dS^T is in shared memory (8 warps)
    uint64_t* ds_free = bars + 15;    // dK and dQ of the block have read dS^T
    uint64_t* dq_full = bars + 16;    // dQ of the block is in tensor memory
    uint64_t* dq_free = bars + 17;    // the dQ warps have copied it out (4 warps)
    uint64_t* acc_done = bars + 18;   // all products have retired: dK and dV are final
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* ld_smem = reinterpret_cast<float*>(smem + SMEM_LD);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.x;            // KV head
    const int G = p.Hq / p.Hkv;          // query heads per KV head
    // one lane of each role of the first CTA keeps the counters (slots are disjoint between roles)
    const bool prof_on = p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 &&
                         (warp == 0 || warp == 1 || warp == kDoWarp || warp == kScoreWarp0 || warp == kDrainWarp0);

    // ---- which (sequence, key block) is this CTA?  Key block 0 of a sequence has the most query blocks.
    int rem = (int)blockIdx.y;
    int seq = -1, jb = 0, tok0 = 0, seqlen = 0, nq = 0;
    for (int s = 0; s < p.nseq; ++s) {
        const int a = p.cu_seqlens[s], b = p.cu_seqlens[s + 1];
        const int nb = (b - a + BKV - 1) / BKV;
        if (rem < nb) { seq = s; jb = rem; tok0 = a; seqlen = b - a; nq = nb; break; }
        rem -= nb;
    }
    if (seq < 0) return;  // padding CTA of the upper-bound grid (uniform for the whole CTA)
    if ((ptx::smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(p.error_flag, 0, (0x28 << 8) | 1);
        return;
    }
    const int n_i = nq - jb;       // query blocks jb .. nq-1
    const int n_it = G * n_i;      // iterations: query heads of the group x query blocks

    if (threadIdx.x == 0) {
        ptx::mbar_init(kv_full, 1);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&q_full[i], 1);
            ptx::mbar_init(&q_empty[i], 1);
            ptx::mbar_init(&ld_full[i], 1);
        }
        ptx::mbar_init(do_full, 1);
        ptx::mbar_init(do_empty, 1);
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(p_ready, 8);
        ptx::mbar_init(dp_full, 1);
        ptx::mbar_init(ds_ready, 8);
        ptx::mbar_init(ds_free, 1);
        ptx::mbar_init(dq_full, 1);
        ptx::mbar_init(dq_free, 4);
        ptx::mbar_init(acc_done, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // cycle counters of this role (written out at the end)

    if (warp == 0 || warp == kDoWarp) {
        // ------------------------------------------------------------------ loads: warp 0 streams K, V once and then the
        // Q ring with the L / D vectors; a warp of its own streams the dO ring, so that neither ring waits for the
        // other's free slot
        const bool q_role = warp == 0;
        bool ok = true;
        if (lane == 0) {
            if (q_role) {
                ptx::tma_prefetch_desc(&tmap_q);
                ptx::tma_prefetch_desc(&tmap_k);
                ptx::tma_prefetch_desc(&tmap_v);
                ptx::mbar_expect_tx(kv_full, 2 * TILE_BYTES);
                for (int c = 0; c < 2; ++c) {
                    ptx::tma_load_2d(smem + SMEM_K + c * CHUNK_BYTES, &tmap_k, g * HD + c * 64, tok0 + jb * BKV, kv_full);
                    ptx::tma_load_2d(smem + SMEM_V + c * CHUNK_BYTES, &tmap_v, g * HD + c * 64, tok0 + jb * BKV, kv_full);
                }
            } else {
                ptx::tma_prefetch_desc(&tmap_do);
            }
        }
        uint64_t* full = q_role ? q_full : do_full;
        uint64_t* empty = q_role ? q_empty : do_empty;
        const CUtensorMap* tmap = q_role ? &tmap_q : &tmap_do;
        uint8_t* ring = smem + (q_role ? SMEM_Q : SMEM_DO);
        int hl = 0, ib = jb;  // query head inside the group, query block
        int issued = 0;
        for (int it = 0; it < n_it; ++it) {
            const int st = q_role ? (it & 1) : 0;                        // Q: two slots, dO: one
            const uint32_t ph = q_role ? ((it >> 1) & 1) : (it & 1);
            const int h = g * G + hl;
            const long long tq = BWD_PROF_T();
            if (!ptx::mbar_wait_bounded(&empty[st], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
            pc[0] += BWD_PROF_T() - tq;
            if (lane == 0) {
                ptx::mbar_expect_tx(&full[st], TILE_BYTES);
                for (int c = 0; c < 2; ++c)
                    ptx::tma_load_2d(ring + st * TILE_BYTES + c * CHUNK_BYTES, tmap, h * HD + c * 64, tok0 + ib * BQ, &full[st]);
            }
            if (q_role) {
                // L (log2 units) and D of the 128 queries; rows past the end of the sequence get L = +inf (P = 0).
                // The slot is free when the Q slot is: both are last read before dK of the block that used them.
                float* lrow = ld_smem + st * 256;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int e = m * 32 + lane;
                    const int qi = ib * BQ + e;
                    float l2 = INFINITY, dd = 0.f;
                    if (qi < seqlen) {
                        const int64_t off = (int64_t)h * p.T + tok0 + qi;
                        l2 = p.lse2[off];
                        dd = p.dsum[off];
                    }
                    lrow[e] = l2;
                    lrow[128 + e] = dd;
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ld_full[st]);
            }
            issued = it + 1;
            if (++ib == nq) { ib = jb; ++hl; }
        }
        if (!ok && lane == 0) {
            atomicCAS(p.error_flag, 0, (0x28 << 8) | 2);
            // copies already issued still land in this CTA's shared memory: give them time before the CTA retires
            const uint64_t t0 = ptx::globaltimer_ns();
            for (int k = max(0, issued - (q_role ? 2 : 1)); k < issued; ++k) {
                uint64_t* bar = q_role ? &full[k & 1] : &full[0];
                const uint32_t ph = q_role ? ((k >> 1) & 1) : (k & 1);
                while (!ptx::mbar_try_wait(bar, ph)) {
                    if (ptx::globaltimer_ns() - t0 > 100000000ull) break;
                }
            }
        }
        if (prof_on) p.prof[q_role ? 0 : 1] += pc[0];
    } else if (warp == 1) {
        // ------------------------------------------------------------------ tensor-core issue
        if (lane == 0) {
            constexpr uint32_t idesc_kk = ptx::make_idesc_bf16(128, 128, false, false);  // S^T, dP^T
            constexpr uint32_t idesc_kn = ptx::make_idesc_bf16(128, 128, false, true);   // dV, dK
            constexpr uint32_t idesc_nn = ptx::make_idesc_bf16(128, 128, true, true);    // dQ
            // Descriptors differ only in the start address (bits 0-13, in 16-byte units): build one per tile and
            // operand form here, add offsets in the loop.  K-major form: rows of 128 bytes, one K step = 32 bytes inside
            // a 64-element chunk; MN-major form: one K step = 16 rows = 2048 bytes, the two 64-wide halves one chunk apart.
            auto kmaj = [&](int off) { return ptx::make_smem_desc_sw128(ptx::smem_u32(smem + off), 16, 1024); };
            auto mnmaj = [&](int off) { return ptx::make_smem_desc_sw128(ptx::smem_u32(smem + off), CHUNK_BYTES, 1024); };
            const uint64_t k_km = kmaj(SMEM_K), k_mn = mnmaj(SMEM_K), v_km = kmaj(SMEM_V);
            const uint64_t ds_km = kmaj(SMEM_DS), ds_mn = mnmaj(SMEM_DS);
            const uint64_t q_km0 = kmaj(SMEM_Q), q_mn0 = mnmaj(SMEM_Q), do_km0 = kmaj(SMEM_DO), do_mn0 = mnmaj(SMEM_DO);
            constexpr uint64_t kStage = TILE_BYTES >> 4;  // second ring slot, in descriptor address units
            // both operands K-major: D[128 x 128] = A[128 x 128 (d)] B[128 x 128 (d)]^T
            auto mma_kk = [&](uint32_t d, uint64_t a, uint64_t b) {
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = ((k >> 2) * CHUNK_BYTES + (k & 3) * 32) >> 4;
                    ptx::mma_bf16_ss(tmem_base + d, a + off, b + off, idesc_kk, k != 0);
                }
            };
            auto issue_s = [&](int it) -> bool {  // S^T = K Q^T
                const long long t0 = BWD_PROF_T();
                if (!ptx::mbar_wait_bounded(&q_full[it & 1], (it >> 1) & 1, abort_flag, kWaitNs)) return false;
                pc[0] += BWD_PROF_T() - t0;
                ptx::tc_fence_after();
                mma_kk(TM_S, k_km, q_km0 + (it & 1) * kStage);
                ptx::mma_commit(s_full);
                return true;
            };
            auto issue_dp = [&](int it) -> bool {  // dP^T = V dO^T, into the columns dQ(it-1) was drained from
                const long long t0 = BWD_PROF_T();
                if (!ptx::mbar_wait_bounded(do_full, it & 1, abort_flag, kWaitNs)) return false;
                pc[1] += BWD_PROF_T() - t0;
                const long long t1 = BWD_PROF_T();
                if (it > 0 && !ptx::mbar_wait_bounded(dq_free, (it - 1) & 1, abort_flag, kWaitNs)) return false;
                pc[2] += BWD_PROF_T() - t1;
                ptx::tc_fence_after();
                mma_kk(TM_DP, v_km, do_km0);
                ptx::mma_commit(dp_full);
                return true;
            };
            auto issue_dv = [&](int it) -> bool {  // dV += P^T dO, A from tensor memory; dO(it) is free afterwards
                const long long t0 = BWD_PROF_T();
                if (!ptx::mbar_wait_bounded(p_ready, it & 1, abort_flag, kWaitNs)) return false;
                pc[3] += BWD_PROF_T() - t0;
                ptx::tc_fence_after();
                const uint64_t dos = do_mn0;
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)
                    ptx::mma_bf16_ts(tmem_base + TM_DV, tmem_base + TM_S + (k >> 2) * 64 + (k & 3) * 8, dos + k * 128, idesc_kn,
                                     (it > 0 || k != 0) ? 1u : 0u);
                ptx::mma_commit(do_empty);
                return true;
            };
            auto issue_dq_dk = [&](int it) -> bool {  // dQ = dS K (drained while dK runs) ; dK += dS^T Q
                const long long t0 = BWD_PROF_T();
                if (!ptx::mbar_wait_bounded(ds_ready, it & 1, abort_flag, kWaitNs)) return false;
                pc[4] += BWD_PROF_T() - t0;
                ptx::tc_fence_after();
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)
                    ptx::mma_bf16_ss(tmem_base + TM_DP, ds_mn + k * 128, k_mn + k * 128, idesc_nn, k != 0);
                ptx::mma_commit(dq_full);
                const uint64_t qs = q_mn0 + (it & 1) * kStage;
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k) {
                    const uint32_t aoff = ((k >> 2) * CHUNK_BYTES + (k & 3) * 32) >> 4;
                    ptx::mma_bf16_ss(tmem_base + TM_DK, ds_km + aoff, qs + k * 128, idesc_kn, (it > 0 || k != 0) ? 1u : 0u);
                }
                ptx::mma_commit(&q_empty[it & 1]);  // Q(it) was read by S(it) and dK(it)
                ptx::mma_commit(ds_free);
                return true;
            };
            const long long tall = BWD_PROF_T();
            bool ok = ptx::mbar_wait_bounded(kv_full, 0, abort_flag, kWaitNs);
            if (ok) ok = issue_s(0);
            if (ok) ok = issue_dp(0);
            if (ok) ok = issue_dv(0);
            if (ok && n_it > 1) ok = issue_s(1);
            for (int it = 0; it < n_it && ok; ++it) {
                ok = issue_dq_dk(it);
                if (ok && it + 1 < n_it) {
                    ok = issue_dp(it + 1);
                    if (ok) ok = issue_dv(it + 1);
                }
                if (ok && it + 2 < n_it) ok = issue_s(it + 2);
            }
            if (ok) ptx::mma_commit(acc_done);
            else atomicCAS(p.error_flag, 0, (0x28 << 8) | 3);
            if (prof_on) {
                for (int i = 0; i < 5; ++i) p.prof[4 + i] += pc[i];
                p.prof[9] += clock64() - tall;
                p.prof[10] += n_it;
            }
        }
    } else if (warp >= kScoreWarp0 && warp < kDrainWarp0) {
        // ------------------------------------------------------------------ S^T -> P^T, dP^T -> dS^T, final dK / dV
        // Two groups of four warps; group cg owns the query columns [64 cg, 64 cg + 64) of every block.
        const int cg = (warp - kScoreWarp0) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // key row of the block owned by this thread
        const int kr = jb * BKV + r;        // position inside the sequence
        const bool row_valid = kr < seqlen;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint8_t* ds_row = smem + SMEM_DS + cg * CHUNK_BYTES + r * 128;  // the group's 64-query chunk of dS^T
        const bool tail_block = jb * BKV + BKV > seqlen;  // some key rows of this block lie past the end
        const int col0 = cg * 64;
        bool ok = true;
        int ib = jb;
        uint32_t pk[32];  // the group's half of the P^T row as packed bf16 pairs
        // one 16-column chunk of scores -> probabilities; mask: diagonal block or key rows past the end
        auto p_chunk = [&](const uint32_t (&s)[16], const float* l2s, int c, int lim, bool mask) {
#pragma unroll
            for (int k = 0; k < 16; k += 2) {
                const float2 l2 = *reinterpret_cast<const float2*>(l2s + col0 + c * 16 + k);
                float p0 = exp2f(fmaf(__uint_as_float(s[k]), p.scale_log2, -l2.x));
                float p1 = exp2f(fmaf(__uint_as_float(s[k + 1]), p.scale_log2, -l2.y));
                if (mask) {
                    if (col0 + c * 16 + k < lim) p0 = 0.f;
                    if (col0 + c * 16 + k + 1 < lim) p1 = 0.f;
                }
                const bf162 b = __floats2bfloat162_rn(p0, p1);
                pk[c * 8 + (k >> 1)] = *reinterpret_cast<const uint32_t*>(&b);
            }
        };
        auto ds_chunk = [&](const uint32_t (&dp)[16], const float* dds, int c) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {  // 16-byte units of 8 queries
                float f8[8];
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    const int col = c * 16 + u * 8 + k;  // inside the group's 64 columns
                    const float2 dd = *reinterpret_cast<const float2*>(dds + col0 + col);
                    const uint32_t w = pk[col >> 1];
                    f8[k] = __uint_as_float(w << 16) * (__uint_as_float(dp[u * 8 + k]) - dd.x);
                    f8[k + 1] = __uint_as_float(w & 0xffff0000u) * (__uint_as_float(dp[u * 8 + k + 1]) - dd.y);
                }
                const int unit = c * 2 + u;  // 0..7 inside the chunk
                *reinterpret_cast<bf16x8*>(ds_row + ((unit ^ (r & 7)) << 4)) = pack8(f8);
            }
        };
        for (int it = 0; it < n_it && ok; ++it) {
            const int st = it & 1;
            const uint32_t ph = it & 1;
            const float* l2s = ld_smem + st * 256;
            const float* dds = l2s + 128;
            // columns (queries of the block) below `lim` are masked for this key row
            const int lim = !row_valid ? 128 : (ib == jb ? r : 0);
            const bool mask = tail_block || ib == jb;  // uniform for the CTA
            const long long ta = BWD_PROF_T();
            if (!ptx::mbar_wait_bounded(&ld_full[st], (it >> 1) & 1, abort_flag, kWaitNs)) { ok = false; break; }
            if (!ptx::mbar_wait_bounded(s_full, ph, abort_flag, kWaitNs)) { ok = false; break; }
            pc[0] += BWD_PROF_T() - ta;
            const long long tb = BWD_PROF_T();
            ptx::tc_fence_after();
            {
                // the load of the next chunk is in flight while this one is turned into probabilities
                uint32_t s0[16], s1[16];
                const uint32_t sa = tmem_base + lane_addr + TM_S + col0;
                ptx::tmem_ld_32x32b_x16(sa, s0);
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x32b_x16(sa + (c + 1) * 16, s1);
                    p_chunk(s0, l2s, c, lim, mask);
                    ptx::tmem_ld_wait();
                    if (c + 2 < 4) ptx::tmem_ld_32x32b_x16(sa + (c + 2) * 16, s0);
                    p_chunk(s1, l2s, c + 1, lim, mask);
                }
            }
            // the group's scores have been read: its half of P^T overwrites the first 32 of its own 64 columns
            ptx::tmem_st_32x32b_x32(tmem_base + lane_addr + TM_S + col0, pk);
            ptx::tmem_st_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_ready);
            pc[1] += BWD_PROF_T() - tb;

            const long long tc = BWD_PROF_T();
            if (!ptx::mbar_wait_bounded(dp_full, ph, abort_flag, kWaitNs)) { ok = false; break; }
            pc[2] += BWD_PROF_T() - tc;
            const long long td = BWD_PROF_T();
            if (it > 0 && !ptx::mbar_wait_bounded(ds_free, (it - 1) & 1, abort_flag, kWaitNs)) { ok = false; break; }
            pc[3] += BWD_PROF_T() - td;
            const long long te = BWD_PROF_T();
            ptx::tc_fence_after();
            {
                uint32_t d0[16], d1[16];
                const uint32_t da = tmem_base + lane_addr + TM_DP + col0;
                ptx::tmem_ld_32x32b_x16(da, d0);
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x32b_x16(da + (c + 1) * 16, d1);
                    ds_chunk(d0, dds, c);
                    ptx::tmem_ld_wait();
                    if (c + 2 < 4) ptx::tmem_ld_32x32b_x16(da + (c + 2) * 16, d0);
                    ds_chunk(d1, dds, c + 1);
                }
            }
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();  // generic-proxy writes of dS^T become visible to the tensor core
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ds_ready);
            pc[4] += BWD_PROF_T() - te;
            if (++ib == nq) ib = jb;
        }
        if (prof_on)
            for (int i = 0; i < 5; ++i) p.prof[12 + i] += pc[i];
        if (ok && !ptx::mbar_wait_bounded(acc_done, 0, abort_flag, kWaitNs)) ok = false;
        if (!ok) {
            if (lane == 0) atomicCAS(p.error_flag, 0, (0x28 << 8) | 4);
        } else {
            // group 0 stores dV, group 1 dK (times the softmax scale)
            ptx::tc_fence_after();
            bf16* dst = (cg == 0 ? p.dv : p.dk) + (int64_t)(tok0 + kr) * p.dkv_row_stride + (int64_t)g * HD;
            const float mul = cg == 0 ? 1.f : p.scale;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t a[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + (cg == 0 ? TM_DV : TM_DK) + c * 32, a);
                ptx::tmem_ld_wait();
                if (row_valid) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float f8[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) f8[k] = __uint_as_float(a[u * 8 + k]) * mul;
                        *reinterpret_cast<bf16x8*>(dst + c * 32 + u * 8) = pack8(f8);
                    }
                }
            }
        }
    } else if (warp >= kDrainWarp0) {
        // ------------------------------------------------------------------ dQ: tensor memory -> shared memory -> TMA add
        // A thread owns a query row.  Two chunks of 32 head-dim columns at a time go through the two staging buffers
        // (rows of 128 bytes in the 128-byte swizzle the tensor map expects); one thread then hands both to the TMA
        // unit, which adds them to the fp32 accumulator.  Rows past the end of the sequence carry exact zeros (their
        // probabilities are zero), rows past the end of the tensor are clipped by the tensor map.
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const bool elected = warp == kDrainWarp0 && lane == 0;
        uint8_t* buf0 = smem + SMEM_DQ + r * 128;
        uint8_t* buf1 = buf0 + DQ_BUF_BYTES;
        bool ok = true;
        int hl = 0, ib = jb;
        if (elected) ptx::tma_prefetch_desc(&tmap_dq);
        for (int it = 0; it < n_it; ++it) {
            const long long ta = BWD_PROF_T();
            if (!ptx::mbar_wait_bounded(dq_full, it & 1, abort_flag, kWaitNs)) { ok = false; break; }
            pc[0] += BWD_PROF_T() - ta;
            ptx::tc_fence_after();
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const long long tb = BWD_PROF_T();
                uint32_t a0[32], a1[32];
                const uint32_t src = tmem_base + lane_addr + TM_DP + half * 64;
                ptx::tmem_ld_32x32b_x32(src, a0);
                ptx::tmem_ld_32x32b_x32(src + 32, a1);
                ptx::tmem_ld_wait();
                if (half == 1) {  // all of dQ is in registers or staged: the columns may take the next dP^T
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(dq_free);
                }
                pc[1] += BWD_PROF_T() - tb;
                const long long tc = BWD_PROF_T();
                // the reductions issued from these buffers (if any) must have finished reading them
                if (elected) ptx::bulk_wait_read<0>();
                ptx::named_barrier_sync(1, 128);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int sw = (u ^ (r & 7)) << 4;
                    *reinterpret_cast<uint4*>(buf0 + sw) = make_uint4(a0[4 * u], a0[4 * u + 1], a0[4 * u + 2], a0[4 * u + 3]);
                    *reinterpret_cast<uint4*>(buf1 + sw) = make_uint4(a1[4 * u], a1[4 * u + 1], a1[4 * u + 2], a1[4 * u + 3]);
                }
                ptx::fence_proxy_async_smem();
                ptx::named_barrier_sync(1, 128);
                if (elected && !(p.debug_flags & 1)) {
                    const int x = (g * G + hl) * HD + half * 64, y = tok0 + ib * BQ;
                    ptx::tma_reduce_add_2d(&tmap_dq, smem + SMEM_DQ, x, y);
                    ptx::tma_reduce_add_2d(&tmap_dq, smem + SMEM_DQ + DQ_BUF_BYTES, x + 32, y);
                    ptx::bulk_commit();
                }
                pc[2] += BWD_PROF_T() - tc;
            }
            if (++ib == nq) { ib = jb; ++hl; }
        }
        if (elected) ptx::bulk_wait<0>();  // every reduction has completed before the CTA (and its shared memory) goes away
        if (!ok && lane == 0) atomicCAS(p.error_flag, 0, (0x28 << 8) | 5);
        if (prof_on)
            for (int i = 0; i < 3; ++i) p.prof[20 + i] += pc[i];
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

// One warp per (token, head): D = sum_d dO * O, and the forward's natural-log L converted to log2 units.
__global__ void fmha_bwd_prep_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, const float* __restrict__ lse,
                                     float* __restrict__ lse2, float* __restrict__ dsum, int64_t T, int Hq,
                                     int64_t o_stride, int64_t do_stride) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= T * Hq) return;
    const int lane = threadIdx.x & 31;
    const int64_t t = row / Hq;
    const int h = (int)(row - t * Hq);
    const uint2 a = *reinterpret_cast<const uint2*>(o + t * o_stride + (int64_t)h * HD + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(dout + t * do_stride + (int64_t)h * HD + lane * 4);
    const float2 a0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&a.x));
    const float2 a1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&a.y));
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&b.y));
    float acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
    acc = warp_sum(acc);
    if (lane == 0) {
        const int64_t off = (int64_t)h * T + t;
        dsum[off] = acc;
        lse2[off] = lse[off] * 1.4426950408889634f;
    }
}

// dQ: fp32 accumulator [T, row8 * 8] -> bf16 rows of ``dq_row_stride`` elements, times the softmax scale.
__global__ void fmha_bwd_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int64_t n8, int64_t row8,
                                           int64_t dq_row_stride, float scale) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const float4 x = reinterpret_cast<const float4*>(acc)[2 * i];
        const float4 y = reinterpret_cast<const float4*>(acc)[2 * i + 1];
        const float f8[8] = {x.x * scale, x.y * scale, x.z * scale, x.w * scale, y.x * scale, y.y * scale, y.z * scale, y.w * scale};
        const int64_t t = i / row8;
        const int64_t c8 = i - t * row8;
        *reinterpret_cast<bf16x8*>(dq + t * dq_row_stride + c8 * 8) = pack8(f8);
    }
}

}  // namespace

static at::Tensor& bwd_profile_buffer(const at::Device& dev) {
    static std::vector<at::Tensor> bufs(64);
    auto& b = bufs[dev.index() < 0 ? 0 : dev.index()];
    if (!b.defined()) b = at::zeros({32}, at::TensorOptions().dtype(at::kLong).device(dev));
    return b;
}

// Cycle counters of the first CTA of the backward launches made while ATB200_FMHA_BWD_PROFILE was set (then cleared).
at::Tensor fmha_bwd_read_profile(const at::Tensor& like) {
    auto& b = bwd_profile_buffer(like.device());
    auto out = b.cpu();
    b.zero_();
    return out;
}

// dout / out [T, Hq, 128], q [T, Hq, 128], k / v [T, Hkv, 128] bf16 (q, k, v may be views of a fused projection),
// lse [Hq, T] fp32 as written by fmha_fwd, cu_seqlens int32 [nseq + 1].  Returns (dq, dk, dv): contiguous tensors, or,
// when ``packed`` is set, views of one new [T, (Hq + 2 Hkv) * 128] tensor laid out like a fused q|k|v projection (its
// gradient then needs no concatenation).
std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                                         const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                                         const at::Tensor& cu_seqlens, int64_t max_blocks, double softmax_scale,
                                                         bool packed) {
    ATB_CHECK_CUDA(q);
    for (const at::Tensor* t : {&dout, &q, &k, &v, &out}) {
        TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->dim() == 3 && t->size(2) == HD, "fmha_bwd: bf16 [tokens, heads, 128] expected");
        TORCH_CHECK(t->stride(2) == 1 && t->stride(1) == HD && t->stride(0) % 8 == 0, "fmha_bwd: heads must be dense, token stride % 8 == 0");
        TORCH_CHECK((reinterpret_cast<uintptr_t>(t->data_ptr()) & 15) == 0, "fmha_bwd: operands must be 16-byte aligned");
    }
    ATB_CHECK_DTYPE(cu_seqlens, at::kInt); ATB_CHECK_CONTIG(cu_seqlens);
    ATB_CHECK_DTYPE(lse, at::kFloat); ATB_CHECK_CONTIG(lse);
    const int64_t T = q.size(0);
    const int Hq = (int)q.size(1), Hkv = (int)k.size(1);
    TORCH_CHECK(k.size(0) == T && v.size(0) == T && v.size(1) == Hkv && Hq % Hkv == 0 && dout.size(0) == T && dout.size(1) == Hq &&
                out.size(0) == T && out.size(1) == Hq && lse.numel() == (int64_t)Hq * T, "fmha_bwd: inconsistent shapes");
    TORCH_CHECK(T < (1ll << 31) - 256, "fmha_bwd: too many tokens for 32-bit tile coordinates");
    const int nseq = (int)cu_seqlens.numel() - 1;
    TORCH_CHECK(nseq >= 1 && max_blocks >= 1 && max_blocks <= 65535, "fmha_bwd: need 1 .. 65535 key blocks");
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor dq, dk, dv;
    if (packed) {
        auto all = at::empty({T, (int64_t)(Hq + 2 * Hkv), HD}, q.options());
        dq = all.narrow(1, 0, Hq);
        dk = all.narrow(1, Hq, Hkv);
        dv = all.narrow(1, Hq + Hkv, Hkv);
    } else {
        dq = at::empty({T, Hq, HD}, q.options());
        dk = at::empty({T, Hkv, HD}, q.options());
        dv = at::empty({T, Hkv, HD}, q.options());
    }
    if (T == 0) return {dq, dk, dv};
    auto fopt = q.options().dtype(at::kFloat);
    auto dq_acc = at::zeros({T, Hq, HD}, fopt);
    auto lse2 = at::empty({Hq, T}, fopt);
    auto dsum = at::empty({Hq, T}, fopt);
    auto stream = current_stream();
    {
        const int64_t rows = T * Hq;
        fmha_bwd_prep_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, stream>>>(
            (const bf16*)out.data_ptr(), (const bf16*)dout.data_ptr(), lse.data_ptr<float>(), lse2.data_ptr<float>(),
            dsum.data_ptr<float>(), T, Hq, out.stride(0), dout.stride(0));
        ATB_LAUNCH_CHECK();
    }
    const CUtensorMap tq = make_tmap_bf16_public(q.data_ptr(), T, (int64_t)Hq * HD, q.stride(0), BQ);
    const CUtensorMap tk = make_tmap_bf16_public(k.data_ptr(), T, (int64_t)Hkv * HD, k.stride(0), BKV);
    const CUtensorMap tv = make_tmap_bf16_public(v.data_ptr(), T, (int64_t)Hkv * HD, v.stride(0), BKV);
    const CUtensorMap tdo = make_tmap_bf16_public(dout.data_ptr(), T, (int64_t)Hq * HD, dout.stride(0), BQ);
    const CUtensorMap tdq = make_tmap_f32_public(dq_acc.data_ptr(), T, (int64_t)Hq * HD, (int64_t)Hq * HD, BQ);
    BwdParams p;
    p.lse2 = lse2.data_ptr<float>();
    p.dsum = dsum.data_ptr<float>();
    p.dk = (bf16*)dk.data_ptr();
    p.dv = (bf16*)dv.data_ptr();
    p.dkv_row_stride = dk.stride(0);
    p.cu_seqlens = cu_seqlens.data_ptr<int>();
    p.nseq = nseq; p.T = (int)T; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = (float)softmax_scale;
    p.scale_log2 = (float)(softmax_scale * 1.4426950408889634);
    p.error_flag = gemm_error_flag(q.device()).data_ptr<int>();
    p.prof = nullptr;
    p.debug_flags = 0;
    if (const char* dbg = std::getenv("ATB200_FMHA_BWD_DEBUG")) p.debug_flags = std::atoi(dbg);
    if (std::getenv("ATB200_FMHA_BWD_PROFILE")) p.prof = reinterpret_cast<long long*>(bwd_profile_buffer(q.device()).data_ptr<int64_t>());
    static bool attr_set = false;
    if (!attr_set) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(fmha_bwd_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr_set = true;
    }
    dim3 grid((unsigned)Hkv, (unsigned)max_blocks);
    fmha_bwd_tcgen05_kernel<<<grid, kThreads, SMEM_TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);
    ATB_LAUNCH_CHECK();
    {
        const int64_t n8 = T * Hq * HD / 8;
        const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n8, 256), 148 * 16);
        fmha_bwd_dq_convert_kernel<<<blocks, 256, 0, stream>>>(dq_acc.data_ptr<float>(), (bf16*)dq.data_ptr(), n8,
                                                               (int64_t)Hq * HD / 8, dq.stride(0), (float)softmax_scale);
        ATB_LAUNCH_CHECK();
    }
    return {dq, dk, dv};
}

}  // namespace atb
