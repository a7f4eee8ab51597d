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
// added to an fp32 accumulator in global memory with 16-byte reductions (the order of these additions is not fixed;
// dQ is reproducible to fp32 rounding only) and converted to bf16, times the softmax scale, by a small kernel.
//
// Roles: warp 0 loads (TMA for K, V and the Q / dO rings; plain loads for L and D), warp 1 issues the tensor-core
// products, warps 2-5 turn S^T into P^T and dP^T into dS^T, warps 6-9 drain dQ.  Issue order per query block i:
//   dK(i) dQ(i) | dV(i+1) dP(i+1) | S(i+2)
// so that the exponentials of block i+1 run under dK / dQ of block i and the drain of dQ(i) runs under dV(i+1).
// All barrier waits are bounded.
//
// The reference obtains the attention backward from the flash-attn package or PyTorch SDPA through Hugging Face
// (arctic_training/config/model.py:48,85-98).

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>

namespace atb {

CUtensorMap make_tmap_bf16_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
at::Tensor& gemm_error_flag(const at::Device& dev);

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int CHUNK_BYTES = 128 * 128;       // [128 rows][64 bf16]
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;  // 128 x 128 bf16
constexpr int SMEM_K = 0;
constexpr int SMEM_V = TILE_BYTES;
constexpr int SMEM_Q = 2 * TILE_BYTES;    // two stages
constexpr int SMEM_DO = 4 * TILE_BYTES;   // two stages
constexpr int SMEM_DS = 6 * TILE_BYTES;   // dS^T of the current query block
constexpr int SMEM_LD = 7 * TILE_BYTES;   // float [2 stages][2][128]: L * log2(e) and D of the stage's query block
constexpr int SMEM_BAR = SMEM_LD + 2 * 2 * 128 * 4;
constexpr int SMEM_TOTAL = SMEM_BAR + 32 * 8;
static_assert(SMEM_TOTAL <= 232448, "shared memory budget of one CTA");
constexpr uint64_t kWaitNs = 2000000000ull;
constexpr int kThreads = 320;  // load warp, MMA warp, four score warps, four dQ warps
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 384;

struct BwdParams {
    const float* lse2;  // [Hq, T]  log-sum-exp in log2 units
    const float* dsum;  // [Hq, T]  rowsum(dO o O)
    float* dq_acc;      // [T, Hq, 128] fp32, zero on entry
    bf16* dk;           // [T, Hkv, 128]
    bf16* dv;
    const int* cu_seqlens;
    int nseq, T, Hq, Hkv;
    float scale, scale_log2;
    int* error_flag;
};

__global__ void __launch_bounds__(kThreads, 1)
fmha_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                        const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
    uint64_t* kv_full = bars;         // 1
    uint64_t* q_full = bars + 1;      // [2]
    uint64_t* q_empty = bars + 3;     // [2]
    uint64_t* do_full = bars + 5;     // [2]
    uint64_t* do_empty = bars + 7;    // [2]
    uint64_t* ld_full = bars + 9;     // [2]  L and D of the stage are in shared memory
    uint64_t* s_full = bars + 11;     // S^T of the block is in tensor memory
    uint64_t* p_ready = bars + 12;    // P^T is back in tensor memory (4 warps)
    uint64_t* dp_full = bars + 13;    // dP^T is in tensor memory
    uint64_t* ds_ready = bars + 14;   // dS^T is in shared memory (4 warps)
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
            ptx::mbar_init(&do_full[i], 1);
            ptx::mbar_init(&do_empty[i], 1);
            ptx::mbar_init(&ld_full[i], 1);
        }
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(p_ready, 4);
        ptx::mbar_init(dp_full, 1);
        ptx::mbar_init(ds_ready, 4);
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

    if (warp == 0) {
        // ------------------------------------------------------------------ loads
        bool ok = true;
        if (lane == 0) {
            ptx::tma_prefetch_desc(&tmap_q);
            ptx::tma_prefetch_desc(&tmap_k);
            ptx::tma_prefetch_desc(&tmap_v);
            ptx::tma_prefetch_desc(&tmap_do);
            ptx::mbar_expect_tx(kv_full, 2 * TILE_BYTES);
            for (int c = 0; c < 2; ++c) {
                ptx::tma_load_2d(smem + SMEM_K + c * CHUNK_BYTES, &tmap_k, g * HD + c * 64, tok0 + jb * BKV, kv_full);
                ptx::tma_load_2d(smem + SMEM_V + c * CHUNK_BYTES, &tmap_v, g * HD + c * 64, tok0 + jb * BKV, kv_full);
            }
        }
        int hl = 0, ib = jb;  // query head inside the group, query block
        int issued = 0;
        for (int it = 0; it < n_it; ++it) {
            const int st = it & 1;
            const uint32_t ph = (it >> 1) & 1;
            const int h = g * G + hl;
            if (!ptx::mbar_wait_bounded(&q_empty[st], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
            if (lane == 0) {
                ptx::mbar_expect_tx(&q_full[st], TILE_BYTES);
                for (int c = 0; c < 2; ++c)
                    ptx::tma_load_2d(smem + SMEM_Q + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_q, h * HD + c * 64,
                                     tok0 + ib * BQ, &q_full[st]);
            }
            // L (log2 units) and D of the 128 queries; rows past the end of the sequence get L = +inf (P = 0)
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
            if (!ptx::mbar_wait_bounded(&do_empty[st], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
            if (lane == 0) {
                ptx::mbar_expect_tx(&do_full[st], TILE_BYTES);
                for (int c = 0; c < 2; ++c)
                    ptx::tma_load_2d(smem + SMEM_DO + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_do, h * HD + c * 64,
                                     tok0 + ib * BQ, &do_full[st]);
            }
            issued = it + 1;
            if (++ib == nq) { ib = jb; ++hl; }
        }
        if (!ok && lane == 0) {
            atomicCAS(p.error_flag, 0, (0x28 << 8) | 2);
            // copies already issued still land in this CTA's shared memory: give them time before the CTA retires
            const uint64_t t0 = ptx::globaltimer_ns();
            for (int k = max(0, issued - 2); k < issued; ++k) {
                const int st = k & 1;
                const uint32_t ph = (k >> 1) & 1;
                while (!(ptx::mbar_try_wait(&q_full[st], ph) && ptx::mbar_try_wait(&do_full[st], ph))) {
                    if (ptx::globaltimer_ns() - t0 > 100000000ull) break;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ tensor-core issue
        if (lane == 0) {
            constexpr uint32_t idesc_kk = ptx::make_idesc_bf16(128, 128, false, false);  // S^T, dP^T
            constexpr uint32_t idesc_kn = ptx::make_idesc_bf16(128, 128, false, true);   // dV, dK
            constexpr uint32_t idesc_nn = ptx::make_idesc_bf16(128, 128, true, true);    // dQ
            const uint32_t ks = ptx::smem_u32(smem + SMEM_K), vs = ptx::smem_u32(smem + SMEM_V);
            const uint32_t dss = ptx::smem_u32(smem + SMEM_DS);
            auto q_addr = [&](int it) { return ptx::smem_u32(smem + SMEM_Q + (it & 1) * TILE_BYTES); };
            auto do_addr = [&](int it) { return ptx::smem_u32(smem + SMEM_DO + (it & 1) * TILE_BYTES); };
            // both operands K-major: D[128 x 128] = A[128 x 128 (d)] B[128 x 128 (d)]^T
            auto mma_kk = [&](uint32_t d, uint32_t a, uint32_t b) {
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_base + d, ptx::make_smem_desc_sw128(a + off, 16, 1024),
                                     ptx::make_smem_desc_sw128(b + off, 16, 1024), idesc_kk, k != 0);
                }
            };
            auto issue_s = [&](int it) -> bool {  // S^T = K Q^T
                if (!ptx::mbar_wait_bounded(&q_full[it & 1], (it >> 1) & 1, abort_flag, kWaitNs)) return false;
                ptx::tc_fence_after();
                mma_kk(TM_S, ks, q_addr(it));
                ptx::mma_commit(s_full);
                return true;
            };
            auto issue_dp = [&](int it) -> bool {  // dP^T = V dO^T, into the columns dQ(it-1) was drained from
                if (!ptx::mbar_wait_bounded(&do_full[it & 1], (it >> 1) & 1, abort_flag, kWaitNs)) return false;
                if (it > 0 && !ptx::mbar_wait_bounded(dq_free, (it - 1) & 1, abort_flag, kWaitNs)) return false;
                ptx::tc_fence_after();
                mma_kk(TM_DP, vs, do_addr(it));
                ptx::mma_commit(dp_full);
                return true;
            };
            auto issue_dv = [&](int it) -> bool {  // dV += P^T dO, A from tensor memory
                if (!ptx::mbar_wait_bounded(p_ready, it & 1, abort_flag, kWaitNs)) return false;
                if (!ptx::mbar_wait_bounded(&do_full[it & 1], (it >> 1) & 1, abort_flag, kWaitNs)) return false;
                ptx::tc_fence_after();
                const uint32_t dos = do_addr(it);
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)
                    ptx::mma_bf16_ts(tmem_base + TM_DV, tmem_base + TM_S + k * 8,
                                     ptx::make_smem_desc_sw128(dos + k * 2048, CHUNK_BYTES, 1024), idesc_kn,
                                     (it > 0 || k != 0) ? 1u : 0u);
                return true;
            };
            auto issue_dk_dq = [&](int it) -> bool {  // dK += dS^T Q ; dQ = dS K
                if (!ptx::mbar_wait_bounded(ds_ready, it & 1, abort_flag, kWaitNs)) return false;
                ptx::tc_fence_after();
                const uint32_t qs = q_addr(it);
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k) {
                    const uint32_t aoff = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_base + TM_DK, ptx::make_smem_desc_sw128(dss + aoff, 16, 1024),
                                     ptx::make_smem_desc_sw128(qs + k * 2048, CHUNK_BYTES, 1024), idesc_kn,
                                     (it > 0 || k != 0) ? 1u : 0u);
                }
                ptx::mma_commit(&q_empty[it & 1]);  // Q(it) was read by S(it) and dK(it)
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)
                    ptx::mma_bf16_ss(tmem_base + TM_DP, ptx::make_smem_desc_sw128(dss + k * 2048, CHUNK_BYTES, 1024),
                                     ptx::make_smem_desc_sw128(ks + k * 2048, CHUNK_BYTES, 1024), idesc_nn, k != 0);
                ptx::mma_commit(ds_free);
                ptx::mma_commit(dq_full);
                return true;
            };
            bool ok = ptx::mbar_wait_bounded(kv_full, 0, abort_flag, kWaitNs);
            if (ok) ok = issue_s(0);
            if (ok) ok = issue_dp(0);
            if (ok) ok = issue_dv(0);
            if (ok) ptx::mma_commit(&do_empty[0]);
            if (ok && n_it > 1) ok = issue_s(1);
            for (int it = 0; it < n_it && ok; ++it) {
                ok = issue_dk_dq(it);
                if (ok && it + 1 < n_it) {
                    ok = issue_dv(it + 1);
                    if (ok) ok = issue_dp(it + 1);
                    if (ok) ptx::mma_commit(&do_empty[(it + 1) & 1]);  // dO(it+1) was read by dV and dP
                }
                if (ok && it + 2 < n_it) ok = issue_s(it + 2);
            }
            if (ok) ptx::mma_commit(acc_done);
            else atomicCAS(p.error_flag, 0, (0x28 << 8) | 3);
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ S^T -> P^T, dP^T -> dS^T, final dK / dV
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // key row of the block owned by this thread
        const int kr = jb * BKV + r;        // position inside the sequence
        const bool row_valid = kr < seqlen;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint8_t* ds_row = smem + SMEM_DS + r * 128;
        bool ok = true;
        int ib = jb;
        for (int it = 0; it < n_it && ok; ++it) {
            const int st = it & 1;
            const uint32_t ph = it & 1;
            const float* l2s = ld_smem + st * 256;
            const float* dds = l2s + 128;
            // columns (queries of the block) below `lim` are masked for this key row
            const int lim = !row_valid ? 128 : (ib == jb ? r : 0);
            if (!ptx::mbar_wait_bounded(&ld_full[st], (it >> 1) & 1, abort_flag, kWaitNs)) { ok = false; break; }
            if (!ptx::mbar_wait_bounded(s_full, ph, abort_flag, kWaitNs)) { ok = false; break; }
            ptx::tc_fence_after();
            uint32_t pk[64];  // P^T row as packed bf16 pairs
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t s[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + TM_S + c * 32, s);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 32; k += 2) {
                    const float2 l2 = *reinterpret_cast<const float2*>(l2s + c * 32 + k);
                    float p0 = exp2f(fmaf(__uint_as_float(s[k]), p.scale_log2, -l2.x));
                    float p1 = exp2f(fmaf(__uint_as_float(s[k + 1]), p.scale_log2, -l2.y));
                    if (c * 32 + k < lim) p0 = 0.f;
                    if (c * 32 + k + 1 < lim) p1 = 0.f;
                    const bf162 b = __floats2bfloat162_rn(p0, p1);
                    pk[c * 16 + (k >> 1)] = *reinterpret_cast<const uint32_t*>(&b);
                }
            }
            // every score has been read: P^T may overwrite the first 64 columns of the S^T buffer
            ptx::tmem_st_32x32b_x32(tmem_base + lane_addr + TM_S, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
            ptx::tmem_st_32x32b_x32(tmem_base + lane_addr + TM_S + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
            ptx::tmem_st_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_ready);

            if (!ptx::mbar_wait_bounded(dp_full, ph, abort_flag, kWaitNs)) { ok = false; break; }
            if (it > 0 && !ptx::mbar_wait_bounded(ds_free, (it - 1) & 1, abort_flag, kWaitNs)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t dp[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + TM_DP + c * 32, dp);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < 4; ++u) {  // 16-byte units of 8 queries
                    float f8[8];
#pragma unroll
                    for (int k = 0; k < 8; k += 2) {
                        const int col = c * 32 + u * 8 + k;
                        const float2 dd = *reinterpret_cast<const float2*>(dds + col);
                        const uint32_t w = pk[col >> 1];
                        f8[k] = __uint_as_float(w << 16) * (__uint_as_float(dp[u * 8 + k]) - dd.x);
                        f8[k + 1] = __uint_as_float(w & 0xffff0000u) * (__uint_as_float(dp[u * 8 + k + 1]) - dd.y);
                    }
                    const int unit = c * 4 + u;
                    *reinterpret_cast<bf16x8*>(ds_row + (unit >> 3) * CHUNK_BYTES + (((unit & 7) ^ (r & 7)) << 4)) = pack8(f8);
                }
            }
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();  // generic-proxy writes of dS^T become visible to the tensor core
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ds_ready);
            if (++ib == nq) ib = jb;
        }
        if (ok && !ptx::mbar_wait_bounded(acc_done, 0, abort_flag, kWaitNs)) ok = false;
        if (!ok) {
            if (lane == 0) atomicCAS(p.error_flag, 0, (0x28 << 8) | 4);
        } else {
            ptx::tc_fence_after();
            const int64_t row_off = ((int64_t)(tok0 + kr) * p.Hkv + g) * HD;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {  // 0: dV, 1: dK (times the softmax scale)
                bf16* dst = (half == 0 ? p.dv : p.dk) + row_off;
                const float mul = half == 0 ? 1.f : p.scale;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t a[32];
                    ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + (half == 0 ? TM_DV : TM_DK) + c * 32, a);
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
        }
    } else {
        // ------------------------------------------------------------------ dQ: tensor memory -> fp32 accumulator
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // query row of the block
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        int hl = 0, ib = jb;
        for (int it = 0; it < n_it; ++it) {
            if (!ptx::mbar_wait_bounded(dq_full, it & 1, abort_flag, kWaitNs)) { ok = false; break; }
            ptx::tc_fence_after();
            uint32_t a[128];
#pragma unroll
            for (int c = 0; c < 4; ++c)
                ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + TM_DP + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&a[c * 32]));
            ptx::tmem_ld_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(dq_free);
            const int qi = ib * BQ + r;
            if (qi < seqlen) {
                float* dst = p.dq_acc + ((int64_t)(tok0 + qi) * p.Hq + (g * G + hl)) * HD;
#pragma unroll
                for (int k = 0; k < 128; k += 4)
                    ptx::red_add_v4_f32(dst + k, __uint_as_float(a[k]), __uint_as_float(a[k + 1]), __uint_as_float(a[k + 2]),
                                        __uint_as_float(a[k + 3]));
            }
            if (++ib == nq) { ib = jb; ++hl; }
        }
        if (!ok && lane == 0) atomicCAS(p.error_flag, 0, (0x28 << 8) | 5);
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

// dQ: fp32 accumulator -> bf16, times the softmax scale.
__global__ void fmha_bwd_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int64_t n8, float scale) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const float4 x = reinterpret_cast<const float4*>(acc)[2 * i];
        const float4 y = reinterpret_cast<const float4*>(acc)[2 * i + 1];
        const float f8[8] = {x.x * scale, x.y * scale, x.z * scale, x.w * scale, y.x * scale, y.y * scale, y.z * scale, y.w * scale};
        reinterpret_cast<bf16x8*>(dq)[i] = pack8(f8);
    }
}

}  // namespace

// dout / out [T, Hq, 128], q [T, Hq, 128], k / v [T, Hkv, 128] bf16 (q, k, v may be views of a fused projection),
// lse [Hq, T] fp32 as written by fmha_fwd, cu_seqlens int32 [nseq + 1].  Returns (dq, dk, dv), contiguous.
std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                                         const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                                         const at::Tensor& cu_seqlens, int64_t max_blocks, double softmax_scale) {
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
    auto dq = at::empty({T, Hq, HD}, q.options());
    auto dk = at::empty({T, Hkv, HD}, q.options());
    auto dv = at::empty({T, Hkv, HD}, q.options());
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
    BwdParams p;
    p.lse2 = lse2.data_ptr<float>();
    p.dsum = dsum.data_ptr<float>();
    p.dq_acc = dq_acc.data_ptr<float>();
    p.dk = (bf16*)dk.data_ptr();
    p.dv = (bf16*)dv.data_ptr();
    p.cu_seqlens = cu_seqlens.data_ptr<int>();
    p.nseq = nseq; p.T = (int)T; p.Hq = Hq; p.Hkv = Hkv;
    p.scale = (float)softmax_scale;
    p.scale_log2 = (float)(softmax_scale * 1.4426950408889634);
    p.error_flag = gemm_error_flag(q.device()).data_ptr<int>();
    static bool attr_set = false;
    if (!attr_set) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(fmha_bwd_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr_set = true;
    }
    dim3 grid((unsigned)Hkv, (unsigned)max_blocks);
    fmha_bwd_tcgen05_kernel<<<grid, kThreads, SMEM_TOTAL, stream>>>(tq, tk, tv, tdo, p);
    ATB_LAUNCH_CHECK();
    {
        const int64_t n8 = T * Hq * HD / 8;
        const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n8, 256), 148 * 16);
        fmha_bwd_dq_convert_kernel<<<blocks, 256, 0, stream>>>(dq_acc.data_ptr<float>(), (bf16*)dq.data_ptr(), n8, (float)softmax_scale);
        ATB_LAUNCH_CHECK();
    }
    return {dq, dk, dv};
}

}  // namespace atb
