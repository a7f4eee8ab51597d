// SPDX-License-Identifier: Apache-2.0
// Causal flash-attention forward for sm_100a: packed (variable-length) sequences, grouped-query heads, head_dim 128.
//
//   O[t, h, :] = softmax_j<=t ( Q[t, h, :] . K[j, g(h), :] * scale ) V[j, g(h), :]     within each packed sequence
//
// One CTA per (sequence, block of 128 queries, query head).  Warp 0 streams K and V blocks of 128 keys with TMA into
// two-stage rings (K and V have their own barriers: a K slot is free again as soon as its scores are computed), warp 1
// issues the GEMMs on the tensor cores, and two groups of four warps do the softmax: group 0 takes the even key blocks,
// group 1 the odd ones.  Each group has its own score buffer and its own output accumulator in TMEM (4 x 128 columns),
// its own running maximum / sum and its own probability tile in shared memory, so the groups never wait for one another
// and the exponentials of one block overlap the barrier latencies and GEMMs of the other; the two partial results are
// merged at the end (O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / l).  A thread owns one query row: it reads the 128 scores
// once from TMEM, needs no cross-thread reduction, writes bf16 probabilities in the swizzled layout the tensor core
// expects, and rescales its accumulator only when the running maximum has grown by more than 2^8.
// Output: O (bf16) and the log-sum-exp per (head, token) in fp32, the layout the backward pass of the flash-attn
// library expects, which serves as backward for now.
//
// The reference obtains attention from the flash-attn package or PyTorch SDPA through Hugging Face
// (arctic_training/config/model.py:48,85-98).  All barrier waits are bounded.

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>

namespace atb {

CUtensorMap make_tmap_bf16_public(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
at::Tensor& gemm_error_flag(const at::Device& dev);

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int CHUNK_BYTES = 128 * 128;        // [128 rows][64 bf16]
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;   // 128 x 128 bf16
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = TILE_BYTES;                  // two stages
constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;     // two stages
constexpr int SMEM_P = SMEM_V + 2 * TILE_BYTES;     // one probability tile per softmax group
constexpr int SMEM_BAR = SMEM_P + 2 * TILE_BYTES;   // 224 KB of tiles
constexpr int SMEM_XCHG = SMEM_BAR + 24 * 8;        // float2 [2 groups][128 rows]: (maximum, sum) for the final merge
constexpr int SMEM_TOTAL = SMEM_XCHG + 2 * 128 * 8;
constexpr uint64_t kAttnWaitNs = 2000000000ull;
constexpr float kRescaleThreshold = 8.f;  // in log2 units
constexpr int kAttnThreads = 320;         // TMA warp, MMA warp, two softmax groups of four warps

#ifdef ATB_ATTN_PROFILE
__device__ long long g_attn_prof[16];
#define PROF_T() clock64()
#define PROF_ADD(i, t0) do { if (prof_on) atomicAdd((unsigned long long*)&g_attn_prof[i], (unsigned long long)(clock64() - (t0))); } while (0)
#else
#define PROF_T() 0ll
#define PROF_ADD(i, t0) do { (void)(t0); } while (0)
#endif

struct AttnParams {
    bf16* O;
    float* lse;           // [Hq, T]
    const int* cu_seqlens;  // [nseq + 1]
    int nseq, T, Hq, Hkv;
    int64_t o_row_stride;  // elements between consecutive tokens of O
    float scale_log2;      // softmax_scale * log2(e)
    int* error_flag;
};

__global__ void __launch_bounds__(kAttnThreads, 1)
fmha_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
    uint64_t* q_full = bars;          // 1
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* k_empty = bars + 3;     // [2]
    uint64_t* v_full = bars + 5;      // [2]
    uint64_t* v_empty = bars + 7;     // [2]
    uint64_t* s_full = bars + 9;      // [2] scores of a block are in the group's TMEM buffer
    uint64_t* s_empty = bars + 11;    // [2] the group has copied the scores into registers
    uint64_t* p_full = bars + 13;     // [2] the group's probability tile is written
    uint64_t* pv_done = bars + 15;    // [2] the group's last P V has retired
    uint64_t* merge_ready = bars + 17;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float2* xchg = reinterpret_cast<float2*>(smem + SMEM_XCHG);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y;
    const int hkv = h / (p.Hq / p.Hkv);

    // ---- which (sequence, query block) is this CTA?  Blocks with the most key blocks come first in launch order.
    int rem = (int)blockIdx.x;
    int seq = -1, qb = 0, tok0 = 0, seqlen = 0;
    for (int s = p.nseq - 1; s >= 0; --s) {
        const int a = p.cu_seqlens[s], b = p.cu_seqlens[s + 1];
        const int nb = (b - a + BQ - 1) / BQ;
        if (rem < nb) { seq = s; qb = nb - 1 - rem; tok0 = a; seqlen = b - a; break; }
        rem -= nb;
    }
    if (seq < 0) return;  // padding CTA of the upper-bound grid (uniform for the whole CTA)
    if ((ptx::smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(p.error_flag, 0, (0x20 << 8) | 1);
        return;
    }
    const int n_kv = qb + 1;  // causal: key blocks 0..qb
#ifdef ATB_ATTN_PROFILE
    const bool prof_on = blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x == 32 || threadIdx.x == 64);
#endif

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&k_full[i], 1);
            ptx::mbar_init(&k_empty[i], 1);
            ptx::mbar_init(&v_full[i], 1);
            ptx::mbar_init(&v_empty[i], 1);
            ptx::mbar_init(&s_full[i], 1);
            ptx::mbar_init(&s_empty[i], 4);
            ptx::mbar_init(&p_full[i], 4);
            ptx::mbar_init(&pv_done[i], 1);
        }
        ptx::mbar_init(merge_ready, 8);
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
    const uint32_t tmem_base = *tmem_slot;  // columns: S_0 [0,128) S_1 [128,256) O_0 [256,384) O_1 [384,512)

    if (warp == 0) {
        // Two independent producers: lane 0 streams Q and the K ring, lane 1 the V ring.  A K slot is free as soon as
        // the scores of its block are computed, a V slot only after the block's P V: with one thread feeding both rings
        // in order the next K would wait behind the V slot and its load latency would be exposed in every iteration.
        if (lane == 0) {
            ptx::tma_prefetch_desc(&tmap_q);
            ptx::tma_prefetch_desc(&tmap_k);
            ptx::mbar_expect_tx(q_full, TILE_BYTES);
            for (int c = 0; c < 2; ++c)
                ptx::tma_load_2d(smem + SMEM_Q + c * CHUNK_BYTES, &tmap_q, h * HD + c * 64, tok0 + qb * BQ, q_full);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1;
                if (!ptx::mbar_wait_bounded(&k_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag, kAttnWaitNs)) {
                    atomicCAS(p.error_flag, 0, (0x21 << 8) | 1);
                    break;
                }
                ptx::mbar_expect_tx(&k_full[st], TILE_BYTES);
                for (int c = 0; c < 2; ++c)
                    ptx::tma_load_2d(smem + SMEM_K + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_k, hkv * HD + c * 64, tok0 + j * BKV,
                                     &k_full[st]);
            }
        } else if (lane == 1) {
            ptx::tma_prefetch_desc(&tmap_v);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1;
                if (!ptx::mbar_wait_bounded(&v_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag, kAttnWaitNs)) {
                    atomicCAS(p.error_flag, 0, (0x21 << 8) | 2);
                    break;
                }
                ptx::mbar_expect_tx(&v_full[st], TILE_BYTES);
                for (int c = 0; c < 2; ++c)
                    ptx::tma_load_2d(smem + SMEM_V + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_v, hkv * HD + c * 64, tok0 + j * BKV,
                                     &v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ptx::make_idesc_bf16(BQ, BKV, false, false);
            constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(BQ, HD, false, true);
            const uint32_t qs = ptx::smem_u32(smem + SMEM_Q);
            bool ok = ptx::mbar_wait_bounded(q_full, 0, abort_flag, kAttnWaitNs);
            auto issue_qk = [&](int j) -> bool {  // S_{j&1} = Q K_j^T
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!ptx::mbar_wait_bounded(&k_full[st], ph, abort_flag, kAttnWaitNs)) return false;
                if (!ptx::mbar_wait_bounded(&s_empty[st], ph ^ 1u, abort_flag, kAttnWaitNs)) return false;
                ptx::tc_fence_after();
                const uint32_t ks = ptx::smem_u32(smem + SMEM_K + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_base + st * 128, ptx::make_smem_desc_sw128(qs + off, 16, 1024),
                                     ptx::make_smem_desc_sw128(ks + off, 16, 1024), idesc_qk, k != 0);
                }
                ptx::mma_commit(&s_full[st]);
                ptx::mma_commit(&k_empty[st]);
                return true;
            };
            auto issue_pv = [&](int j) -> bool {  // O_{j&1} += P_{j&1} V_j
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const long long tp0 = PROF_T();
                if (!ptx::mbar_wait_bounded(&p_full[st], ph, abort_flag, kAttnWaitNs)) return false;
                PROF_ADD(0, tp0);
                if (!ptx::mbar_wait_bounded(&v_full[st], ph, abort_flag, kAttnWaitNs)) return false;
                ptx::tc_fence_after();
                const uint32_t ps = ptx::smem_u32(smem + SMEM_P + st * TILE_BYTES);
                const uint32_t vs = ptx::smem_u32(smem + SMEM_V + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    const uint32_t poff = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_base + 256 + st * 128, ptx::make_smem_desc_sw128(ps + poff, 16, 1024),
                                     ptx::make_smem_desc_sw128(vs + k * 2048, CHUNK_BYTES, 1024), idesc_pv, (j >= 2 || k != 0) ? 1u : 0u);
                }
                ptx::mma_commit(&pv_done[st]);
                ptx::mma_commit(&v_empty[st]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            if (ok && n_kv > 1) ok = issue_qk(1);
            for (int j = 0; j < n_kv && ok; ++j) {
                const long long tq0 = PROF_T();
                if (j + 2 < n_kv) ok = issue_qk(j + 2);  // needs only that the group has copied S_j out of TMEM
                PROF_ADD(1, tq0);
                if (ok) ok = issue_pv(j);
            }
            if (!ok) atomicCAS(p.error_flag, 0, (0x22 << 8) | 1);
        }
    } else {
        // ------------------------------------------------------------------ softmax groups / merge / epilogue
        const int g = (warp - 2) >> 2;              // group: key blocks j with j % 2 == g
        const int quarter = warp & 3;               // TMEM lane quarter this warp may access
        const int r = quarter * 32 + lane;          // row of the query block owned by this thread
        const int qidx = qb * BQ + r;               // position inside the sequence
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_addr + g * 128;
        const uint32_t o_addr = tmem_base + lane_addr + 256 + g * 128;
        uint8_t* prow = smem + SMEM_P + g * TILE_BYTES + r * 128;  // row r of both 64-key chunks of the group's P tile
        const int n_mine = (n_kv - g + 1) / 2;      // blocks of this group
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_mine && ok; ++it) {
            const int j = 2 * it + g;
            const uint32_t ph = it & 1;
            const long long ts0 = PROF_T();
            if (!ptx::mbar_wait_bounded(&s_full[g], ph, abort_flag, kAttnWaitNs)) { ok = false; break; }
            PROF_ADD(2, ts0);
            PROF_ADD(8, PROF_T() - 1);
            ptx::tc_fence_after();
            const long long t10 = PROF_T();
            uint32_t s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32b_x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            ptx::tmem_ld_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&s_empty[g]);  // the next scores of this group may be computed
            const int kbase = j * BKV;
            const int klimit = min(seqlen, qidx + 1) - kbase;  // columns c < klimit are visible to this row
            // only the diagonal block and the block that holds the end of the sequence need masking (uniform per CTA)
            const bool need_mask = kbase + BKV > min(seqlen, qb * BQ + 1);
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i >= klimit) s[i] = 0xff800000u;  // -inf
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(s[i]));
                mx1 = fmaxf(mx1, __uint_as_float(s[32 + i]));
                mx2 = fmaxf(mx2, __uint_as_float(s[64 + i]));
                mx3 = fmaxf(mx3, __uint_as_float(s[96 + i]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            PROF_ADD(3, t10);
            // the group's previous P V must have retired before its P tile is overwritten or its accumulator is touched
            const long long tv0 = PROF_T();
            if (it > 0 && !ptx::mbar_wait_bounded(&pv_done[g], (it - 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
            PROF_ADD(5, tv0);
            ptx::tc_fence_after();
            const long long tr0 = PROF_T();
            const bool grow = mx > m_used + kRescaleThreshold || m_used == -INFINITY;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? fmaxf(mx, m_used) : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
                if (it > 0) {
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(o_addr + c * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_32x32b_x32(o_addr + c * 32, v);
                    }
                    ptx::tmem_st_wait();
                }
                l *= alpha;
                m_used = m_new;
            }
            PROF_ADD(6, tr0);
            const long long t20 = PROF_T();
            // probabilities -> bf16 -> swizzled shared memory; running sum (masked scores are -inf: exp2 gives 0)
            float l0 = 0.f, l1 = 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u) {  // sixteen 16-byte units of 8 probabilities
                float f8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float e = exp2f(fmaf(__uint_as_float(s[u * 8 + i]), p.scale_log2, -m_used));
                    f8[i] = e;
                    if (i & 1) l1 += e; else l0 += e;
                }
                *reinterpret_cast<bf16x8*>(prow + (u >> 3) * CHUNK_BYTES + (((u & 7) ^ (r & 7)) << 4)) = pack8(f8);
            }
            l += l0 + l1;
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();  // generic-proxy writes of P become visible to the tensor core
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&p_full[g]);
            PROF_ADD(7, t20);
        }
        // ---- merge the two groups' partial results; group g stores head-dim columns [64 g, 64 g + 64)
        if (ok && n_mine > 0 && !ptx::mbar_wait_bounded(&pv_done[g], (n_mine - 1) & 1, abort_flag, kAttnWaitNs)) ok = false;
        const int n_other = n_kv - n_mine;
        if (ok && n_other > 0 && !ptx::mbar_wait_bounded(&pv_done[g ^ 1], (n_other - 1) & 1, abort_flag, kAttnWaitNs)) ok = false;
        if (ok) {
            xchg[g * 128 + r] = make_float2(m_used, l);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(merge_ready);
            if (!ptx::mbar_wait_bounded(merge_ready, 0, abort_flag, kAttnWaitNs)) ok = false;
        }
        if (!ok) {
            if (lane == 0) atomicCAS(p.error_flag, 0, (0x23 << 8) | 1);
        } else {
            ptx::tc_fence_after();
            const float2 other = xchg[(g ^ 1) * 128 + r];
            const float m = fmaxf(m_used, other.x);
            const float a_self = n_mine > 0 ? exp2f(m_used - m) : 0.f;
            const float a_other = n_other > 0 ? exp2f(other.x - m) : 0.f;
            const float l_tot = l * a_self + other.y * a_other;
            const float inv_l = 1.f / l_tot;
            const float w_self = a_self * inv_l, w_other = a_other * inv_l;
            const bool valid = qidx < seqlen;
            const uint32_t o_self = tmem_base + lane_addr + 256 + g * 128 + g * 64;
            const uint32_t o_oth = tmem_base + lane_addr + 256 + (g ^ 1) * 128 + g * 64;
            bf16* orow = p.O + (int64_t)(tok0 + qidx) * p.o_row_stride + (int64_t)h * HD + g * 64;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t a[32], b[32];
                if (n_mine > 0) ptx::tmem_ld_32x32b_x32(o_self + c * 32, a);
                if (n_other > 0) ptx::tmem_ld_32x32b_x32(o_oth + c * 32, b);
                ptx::tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float f8[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float acc = 0.f;
                            if (n_mine > 0) acc = __uint_as_float(a[u * 8 + i]) * w_self;
                            if (n_other > 0) acc = fmaf(__uint_as_float(b[u * 8 + i]), w_other, acc);
                            f8[i] = acc;
                        }
                        *reinterpret_cast<bf16x8*>(orow + c * 32 + u * 8) = pack8(f8);
                    }
                }
            }
            if (valid && g == 0) p.lse[(int64_t)h * p.T + tok0 + qidx] = (m + log2f(l_tot)) * 0.6931471805599453f;
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

#ifdef ATB_ATTN_PROFILE
at::Tensor fmha_read_profile() {
    long long h[16];
    C10_CUDA_CHECK(cudaMemcpyFromSymbol(h, g_attn_prof, sizeof(h)));
    long long z[16] = {0};
    C10_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_prof, z, sizeof(z)));
    auto out = at::empty({16}, at::kLong);
    for (int i = 0; i < 16; ++i) out.data_ptr<int64_t>()[i] = h[i];
    return out;
}
#endif

// q [T, Hq, 128], k / v [T, Hkv, 128] bf16 (token stride may exceed heads * 128: views of a fused projection are fine),
// cu_seqlens int32 [nseq + 1] on the device.  Returns (out [T, Hq, 128] bf16, lse [Hq, T] fp32).
std::tuple<at::Tensor, at::Tensor> fmha_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                            const at::Tensor& cu_seqlens, int64_t max_blocks, double softmax_scale) {
    ATB_CHECK_CUDA(q); ATB_CHECK_DTYPE(q, at::kBFloat16); ATB_CHECK_DTYPE(k, at::kBFloat16); ATB_CHECK_DTYPE(v, at::kBFloat16);
    ATB_CHECK_DTYPE(cu_seqlens, at::kInt); ATB_CHECK_CONTIG(cu_seqlens);
    TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "fmha: q, k, v must be [tokens, heads, head_dim]");
    const int64_t T = q.size(0);
    const int Hq = (int)q.size(1), Hkv = (int)k.size(1);
    TORCH_CHECK(q.size(2) == HD && k.size(2) == HD && v.size(2) == HD, "fmha: head_dim must be 128");
    TORCH_CHECK(k.size(0) == T && v.size(0) == T && v.size(1) == Hkv && Hq % Hkv == 0, "fmha: inconsistent shapes");
    for (const at::Tensor* t : {&q, &k, &v}) {
        TORCH_CHECK(t->stride(2) == 1 && t->stride(1) == HD && t->stride(0) % 8 == 0, "fmha: heads must be dense, token stride % 8 == 0");
        TORCH_CHECK((reinterpret_cast<uintptr_t>(t->data_ptr()) & 15) == 0, "fmha: operands must be 16-byte aligned");
    }
    const int nseq = (int)cu_seqlens.numel() - 1;
    TORCH_CHECK(nseq >= 1 && max_blocks >= 1, "fmha: need at least one sequence");
    c10::cuda::CUDAGuard guard(q.device());
    auto out = at::empty({T, Hq, HD}, q.options());
    auto lse = at::empty({Hq, T}, q.options().dtype(at::kFloat));
    if (T == 0) return {out, lse};
    const CUtensorMap tq = make_tmap_bf16_public(q.data_ptr(), T, (int64_t)Hq * HD, q.stride(0), BQ);
    const CUtensorMap tk = make_tmap_bf16_public(k.data_ptr(), T, (int64_t)Hkv * HD, k.stride(0), BKV);
    const CUtensorMap tv = make_tmap_bf16_public(v.data_ptr(), T, (int64_t)Hkv * HD, v.stride(0), BKV);
    AttnParams p;
    p.O = (bf16*)out.data_ptr();
    p.lse = lse.data_ptr<float>();
    p.cu_seqlens = cu_seqlens.data_ptr<int>();
    p.nseq = nseq; p.T = (int)T; p.Hq = Hq; p.Hkv = Hkv;
    p.o_row_stride = out.stride(0);
    p.scale_log2 = (float)(softmax_scale * 1.4426950408889634);
    p.error_flag = gemm_error_flag(q.device()).data_ptr<int>();
    static bool attr_set = false;
    constexpr int smem_bytes = SMEM_TOTAL;
    if (!attr_set) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(fmha_fwd_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        attr_set = true;
    }
    dim3 grid((unsigned)max_blocks, (unsigned)Hq);
    fmha_fwd_tcgen05_kernel<<<grid, kAttnThreads, smem_bytes, current_stream()>>>(tq, tk, tv, p);
    ATB_LAUNCH_CHECK();
    return {out, lse};
}

}  // namespace atb
