// Causal flash-attention forward for sm_100a: packed (variable-length) sequences, grouped-query heads, head_dim 128.
//
//   O[t, h, :] = softmax_j<=t ( Q[t, h, :] . K[j, g(h), :] * scale ) V[j, g(h), :]     within each packed sequence
//
// One CTA per (sequence, block of 128 queries, query head).  Warp 0 streams K/V blocks of 128 keys with TMA into a
// two-stage shared-memory ring, warp 1 issues the two GEMMs of every block on the tensor cores (S = Q K^T into one of
// two TMEM score buffers, O += P V into a TMEM accumulator), warps 2..5 own one query row per thread: they read the
// scores from TMEM, keep the running maximum and sum in registers (no cross-thread reduction is needed because a
// thread sees its whole row), write the bf16 probabilities into shared memory in the swizzled layout the tensor core
// expects, and rescale the accumulator only when the running maximum has grown by more than 2^8 (the final division
// by the row sum makes the result independent of which maximum was used).  The score GEMM of block j+1 overlaps the
// softmax of block j.  Output: O (bf16) and the log-sum-exp per (head, token) in fp32, the layout the backward pass
// of the flash-attn library expects, which serves as backward for now.
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
constexpr int KV_STAGES = 2;
constexpr int SMEM_Q = 0;
constexpr int SMEM_KV = TILE_BYTES;                              // stage s: K at +s*2*TILE, V right after K
constexpr int SMEM_P = SMEM_KV + KV_STAGES * 2 * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_P + TILE_BYTES;
constexpr int SMEM_XCHG = SMEM_BAR + 16 * 8 + 16;       // float [2 parities][2 halves][128 rows]
constexpr int SMEM_TOTAL = SMEM_XCHG + 2 * 2 * 128 * 4;
constexpr uint64_t kAttnWaitNs = 2000000000ull;
constexpr float kRescaleThreshold = 8.f;  // in log2 units
constexpr int kAttnThreads = 320;        // TMA warp, MMA warp, eight softmax warps (two per TMEM lane quarter)

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

// Maximum over 64 score columns of one row in TMEM (raw, unscaled scores); columns >= klimit are ignored when MASK.
// `col0` is the first of the 64 columns inside the 128-key block.
template <bool MASK>
__device__ __forceinline__ float score_row_max(uint32_t s_addr, int col0, int klimit) {
    uint32_t a[32], b[32];
    ptx::tmem_ld_32x32b_x32(s_addr, a);
    ptx::tmem_ld_32x32b_x32(s_addr + 32, b);
    ptx::tmem_ld_wait();
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (!MASK || col0 + i < klimit) m0 = fmaxf(m0, __uint_as_float(a[i]));
        if (!MASK || col0 + 32 + i < klimit) m1 = fmaxf(m1, __uint_as_float(b[i]));
    }
    return fmaxf(m0, m1);
}

// p = exp2(s * scale - m) for 64 columns of one row: bf16 into one 64-key chunk of the swizzled P tile (row `crow`,
// swizzle phase r & 7); returns the sum of the 64 probabilities.
template <bool MASK>
__device__ __forceinline__ float score_row_exp(uint32_t s_addr, int col0, int klimit, float scale, float m, uint8_t* crow,
                                               int r) {
    uint32_t a[32], b[32];
    ptx::tmem_ld_32x32b_x32(s_addr, a);
    ptx::tmem_ld_32x32b_x32(s_addr + 32, b);
    ptx::tmem_ld_wait();
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {  // eight 16-byte units of 8 probabilities
        float f8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int col = u * 8 + i;  // 0..63 inside the chunk
            const float sv = __uint_as_float(col < 32 ? a[col & 31] : b[col & 31]);
            float e = exp2f(fmaf(sv, scale, -m));
            if (MASK && col0 + col >= klimit) e = 0.f;
            f8[i] = e;
            if (i & 1) l1 += e; else l0 += e;
        }
        *reinterpret_cast<bf16x8*>(crow + ((u ^ (r & 7)) << 4)) = pack8(f8);
    }
    return l0 + l1;
}

__global__ void __launch_bounds__(kAttnThreads, 1)
fmha_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
    uint64_t* q_full = bars;            // 1
    uint64_t* kv_full = bars + 1;       // [2]
    uint64_t* kv_empty = bars + 3;      // [2]
    uint64_t* s_full = bars + 5;        // [2]
    uint64_t* s_empty = bars + 7;       // [2]
    uint64_t* p_full = bars + 9;        // 1
    uint64_t* pv_done = bars + 10;      // 1
    uint64_t* max_ready = bars + 11;    // [2]: both column halves have published their row maxima
    float* xchg = reinterpret_cast<float*>(smem + SMEM_XCHG);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y;
    const int hkv = h / (p.Hq / p.Hkv);

    // ---- which (sequence, query block) is this CTA?  longest (most key blocks) first within the launch order
    int rem = (int)(gridDim.x - 1 - blockIdx.x);
    int seq = -1, qb = 0, tok0 = 0, seqlen = 0;
    for (int s = p.nseq - 1; s >= 0; --s) {
        const int a = p.cu_seqlens[s], b = p.cu_seqlens[s + 1];
        const int nb = (b - a + BQ - 1) / BQ;
        if (rem < nb) { seq = s; qb = nb - 1 - rem; tok0 = a; seqlen = b - a; break; }
        rem -= nb;
    }
    if (seq < 0) return;  // padding CTA of the upper-bound grid (uniform for the whole CTA)
    const int n_kv = qb + 1;  // causal: key blocks 0..qb
#ifdef ATB_ATTN_PROFILE
    const bool prof_on = blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x == 32 || threadIdx.x == 64);
#endif

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&kv_full[i], 1);
            ptx::mbar_init(&kv_empty[i], 1);
            ptx::mbar_init(&s_full[i], 1);
            ptx::mbar_init(&s_empty[i], 8);
            ptx::mbar_init(&max_ready[i], 8);
        }
        ptx::mbar_init(p_full, 8);
        ptx::mbar_init(pv_done, 1);
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
    const uint32_t tmem_o = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            ptx::tma_prefetch_desc(&tmap_q);
            ptx::tma_prefetch_desc(&tmap_k);
            ptx::tma_prefetch_desc(&tmap_v);
            ptx::mbar_expect_tx(q_full, TILE_BYTES);
            for (int c = 0; c < 2; ++c)
                ptx::tma_load_2d(smem + SMEM_Q + c * CHUNK_BYTES, &tmap_q, h * HD + c * 64, tok0 + qb * BQ, q_full);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1;
                if (!ptx::mbar_wait_bounded(&kv_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag, kAttnWaitNs)) {
                    atomicCAS(p.error_flag, 0, (0x21 << 8) | 1);
                    break;
                }
                uint8_t* ks = smem + SMEM_KV + st * 2 * TILE_BYTES;
                uint8_t* vs = ks + TILE_BYTES;
                ptx::mbar_expect_tx(&kv_full[st], 2 * TILE_BYTES);
                for (int c = 0; c < 2; ++c) {
                    ptx::tma_load_2d(ks + c * CHUNK_BYTES, &tmap_k, hkv * HD + c * 64, tok0 + j * BKV, &kv_full[st]);
                    ptx::tma_load_2d(vs + c * CHUNK_BYTES, &tmap_v, hkv * HD + c * 64, tok0 + j * BKV, &kv_full[st]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = ptx::make_idesc_bf16(BQ, BKV, false, false);
            constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(BQ, HD, false, true);
            const uint32_t qs = ptx::smem_u32(smem + SMEM_Q), ps = ptx::smem_u32(smem + SMEM_P);
            bool ok = ptx::mbar_wait_bounded(q_full, 0, abort_flag, kAttnWaitNs);
            auto issue_qk = [&](int j) -> bool {
                const int st = j & 1;
                if (!ptx::mbar_wait_bounded(&kv_full[st], (j >> 1) & 1, abort_flag, kAttnWaitNs)) return false;
                if (!ptx::mbar_wait_bounded(&s_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag, kAttnWaitNs)) return false;
                ptx::tc_fence_after();
                const uint32_t ks = ptx::smem_u32(smem + SMEM_KV + st * 2 * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_base + st * 128, ptx::make_smem_desc_sw128(qs + off, 16, 1024),
                                     ptx::make_smem_desc_sw128(ks + off, 16, 1024), idesc_qk, k != 0);
                }
                ptx::mma_commit(&s_full[st]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                const long long tq0 = PROF_T();
                if (j + 1 < n_kv) ok = issue_qk(j + 1);
                PROF_ADD(1, tq0);
                if (!ok) break;
                const long long tp0 = PROF_T();
                if (!ptx::mbar_wait_bounded(p_full, j & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
                PROF_ADD(0, tp0);
                ptx::tc_fence_after();
                const uint32_t vs = ptx::smem_u32(smem + SMEM_KV + (j & 1) * 2 * TILE_BYTES + TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    const uint32_t poff = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    ptx::mma_bf16_ss(tmem_o, ptx::make_smem_desc_sw128(ps + poff, 16, 1024),
                                     ptx::make_smem_desc_sw128(vs + k * 2048, CHUNK_BYTES, 1024), idesc_pv, (j | k) != 0);
                }
                ptx::mma_commit(pv_done);
                ptx::mma_commit(&kv_empty[j & 1]);
            }
            if (!ok) atomicCAS(p.error_flag, 0, (0x22 << 8) | 1);
        }
    } else {
        // ------------------------------------------------------------------ softmax / correction / epilogue
        // Two warps share each TMEM lane quarter: for the same 32 query rows one takes key columns 0..63 of every block
        // (and head-dim columns 0..63 of O), the other the upper halves.  They agree on the row maximum through shared
        // memory once per block; the row sums are combined at the end.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;          // row of the query block owned by this thread
        const int qidx = qb * BQ + r;               // position inside the sequence
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int col0 = half * 64;
        uint8_t* crow = smem + SMEM_P + half * CHUNK_BYTES + r * 128;  // row r of this half's 64-key chunk of P
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int st = j & 1;
            const long long ts0 = PROF_T();
            if (!ptx::mbar_wait_bounded(&s_full[st], (j >> 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
            PROF_ADD(2, ts0);
            PROF_ADD(8, PROF_T() - 1);
            ptx::tc_fence_after();
            const uint32_t s_addr = tmem_base + lane_addr + st * 128 + col0;
            const int kbase = j * BKV;
            const int klimit = min(seqlen, qidx + 1) - kbase;  // columns c < klimit are visible to this row
            // only the diagonal block and the block that holds the end of the sequence need masking (uniform per CTA)
            const bool need_mask = kbase + BKV > min(seqlen, qb * BQ + 1);
            // pass 1: row maximum of the scores, agreed between the two halves
            const long long t10 = PROF_T();
            float mx = need_mask ? score_row_max<true>(s_addr, col0, klimit) : score_row_max<false>(s_addr, col0, klimit);
            PROF_ADD(3, t10);
            xchg[(st * 2 + half) * 128 + r] = mx;
            __syncwarp();
            const long long tx0 = PROF_T();
            if (lane == 0) ptx::mbar_arrive(&max_ready[st]);
            if (!ptx::mbar_wait_bounded(&max_ready[st], (j >> 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
            PROF_ADD(4, tx0);
            mx = fmaxf(mx, xchg[(st * 2 + (half ^ 1)) * 128 + r]) * p.scale_log2;
            // previous P V must have retired before P is overwritten or O is touched
            const long long tv0 = PROF_T();
            if (j > 0 && !ptx::mbar_wait_bounded(pv_done, (j - 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
            PROF_ADD(5, tv0);
            ptx::tc_fence_after();
            const long long tr0 = PROF_T();
            const bool grow = mx > m_used + kRescaleThreshold || m_used == -INFINITY;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? fmaxf(mx, m_used) : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
                if (j > 0) {
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(tmem_o + lane_addr + col0 + c * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_32x32b_x32(tmem_o + lane_addr + col0 + c * 32, v);
                    }
                    ptx::tmem_st_wait();
                }
                l *= alpha;
                m_used = m_new;
            }
            PROF_ADD(6, tr0);
            const long long t20 = PROF_T();
            // pass 2: probabilities -> bf16 -> swizzled shared memory; running sum
            l += need_mask ? score_row_exp<true>(s_addr, col0, klimit, p.scale_log2, m_used, crow, r)
                           : score_row_exp<false>(s_addr, col0, klimit, p.scale_log2, m_used, crow, r);
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();  // generic-proxy writes of P become visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&s_empty[st]);
                ptx::mbar_arrive(p_full);
            }
            PROF_ADD(7, t20);
        }
        if (ok && !ptx::mbar_wait_bounded(pv_done, (n_kv - 1) & 1, abort_flag, kAttnWaitNs)) ok = false;
        if (ok) {
            // combine the row sums of the two halves (both used the same maxima); parity slot of a block not in use
            const int st = n_kv & 1;
            xchg[(st * 2 + half) * 128 + r] = l;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&max_ready[st]);
            if (!ptx::mbar_wait_bounded(&max_ready[st], (n_kv >> 1) & 1, abort_flag, kAttnWaitNs)) ok = false;
            else l += xchg[(st * 2 + (half ^ 1)) * 128 + r];
        }
        if (!ok) {
            if (lane == 0) atomicCAS(p.error_flag, 0, (0x23 << 8) | 1);
        } else {
            ptx::tc_fence_after();
            const float inv_l = 1.f / l;
            const bool valid = qidx < seqlen;
            bf16* orow = p.O + (int64_t)(tok0 + qidx) * p.o_row_stride + (int64_t)h * HD + col0;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(tmem_o + lane_addr + col0 + c * 32, v);
                ptx::tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float f8[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f8[i] = __uint_as_float(v[u * 8 + i]) * inv_l;
                        *reinterpret_cast<bf16x8*>(orow + c * 32 + u * 8) = pack8(f8);
                    }
                }
            }
            if (valid && half == 0) p.lse[(int64_t)h * p.T + tok0 + qidx] = (m_used + log2f(l)) * 0.6931471805599453f;
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
    constexpr int smem_bytes = SMEM_TOTAL + 1024;
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
