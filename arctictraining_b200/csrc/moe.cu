// SPDX-License-Identifier: Apache-2.0
// Mixture-of-experts routing and token permutation kernels.
//
//   moe_topk_gating_fwd / _bwd : softmax over all experts (fp32), top-k with ties resolved to the lower
//                                expert index, optional renormalisation of the k scores; backward through
//                                both, plus an additive term on d(probs) (the load-balancing gradient).
//   moe_assign_slots           : deterministic expert-major slot for every (token, k) pair: pairs of one
//                                expert keep their (token, k) order; expert segments start at multiples of
//                                `align` rows (128 for the grouped GEMM, 1 for a send buffer).  No atomics.
//   moe_scatter_fwd / _bwd     : rows of x copied to their slots / summed back over k.
//   moe_gather_fwd / _bwd      : out[t] = sum_k score[t,k] * y[slot[t,k]] and its gradients.
//
// They take the place of the reference's "ragged ops" extension (arctic_training/kernels/moe_ops/
// top_k_gating/top_k_gating_cuda.cu:74-314, moe_scatter/moe_scatter_cuda.cu:22-355,
// moe_gather/moe_gather_cuda.cu:24-321), which assigns slots with atomicAdd (non-deterministic order) and
// pads every expert to a globally all-reduced capacity.

#include "common.cuh"

namespace atb {

constexpr int kMaxExpertsPerLane = 32;  // E <= 1024

// ------------------------------------------------------------------------------------------- gating fwd
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(128) moe_topk_gating_fwd_kernel(const T* __restrict__ logits, float* __restrict__ probs,
                                                                  float* __restrict__ scores, int* __restrict__ experts,
                                                                  int64_t Tn, int E, int K, int normalize) {
    const int lane = threadIdx.x & 31;
    const int64_t t = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= Tn) return;
    const int per_lane = (E + 31) >> 5;
    float v[kMaxExpertsPerLane];
    float mx = -INFINITY;
#pragma unroll 4
    for (int i = 0; i < per_lane; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? to_f32(logits[t * E + e]) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = 0; i < per_lane; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? __expf(v[i] - mx) : 0.f;
        sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int i = 0; i < per_lane; ++i) {
        const int e = lane + 32 * i;
        v[i] *= inv;
        if (e < E) probs[t * E + e] = v[i];
    }
    // iterative arg-max; a taken entry is marked with -1 (probabilities are >= 0)
    float chosen_sum = 0.f;
    float my_score = 0.f;  // lane k keeps the k-th score (K <= 32)
    int my_expert = 0;
    for (int k = 0; k < K; ++k) {
        float best = -1.f;
        int best_e = 0x7fffffff;
        for (int i = 0; i < per_lane; ++i) {
            const int e = lane + 32 * i;
            if (e < E && v[i] > best) { best = v[i]; best_e = e; }  // strict '>' keeps the lowest index of this lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;
        if (lane == k) { my_score = best; my_expert = best_e; }
        chosen_sum += best;
    }
    if (lane < K) {
        scores[t * K + lane] = normalize ? my_score / chosen_sum : my_score;
        experts[t * K + lane] = my_expert;
    }
}

// ------------------------------------------------------------------------------------------- gating bwd
__global__ void __launch_bounds__(128) moe_topk_gating_bwd_kernel(const float* __restrict__ dscores,
                                                                  const float* __restrict__ probs,
                                                                  const int* __restrict__ experts,
                                                                  const float* __restrict__ dprobs_extra,  // [E] or null
                                                                  float* __restrict__ dlogits, int64_t Tn, int E, int K,
                                                                  int normalize) {
    const int lane = threadIdx.x & 31;
    const int64_t t = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= Tn) return;
    const int per_lane = (E + 31) >> 5;
    // gradient wrt the chosen probabilities
    float ds = 0.f, pk = 0.f;
    int ek = -1;
    if (lane < K) {
        ds = dscores[t * K + lane];
        ek = experts[t * K + lane];
        pk = probs[t * E + ek];
    }
    float gk = ds;
    if (normalize) {
        const float S = warp_sum(pk);
        const float dot = warp_sum(ds * pk) / S;  // sum_k ds_k * s_k
        gk = (ds - dot) / S;
    }
    float g[kMaxExpertsPerLane];
    float p[kMaxExpertsPerLane];
    for (int i = 0; i < per_lane; ++i) {
        const int e = lane + 32 * i;
        p[i] = e < E ? probs[t * E + e] : 0.f;
        g[i] = (e < E && dprobs_extra) ? dprobs_extra[e] : 0.f;
    }
    for (int k = 0; k < K; ++k) {
        const int e = __shfl_sync(0xffffffffu, ek, k);
        const float gv = __shfl_sync(0xffffffffu, gk, k);
        if ((e & 31) == lane) g[e >> 5] += gv;
    }
    float dot = 0.f;
    for (int i = 0; i < per_lane; ++i) dot += p[i] * g[i];
    dot = warp_sum(dot);
    for (int i = 0; i < per_lane; ++i) {
        const int e = lane + 32 * i;
        if (e < E) dlogits[t * E + e] = p[i] * (g[i] - dot);
    }
}

// ------------------------------------------------------------------------------------------- slot assignment
constexpr int kPairsPerBlock = 2048;

// pass 1: per-block histogram of expert ids over a contiguous range of (token, k) pairs
__global__ void __launch_bounds__(256) moe_hist_kernel(const int* __restrict__ experts, int64_t n_pairs, int E,
                                                       int* __restrict__ block_hist) {
    extern __shared__ int sh[];
    for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * kPairsPerBlock;
    for (int i = threadIdx.x; i < kPairsPerBlock; i += blockDim.x) {
        const int64_t p = base + i;
        if (p < n_pairs) atomicAdd(&sh[experts[p]], 1);  // integer counts: order does not matter
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[(int64_t)blockIdx.x * E + e] = sh[e];
}

// pass 2 (one block): per-expert totals, aligned segment offsets, and the start of each block inside each expert
__global__ void __launch_bounds__(1024) moe_scan_kernel(int* __restrict__ block_hist, int nblk, int E, int align,
                                                        int* __restrict__ counts, int* __restrict__ offsets /*[E+1]*/) {
    __shared__ int seg[1025];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int b = 0; b < nblk; ++b) {
            const int c = block_hist[(int64_t)b * E + e];
            block_hist[(int64_t)b * E + e] = run;  // exclusive prefix over blocks
            run += c;
        }
        counts[e] = run;
        seg[e] = (run + align - 1) / align * align;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = acc;
            acc += seg[e];
        }
        offsets[E] = acc;
    }
}

// pass 3: thread e walks the block's pairs in order and hands out consecutive slots to the pairs of expert e
__global__ void __launch_bounds__(256) moe_slot_kernel(const int* __restrict__ experts, int64_t n_pairs, int E,
                                                       const int* __restrict__ block_prefix,
                                                       const int* __restrict__ offsets, int* __restrict__ slots) {
    __shared__ int ids[kPairsPerBlock];
    const int64_t base = (int64_t)blockIdx.x * kPairsPerBlock;
    const int n = (int)min((int64_t)kPairsPerBlock, n_pairs - base);
    for (int i = threadIdx.x; i < n; i += blockDim.x) ids[i] = experts[base + i];
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int next = offsets[e] + block_prefix[(int64_t)blockIdx.x * E + e];
        for (int i = 0; i < n; ++i) {
            if (ids[i] == e) slots[base + i] = next++;
        }
    }
}

// ------------------------------------------------------------------------------------------- scatter / gather
__global__ void __launch_bounds__(256) moe_scatter_fwd_kernel(const bf16* __restrict__ x, const int* __restrict__ slots,
                                                              bf16* __restrict__ out, int H, int K) {
    const int64_t t = blockIdx.x;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + t * H);
    const int nvec = H >> 3;
    for (int k = 0; k < K; ++k) {
        bf16x8* dst = reinterpret_cast<bf16x8*>(out + (int64_t)slots[t * K + k] * H);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
    }
}

__global__ void __launch_bounds__(256) moe_scatter_bwd_kernel(const bf16* __restrict__ dout, const int* __restrict__ slots,
                                                              bf16* __restrict__ dx, int H, int K) {
    const int64_t t = blockIdx.x;
    const int nvec = H >> 3;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < K; ++k) {
            float f[8];
            unpack8(reinterpret_cast<const bf16x8*>(dout + (int64_t)slots[t * K + k] * H)[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
        reinterpret_cast<bf16x8*>(dx + t * H)[i] = pack8(acc);
    }
}

__global__ void __launch_bounds__(256) moe_gather_fwd_kernel(const bf16* __restrict__ y, const int* __restrict__ slots,
                                                             const float* __restrict__ scores, bf16* __restrict__ out,
                                                             int H, int K) {
    const int64_t t = blockIdx.x;
    const int nvec = H >> 3;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < K; ++k) {
            const float s = scores[t * K + k];
            float f[8];
            unpack8(reinterpret_cast<const bf16x8*>(y + (int64_t)slots[t * K + k] * H)[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += s * f[j];
        }
        reinterpret_cast<bf16x8*>(out + t * H)[i] = pack8(acc);
    }
}

// dy[slot] = dout[t] * score ; dscores[t,k] = <dout[t], y[slot]>
__global__ void __launch_bounds__(256) moe_gather_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ y,
                                                             const int* __restrict__ slots,
                                                             const float* __restrict__ scores, bf16* __restrict__ dy,
                                                             float* __restrict__ dscores, int H, int K) {
    __shared__ float scratch[32];
    const int64_t t = blockIdx.x;
    const int nvec = H >> 3;
    for (int k = 0; k < K; ++k) {
        const float s = scores[t * K + k];
        const int64_t row = slots[t * K + k];
        float dot = 0.f;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            float g[8], yy[8], o[8];
            unpack8(reinterpret_cast<const bf16x8*>(dout + t * H)[i], g);
            unpack8(reinterpret_cast<const bf16x8*>(y + row * H)[i], yy);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dot += g[j] * yy[j];
                o[j] = g[j] * s;
            }
            reinterpret_cast<bf16x8*>(dy + row * H)[i] = pack8(o);
        }
        dot = block_sum(dot, scratch);
        if (threadIdx.x == 0) dscores[t * K + k] = dot;
    }
}

// ------------------------------------------------------------------------------------------- host wrappers
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_topk_gating_fwd(const at::Tensor& logits, int64_t K, bool normalize) {
    ATB_CHECK_CUDA(logits); ATB_CHECK_CONTIG(logits);
    TORCH_CHECK(logits.dim() == 2, "gating: logits must be [tokens, experts]");
    const int64_t T = logits.size(0);
    const int E = (int)logits.size(1);
    TORCH_CHECK(E <= 32 * kMaxExpertsPerLane && K >= 1 && K <= 32 && K <= E, "gating: need E <= 1024 and 1 <= K <= min(32, E)");
    c10::cuda::CUDAGuard guard(logits.device());
    auto f32 = logits.options().dtype(at::kFloat);
    auto probs = at::empty({T, E}, f32);
    auto scores = at::empty({T, K}, f32);
    auto experts = at::empty({T, K}, logits.options().dtype(at::kInt));
    if (T > 0) {
        const unsigned grid = (unsigned)ceil_div(T, 4);
        if (logits.scalar_type() == at::kFloat) {
            moe_topk_gating_fwd_kernel<float><<<grid, 128, 0, current_stream()>>>(
                logits.data_ptr<float>(), probs.data_ptr<float>(), scores.data_ptr<float>(), experts.data_ptr<int>(), T, E,
                (int)K, normalize ? 1 : 0);
        } else {
            ATB_CHECK_DTYPE(logits, at::kBFloat16);
            moe_topk_gating_fwd_kernel<bf16><<<grid, 128, 0, current_stream()>>>(
                (const bf16*)logits.data_ptr(), probs.data_ptr<float>(), scores.data_ptr<float>(), experts.data_ptr<int>(),
                T, E, (int)K, normalize ? 1 : 0);
        }
        ATB_LAUNCH_CHECK();
    }
    return {probs, scores, experts};
}

at::Tensor moe_topk_gating_bwd(const at::Tensor& dscores, const at::Tensor& probs, const at::Tensor& experts,
                               const c10::optional<at::Tensor>& dprobs_extra, bool normalize) {
    ATB_CHECK_CUDA(probs); ATB_CHECK_CONTIG(probs); ATB_CHECK_CONTIG(dscores); ATB_CHECK_CONTIG(experts);
    ATB_CHECK_DTYPE(probs, at::kFloat); ATB_CHECK_DTYPE(dscores, at::kFloat); ATB_CHECK_DTYPE(experts, at::kInt);
    const int64_t T = probs.size(0);
    const int E = (int)probs.size(1), K = (int)experts.size(1);
    const float* extra = nullptr;
    if (dprobs_extra.has_value()) {
        ATB_CHECK_DTYPE(*dprobs_extra, at::kFloat); ATB_CHECK_CONTIG(*dprobs_extra);
        TORCH_CHECK(dprobs_extra->numel() == E, "gating_bwd: extra gradient must have one entry per expert");
        extra = dprobs_extra->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(probs.device());
    auto dlogits = at::empty_like(probs);
    if (T > 0) {
        moe_topk_gating_bwd_kernel<<<(unsigned)ceil_div(T, 4), 128, 0, current_stream()>>>(
            dscores.data_ptr<float>(), probs.data_ptr<float>(), experts.data_ptr<int>(), extra, dlogits.data_ptr<float>(), T,
            E, K, normalize ? 1 : 0);
        ATB_LAUNCH_CHECK();
    }
    return dlogits;
}

// experts [T, K] int32 -> (slots [T, K] int32, counts [E] int32, offsets [E+1] int32)
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_assign_slots(const at::Tensor& experts, int64_t E, int64_t align) {
    ATB_CHECK_CUDA(experts); ATB_CHECK_CONTIG(experts); ATB_CHECK_DTYPE(experts, at::kInt);
    TORCH_CHECK(E >= 1 && E <= 1024 && align >= 1, "assign_slots: need 1 <= E <= 1024 and align >= 1");
    const int64_t n_pairs = experts.numel();
    c10::cuda::CUDAGuard guard(experts.device());
    auto iopt = experts.options();
    auto slots = at::empty_like(experts);
    auto counts = at::empty({E}, iopt);
    auto offsets = at::empty({E + 1}, iopt);
    const int nblk = (int)std::max<int64_t>(1, ceil_div(n_pairs, kPairsPerBlock));
    auto hist = at::empty({nblk, E}, iopt);
    moe_hist_kernel<<<nblk, 256, E * sizeof(int), current_stream()>>>(experts.data_ptr<int>(), n_pairs, (int)E,
                                                                       hist.data_ptr<int>());
    ATB_LAUNCH_CHECK();
    moe_scan_kernel<<<1, 1024, 0, current_stream()>>>(hist.data_ptr<int>(), nblk, (int)E, (int)align,
                                                      counts.data_ptr<int>(), offsets.data_ptr<int>());
    ATB_LAUNCH_CHECK();
    if (n_pairs > 0) {
        moe_slot_kernel<<<nblk, 256, 0, current_stream()>>>(experts.data_ptr<int>(), n_pairs, (int)E, hist.data_ptr<int>(),
                                                            offsets.data_ptr<int>(), slots.data_ptr<int>());
        ATB_LAUNCH_CHECK();
    }
    return {slots, counts, offsets};
}

static void check_rows(const at::Tensor& x, const char* what) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.dim() == 2, what,
                ": expected a contiguous 2-D bf16 CUDA tensor");
    TORCH_CHECK(x.size(1) % 8 == 0, what, ": row length must be a multiple of 8");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, what, ": must be 16-byte aligned");
}

at::Tensor moe_scatter_fwd(const at::Tensor& x, const at::Tensor& slots, int64_t out_rows) {
    check_rows(x, "scatter x");
    ATB_CHECK_DTYPE(slots, at::kInt); ATB_CHECK_CONTIG(slots);
    const int64_t T = x.size(0);
    const int H = (int)x.size(1), K = (int)slots.size(1);
    TORCH_CHECK(slots.size(0) == T, "scatter: one row of slots per token");
    c10::cuda::CUDAGuard guard(x.device());
    auto out = at::zeros({out_rows, H}, x.options());  // padding rows must be zero
    if (T > 0) {
        moe_scatter_fwd_kernel<<<(unsigned)T, 256, 0, current_stream()>>>((const bf16*)x.data_ptr(), slots.data_ptr<int>(),
                                                                          (bf16*)out.data_ptr(), H, K);
        ATB_LAUNCH_CHECK();
    }
    return out;
}

at::Tensor moe_scatter_bwd(const at::Tensor& dout, const at::Tensor& slots) {
    check_rows(dout, "scatter dout");
    ATB_CHECK_DTYPE(slots, at::kInt); ATB_CHECK_CONTIG(slots);
    const int64_t T = slots.size(0);
    const int H = (int)dout.size(1), K = (int)slots.size(1);
    c10::cuda::CUDAGuard guard(dout.device());
    auto dx = at::empty({T, H}, dout.options());
    if (T > 0) {
        moe_scatter_bwd_kernel<<<(unsigned)T, 256, 0, current_stream()>>>((const bf16*)dout.data_ptr(),
                                                                          slots.data_ptr<int>(), (bf16*)dx.data_ptr(), H, K);
        ATB_LAUNCH_CHECK();
    }
    return dx;
}

at::Tensor moe_gather_fwd(const at::Tensor& y, const at::Tensor& slots, const at::Tensor& scores) {
    check_rows(y, "gather y");
    ATB_CHECK_DTYPE(slots, at::kInt); ATB_CHECK_CONTIG(slots); ATB_CHECK_DTYPE(scores, at::kFloat); ATB_CHECK_CONTIG(scores);
    const int64_t T = slots.size(0);
    const int H = (int)y.size(1), K = (int)slots.size(1);
    c10::cuda::CUDAGuard guard(y.device());
    auto out = at::empty({T, H}, y.options());
    if (T > 0) {
        moe_gather_fwd_kernel<<<(unsigned)T, 256, 0, current_stream()>>>((const bf16*)y.data_ptr(), slots.data_ptr<int>(),
                                                                         scores.data_ptr<float>(), (bf16*)out.data_ptr(), H, K);
        ATB_LAUNCH_CHECK();
    }
    return out;
}

std::tuple<at::Tensor, at::Tensor> moe_gather_bwd(const at::Tensor& dout, const at::Tensor& y, const at::Tensor& slots,
                                                  const at::Tensor& scores) {
    check_rows(dout, "gather dout");
    check_rows(y, "gather y");
    const int64_t T = slots.size(0);
    const int H = (int)y.size(1), K = (int)slots.size(1);
    c10::cuda::CUDAGuard guard(y.device());
    auto dy = at::zeros_like(y);  // rows that belong to no token (padding) keep a zero gradient
    auto dscores = at::empty({T, K}, scores.options());
    if (T > 0) {
        moe_gather_bwd_kernel<<<(unsigned)T, 256, 0, current_stream()>>>(
            (const bf16*)dout.data_ptr(), (const bf16*)y.data_ptr(), slots.data_ptr<int>(), scores.data_ptr<float>(),
            (bf16*)dy.data_ptr(), dscores.data_ptr<float>(), H, K);
        ATB_LAUNCH_CHECK();
    }
    return {dy, dscores};
}

}  // namespace atb
