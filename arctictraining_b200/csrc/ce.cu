// SPDX-License-Identifier: Apache-2.0
// Cross-entropy over one chunk of logits, forward and backward in a single kernel.
//
// For every row: loss = logsumexp(logits) - logits[label]; the logits are then overwritten in place by
// d(loss_sum)/d(logits) * grad_scale = (softmax - onehot(label)) * grad_scale.  Rows whose label is
// -100 get loss 0 and a zero gradient.  The [tokens, vocab] matrix is the output of the lm_head GEMM
// for one sequence tile, so the full-sequence logits never exist in memory; this replaces the Triton
// fused-linear-cross-entropy and the tiled logits+loss autograd function used by the reference
// (arctic_training/trainer/sft_trainer.py:79-156).
//
// One CTA of 512 threads per row; two passes over the row (the second is served from L2): online
// max / sum-of-exponentials, then the gradient write.  `grad_scale` is read from device memory so the
// 1/(number of valid tokens) factor computed on the device needs no host synchronisation.

#include "common.cuh"

namespace atb {

__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(bf16* __restrict__ logits, int64_t ld,
                                                         const int64_t* __restrict__ labels,
                                                         float* __restrict__ loss, float* __restrict__ lse_out, int V,
                                                         const float* __restrict__ grad_scale_ptr,
                                                         const float* __restrict__ row_scale, int write_grad) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    bf16* lr = logits + row * ld;
    const int64_t label = labels[row];
    const int nvec = V >> 3;
    const bool valid = (label >= 0 && label < V);

    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(reinterpret_cast<const bf16x8*>(lr)[i], f);
        float lm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
        const float nm = fmaxf(m, lm);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
        s = s * __expf(m - nm) + acc;
        m = nm;
    }
    const float gmax = block_max(m, scratch);
    const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gmax);
    const float gsum = block_sum(contrib, scratch);
    const float lse = gmax + __logf(gsum);
    if (threadIdx.x == 0) {
        const float xl = valid ? __bfloat162float(lr[label]) : 0.f;
        loss[row] = valid ? (lse - xl) : 0.f;
        if (lse_out) lse_out[row] = lse;
    }
    if (!write_grad) return;
    __syncthreads();  // the label logit has been read before anyone overwrites it
    const float gs = valid ? (grad_scale_ptr ? *grad_scale_ptr : 1.f) * (row_scale ? row_scale[row] : 1.f) : 0.f;
    const float inv = 1.f / gsum;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(reinterpret_cast<const bf16x8*>(lr)[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float pr = __expf(f[j] - gmax) * inv;
            if ((int64_t)(i * 8 + j) == label) pr -= 1.f;
            f[j] = pr * gs;
        }
        reinterpret_cast<bf16x8*>(lr)[i] = pack8(f);
    }
}

// Distillation loss over one tile: KL(softmax(t / T) || softmax(s / T)) * T^2 per row, with the student logits
// overwritten in place by the gradient  T * (softmax(s / T) - softmax(t / T)) * row_weight[row] * grad_scale.
// Replaces the tiled KL-divergence loss of the reference's SwiftKV trainer (projects/swiftkv/train.py:176-224).
__global__ void __launch_bounds__(512) kl_fwd_bwd_kernel(bf16* __restrict__ student, const bf16* __restrict__ teacher,
                                                         int64_t ld_s, int64_t ld_t, const float* __restrict__ row_weight,
                                                         float* __restrict__ loss, int V, float inv_temp,
                                                         const float* __restrict__ grad_scale_ptr, int write_grad) {
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    bf16* sr = student + row * ld_s;
    const bf16* tr = teacher + row * ld_t;
    const int nvec = V >> 3;
    const float wgt = row_weight ? row_weight[row] : 1.f;
    float ms = -INFINITY, ss = 0.f, mt = -INFINITY, st = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float a[8], b[8];
        unpack8(reinterpret_cast<const bf16x8*>(sr)[i], a);
        unpack8(reinterpret_cast<const bf16x8*>(tr)[i], b);
        float la = a[0] * inv_temp, lb = b[0] * inv_temp;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            a[j] *= inv_temp;
            b[j] *= inv_temp;
            la = fmaxf(la, a[j]);
            lb = fmaxf(lb, b[j]);
        }
        const float nms = fmaxf(ms, la), nmt = fmaxf(mt, lb);
        float acc_s = 0.f, acc_t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc_s += __expf(a[j] - nms);
            acc_t += __expf(b[j] - nmt);
        }
        ss = ss * __expf(ms - nms) + acc_s;
        st = st * __expf(mt - nmt) + acc_t;
        ms = nms;
        mt = nmt;
    }
    const float gms = block_max(ms, scratch);
    const float gss = block_sum(ms == -INFINITY ? 0.f : ss * __expf(ms - gms), scratch);
    const float gmt = block_max(mt, scratch);
    const float gst = block_sum(mt == -INFINITY ? 0.f : st * __expf(mt - gmt), scratch);
    const float lse_s = gms + __logf(gss), lse_t = gmt + __logf(gst);
    const float gs = (grad_scale_ptr ? *grad_scale_ptr : 1.f) * wgt / inv_temp;  // T * weight * scale
    float kl = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float a[8], b[8];
        unpack8(reinterpret_cast<const bf16x8*>(sr)[i], a);
        unpack8(reinterpret_cast<const bf16x8*>(tr)[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float ls = a[j] * inv_temp - lse_s, lt = b[j] * inv_temp - lse_t;
            const float pt = __expf(lt), ps = __expf(ls);
            kl += pt * (lt - ls);
            a[j] = (ps - pt) * gs;
        }
        if (write_grad) reinterpret_cast<bf16x8*>(sr)[i] = pack8(a);
    }
    kl = block_sum(kl, scratch);
    if (threadIdx.x == 0) loss[row] = kl * wgt / (inv_temp * inv_temp);
}

at::Tensor kl_fwd_bwd(at::Tensor student, const at::Tensor& teacher, const c10::optional<at::Tensor>& row_weight,
                      double temperature, const c10::optional<at::Tensor>& grad_scale, bool write_grad) {
    ATB_CHECK_CUDA(student); ATB_CHECK_DTYPE(student, at::kBFloat16); ATB_CHECK_DTYPE(teacher, at::kBFloat16);
    TORCH_CHECK(student.dim() == 2 && teacher.dim() == 2 && student.sizes() == teacher.sizes(), "kl: logits must be two [T, V] tensors");
    TORCH_CHECK(student.stride(1) == 1 && teacher.stride(1) == 1, "kl: unit inner stride");
    const int64_t T = student.size(0);
    const int V = (int)student.size(1);
    TORCH_CHECK(V % 8 == 0 && student.stride(0) % 8 == 0 && teacher.stride(0) % 8 == 0, "kl: vocab and pitches must be multiples of 8");
    ATB_CHECK_ALIGNED16(student); ATB_CHECK_ALIGNED16(teacher);
    c10::cuda::CUDAGuard guard(student.device());
    auto loss = at::empty({T}, student.options().dtype(at::kFloat));
    const float* rw = nullptr;
    if (row_weight.has_value()) {
        ATB_CHECK_DTYPE(*row_weight, at::kFloat); ATB_CHECK_CONTIG(*row_weight);
        TORCH_CHECK(row_weight->numel() == T, "kl: one weight per row");
        rw = row_weight->data_ptr<float>();
    }
    const float* gs = nullptr;
    if (grad_scale.has_value()) {
        ATB_CHECK_DTYPE(*grad_scale, at::kFloat);
        gs = grad_scale->data_ptr<float>();
    }
    if (T > 0) {
        kl_fwd_bwd_kernel<<<(unsigned)T, 512, 0, current_stream()>>>((bf16*)student.data_ptr(), (const bf16*)teacher.data_ptr(),
                                                                     student.stride(0), teacher.stride(0), rw,
                                                                     loss.data_ptr<float>(), V, (float)(1.0 / temperature), gs,
                                                                     write_grad ? 1 : 0);
        ATB_LAUNCH_CHECK();
    }
    return loss;
}

// logits [T, V] bf16 (modified in place when write_grad), labels [T] int64 -> (loss [T] fp32, lse [T] fp32).
// The gradient of row t is scaled by grad_scale[0] * row_scale[t] (both optional).
std::tuple<at::Tensor, at::Tensor> ce_fwd_bwd(at::Tensor logits, const at::Tensor& labels,
                                              const c10::optional<at::Tensor>& grad_scale,
                                              const c10::optional<at::Tensor>& row_scale, bool write_grad) {
    ATB_CHECK_CUDA(logits); ATB_CHECK_DTYPE(logits, at::kBFloat16); ATB_CHECK_DTYPE(labels, at::kLong);
    ATB_CHECK_CONTIG(labels);
    TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "ce: logits must be [T, V] with unit inner stride");
    const int64_t T = logits.size(0);
    const int V = (int)logits.size(1);
    TORCH_CHECK(V % 8 == 0 && logits.stride(0) % 8 == 0, "ce: vocab and row pitch must be multiples of 8");
    TORCH_CHECK(labels.numel() == T, "ce: one label per row");
    ATB_CHECK_ALIGNED16(logits);
    c10::cuda::CUDAGuard guard(logits.device());
    auto loss = at::empty({T}, logits.options().dtype(at::kFloat));
    auto lse = at::empty({T}, logits.options().dtype(at::kFloat));
    const float* gs = nullptr;
    if (grad_scale.has_value()) {
        ATB_CHECK_DTYPE(*grad_scale, at::kFloat);
        gs = grad_scale->data_ptr<float>();
    }
    const float* rs = nullptr;
    if (row_scale.has_value()) {
        ATB_CHECK_DTYPE(*row_scale, at::kFloat); ATB_CHECK_CONTIG(*row_scale);
        TORCH_CHECK(row_scale->numel() == T, "ce: one row scale per row");
        rs = row_scale->data_ptr<float>();
    }
    if (T > 0) {
        ce_fwd_bwd_kernel<<<(unsigned)T, 512, 0, current_stream()>>>((bf16*)logits.data_ptr(), logits.stride(0),
                                                                     labels.data_ptr<int64_t>(), loss.data_ptr<float>(),
                                                                     lse.data_ptr<float>(), V, gs, rs, write_grad ? 1 : 0);
        ATB_LAUNCH_CHECK();
    }
    return {loss, lse};
}

}  // namespace atb
