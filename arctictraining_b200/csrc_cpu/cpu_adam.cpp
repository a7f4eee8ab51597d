// SPDX-License-Identifier: Apache-2.0
// Host-side AdamW for optimizer states that live in (pinned) host memory: one fused pass over master weights, moments
// and gradient, spread over ATen's intra-op thread pool, with the bf16 copy of the updated weights written in the same pass.  The reference gets
// this from its engine dependency's vectorised host optimizer (arctic_training/optimizer/adam_factory.py:100-126).
//
// Vector width is chosen at run time (function multi-versioning), so a library built on one machine runs on another.

#include <torch/extension.h>

#include <cmath>
#include <cstdint>
#include <cstring>

#include <ATen/Parallel.h>

namespace {

inline uint16_t float_to_bf16_rn(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

__attribute__((target_clones("avx512f", "avx2", "default")))
void adamw_range(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 uint16_t* __restrict__ lp, int64_t n, float lr, float b1, float b2, float eps, float wd, float inv_bc1,
                 float inv_sqrt_bc2, float gs) {
    const float decay = 1.f - lr * wd;
#pragma omp simd
    for (int64_t i = 0; i < n; ++i) {
        const float gi = g[i] * gs;
        const float mi = b1 * m[i] + (1.f - b1) * gi;
        const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        const float denom = std::sqrt(vi) * inv_sqrt_bc2 + eps;
        const float pi = p[i] * decay - lr * (mi * inv_bc1) / denom;
        m[i] = mi;
        v[i] = vi;
        p[i] = pi;
    }
    if (lp != nullptr)
        for (int64_t i = 0; i < n; ++i) lp[i] = float_to_bf16_rn(p[i]);
}

}  // namespace

// master / grad / exp_avg / exp_avg_sq: contiguous fp32 CPU tensors of equal length; out_lp: optional bf16 CPU tensor
// that receives the rounded updated weights (typically pinned, then copied to the device asynchronously).
void cpu_adamw_step(at::Tensor master, const at::Tensor& grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
                    const c10::optional<at::Tensor>& out_lp, double lr, double beta1, double beta2, double eps, double wd,
                    int64_t step, double grad_scale) {
    TORCH_CHECK(master.device().is_cpu() && grad.device().is_cpu() && exp_avg.device().is_cpu() && exp_avg_sq.device().is_cpu(),
                "cpu_adamw_step: host tensors expected");
    TORCH_CHECK(master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat && exp_avg.scalar_type() == at::kFloat &&
                exp_avg_sq.scalar_type() == at::kFloat, "cpu_adamw_step: fp32 tensors expected");
    TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && exp_avg.is_contiguous() && exp_avg_sq.is_contiguous(),
                "cpu_adamw_step: contiguous tensors expected");
    const int64_t n = master.numel();
    TORCH_CHECK(grad.numel() == n && exp_avg.numel() == n && exp_avg_sq.numel() == n, "cpu_adamw_step: size mismatch");
    uint16_t* lp = nullptr;
    if (out_lp.has_value()) {
        TORCH_CHECK(out_lp->device().is_cpu() && out_lp->scalar_type() == at::kBFloat16 && out_lp->is_contiguous() &&
                    out_lp->numel() == n, "cpu_adamw_step: out_lp must be a contiguous bf16 host tensor of the same length");
        lp = reinterpret_cast<uint16_t*>(out_lp->data_ptr());
    }
    const float inv_bc1 = 1.f / (1.f - (float)std::pow(beta1, (double)step));
    const float inv_sqrt_bc2 = 1.f / std::sqrt(1.f - (float)std::pow(beta2, (double)step));
    float* p = master.data_ptr<float>();
    const float* g = grad.data_ptr<float>();
    float* m = exp_avg.data_ptr<float>();
    float* v = exp_avg_sq.data_ptr<float>();
    constexpr int64_t kChunk = 1 << 16;
    const int64_t chunks = (n + kChunk - 1) / kChunk;
    at::parallel_for(0, chunks, 1, [&](int64_t begin, int64_t end) {
        for (int64_t c = begin; c < end; ++c) {
            const int64_t lo = c * kChunk, len = std::min(kChunk, n - lo);
            adamw_range(p + lo, g + lo, m + lo, v + lo, lp ? lp + lo : nullptr, len, (float)lr, (float)beta1, (float)beta2,
                        (float)eps, (float)wd, inv_bc1, inv_sqrt_bc2, (float)grad_scale);
        }
    });
}

TORCH_LIBRARY(atb200_cpu, m) {
    m.def("cpu_adamw_step(Tensor(a!) master, Tensor grad, Tensor(b!) exp_avg, Tensor(c!) exp_avg_sq, Tensor? out_lp, float lr, "
          "float beta1, float beta2, float eps, float wd, int step, float grad_scale) -> ()", &cpu_adamw_step);
}
