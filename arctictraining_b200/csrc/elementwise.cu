// SPDX-License-Identifier: Apache-2.0
// Bandwidth-bound fused kernels: RMSNorm (fwd/bwd), rotary embedding, SwiGLU (fwd/bwd),
// fused AdamW on flat shards, squared-norm partials.  All kernels use 16-byte vector accesses and
// 64-bit row offsets (sequences of millions of tokens).
//
// These replace the Triton kernels (RMSNorm / RoPE / SwiGLU) and the multi-tensor Adam kernel that
// the reference obtains from third-party packages (arctic_training/model/liger_factory.py:27-69,
// arctic_training/optimizer/adam_factory.py:77-81).

#include "common.cuh"
#include "rmsnorm_kernels.cuh"

namespace atb {

// ---------------------------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w.  A CTA of 128 threads walks rows blockIdx.x, + gridDim.x, ...;
// a row lives in registers between the reduction and the scaling (one read of x), the weight vector is read once per
// CTA, and the next row is already in flight while the current one is reduced.
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(128) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          bf16* __restrict__ y, float* __restrict__ rstd, int64_t T, int H,
                                                          float eps) {
    __shared__ float scratch[2][4];
    const int nvec = H >> 3;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float wreg[VPT][8];
    const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * 128;
        if (i < nvec) unpack8(wr[i], wreg[v]);
    }
    bf16x8 cur[VPT], nxt[VPT];
    int64_t row = blockIdx.x;
    if (row < T) {
        const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 128;
            if (i < nvec) cur[v] = xr[i];
        }
    }
    int parity = 0;
    for (; row < T; row += gridDim.x, parity ^= 1) {
        const int64_t next = row + gridDim.x;
        if (next < T) {
            const bf16x8* xn = reinterpret_cast<const bf16x8*>(x + next * H);
#pragma unroll
            for (int v = 0; v < VPT; ++v) {
                const int i = threadIdx.x + v * 128;
                if (i < nvec) nxt[v] = xn[i];
            }
        }
        float f[VPT][8];
        float ss = 0.f;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 128;
            if (i < nvec) {
                unpack8(cur[v], f[v]);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += f[v][j] * f[v][j];
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) scratch[parity][warp] = ss;
        __syncthreads();  // one barrier per row: the scratch slots alternate
        ss = scratch[parity][0] + scratch[parity][1] + scratch[parity][2] + scratch[parity][3];
        const float r = rsqrtf(ss / (float)H + eps);
        if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
        bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * H);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 128;
            if (i < nvec) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[v][j] = f[v][j] * r * wreg[v][j];
                yr[i] = pack8(f[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < VPT; ++v) cur[v] = nxt[v];
    }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding, in place, rotate-half convention: pairs (x[i], x[i + D/2]).
// x is [T, NH, D] (row stride given), cos/sin are [T, D/2] fp32.  One CTA per token.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(bf16* __restrict__ x, int64_t row_stride, int NH, int D,
                                                   const float* __restrict__ cosb, const float* __restrict__ sinb,
                                                   float sin_sign) {
    const int64_t t = blockIdx.x;
    const int d2 = D >> 1;
    const int pairs_vec = d2 >> 3;  // 8 pairs per vector op
    bf16* base = x + t * row_stride;
    const float* c = cosb + t * d2;
    const float* s = sinb + t * d2;
    for (int idx = threadIdx.x; idx < NH * pairs_vec; idx += blockDim.x) {
        const int h = idx / pairs_vec, pv = idx % pairs_vec;
        bf16x8* lo = reinterpret_cast<bf16x8*>(base + (int64_t)h * D + pv * 8);
        bf16x8* hi = reinterpret_cast<bf16x8*>(base + (int64_t)h * D + d2 + pv * 8);
        float a[8], b[8], oa[8], ob[8];
        unpack8(*lo, a);
        unpack8(*hi, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float cc = c[pv * 8 + j], ssn = s[pv * 8 + j] * sin_sign;
            oa[j] = a[j] * cc - b[j] * ssn;
            ob[j] = b[j] * cc + a[j] * ssn;
        }
        *lo = pack8(oa);
        *hi = pack8(ob);
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on a block-interleaved gate/up tensor: columns [128b, 128b+64) are gate, [128b+64, 128b+128) up.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out,
                                                         int64_t T, int I) {
    const int vec_per_row = I >> 3;
    const int64_t total = T * vec_per_row;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / vec_per_row;
        const int j = (int)(idx % vec_per_row) * 8;
        const int blk = j >> 6, jj = j & 63;
        const bf16* row = gu + t * (2 * (int64_t)I) + blk * 128;
        float g[8], u[8], o[8];
        unpack8(*reinterpret_cast<const bf16x8*>(row + jj), g);
        unpack8(*reinterpret_cast<const bf16x8*>(row + 64 + jj), u);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
        *reinterpret_cast<bf16x8*>(out + t * (int64_t)I + j) = pack8(o);
    }
}

// `h_out` (optional): also writes h = silu(gate) * up again, for a caller that did not keep it after the forward.
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu,
                                                         bf16* __restrict__ dgu, bf16* __restrict__ h_out, int64_t T,
                                                         int I) {
    // Two 8-element pieces per thread and iteration, all six loads issued before the arithmetic: the kernel moves
    // six streams (three in, three out) and is bound by the number of loads in flight per SM.
    const int vec_per_row = I >> 3;
    const int64_t total = T * vec_per_row;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx0 < total; idx0 += 2 * step) {
        int64_t off[2], hoff[2];
        bool live[2];
        bf16x8 rg[2], ru[2], rd[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int64_t idx = idx0 + q * step;
            live[q] = idx < total;
            const int64_t t = live[q] ? idx / vec_per_row : 0;
            const int j = live[q] ? (int)(idx - t * vec_per_row) * 8 : 0;
            off[q] = t * (2 * (int64_t)I) + (j >> 6) * 128 + (j & 63);
            hoff[q] = t * (int64_t)I + j;
            if (live[q]) {
                rg[q] = *reinterpret_cast<const bf16x8*>(gu + off[q]);
                ru[q] = *reinterpret_cast<const bf16x8*>(gu + off[q] + 64);
                rd[q] = *reinterpret_cast<const bf16x8*>(dout + hoff[q]);
            }
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            if (!live[q]) continue;
            float g[8], u[8], d[8], dg[8], du[8], hh[8];
            unpack8(rg[q], g);
            unpack8(ru[q], u);
            unpack8(rd[q], d);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float sig = 1.f / (1.f + __expf(-g[k]));
                const float silu = g[k] * sig;
                dg[k] = d[k] * u[k] * (sig * (1.f + g[k] * (1.f - sig)));
                du[k] = d[k] * silu;
                hh[k] = silu * u[k];
            }
            *reinterpret_cast<bf16x8*>(dgu + off[q]) = pack8(dg);
            *reinterpret_cast<bf16x8*>(dgu + off[q] + 64) = pack8(du);
            if (h_out) *reinterpret_cast<bf16x8*>(h_out + hoff[q]) = pack8(hh);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fused AdamW on a flat fp32 shard: reads grad (fp32), updates exp_avg / exp_avg_sq / master and
// writes the bf16 parameter copy.  `grad_scale` is read from device memory so that a clip factor
// computed on the device needs no host round trip.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 load_grad4(const float* g, int64_t i) { return reinterpret_cast<const float4*>(g)[i]; }
__device__ __forceinline__ float4 load_grad4(const bf16* g, int64_t i) {
    const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float load_grad1(const float* g, int64_t i) { return g[i]; }
__device__ __forceinline__ float load_grad1(const bf16* g, int64_t i) { return __bfloat162float(g[i]); }

template <typename G>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, const G* __restrict__ grad,
                                                    float* __restrict__ m, float* __restrict__ v,
                                                    bf16* __restrict__ out_lp, int64_t n, float lr, float beta1,
                                                    float beta2, float eps, float wd, float bc1, float bc2,
                                                    const float* __restrict__ grad_scale_ptr) {
    const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
    const int64_t nvec = n >> 2;
    const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        float4 p = reinterpret_cast<float4*>(master)[i];
        float4 g = load_grad4(grad, i);
        float4 mm = reinterpret_cast<float4*>(m)[i];
        float4 vv = reinterpret_cast<float4*>(v)[i];
        float* pp = &p.x;
        float* gp = &g.x;
        float* mp = &mm.x;
        float* vp = &vv.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gk = gp[k] * gs;
            mp[k] = beta1 * mp[k] + (1.f - beta1) * gk;
            vp[k] = beta2 * vp[k] + (1.f - beta2) * gk * gk;
            const float denom = sqrtf(vp[k]) * inv_sqrt_bc2 + eps;
            pp[k] = pp[k] * (1.f - lr * wd) - lr * (mp[k] * inv_bc1) / denom;
        }
        reinterpret_cast<float4*>(master)[i] = p;
        reinterpret_cast<float4*>(m)[i] = mm;
        reinterpret_cast<float4*>(v)[i] = vv;
        if (out_lp) {
            bf162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out_lp)[i] = pk;
        }
    }
    // tail (n not a multiple of 4)
    for (int64_t i = (nvec << 2) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float gk = load_grad1(grad, i) * gs;
        const float mk = beta1 * m[i] + (1.f - beta1) * gk;
        const float vk = beta2 * v[i] + (1.f - beta2) * gk * gk;
        const float denom = sqrtf(vk) * inv_sqrt_bc2 + eps;
        const float pk = master[i] * (1.f - lr * wd) - lr * (mk * inv_bc1) / denom;
        m[i] = mk;
        v[i] = vk;
        master[i] = pk;
        if (out_lp) out_lp[i] = __float2bfloat16_rn(pk);
    }
}

// Deterministic squared-norm partials: out[blockIdx.x] = sum of x^2 over this CTA's grid-stride slice.
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ out) {
    __shared__ float scratch[32];
    float acc = 0.f;
    const int64_t nvec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? (n >> 2) : 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 f = load_grad4(x, i);
        acc += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
    }
    for (int64_t i = (nvec << 2) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float f = load_grad1(x, i);
        acc += f * f;
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = acc;
}

// bf16 -> fp32 accumulate: acc (+)= scale * src ; optional squared-norm partials of the result.
__global__ void __launch_bounds__(256) accum_bf16_kernel(const bf16* __restrict__ src, float* __restrict__ acc,
                                                         int64_t n, float scale, int overwrite) {
    const int64_t nvec = n >> 3;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        float f[8];
        unpack8(reinterpret_cast<const bf16x8*>(src)[i], f);
        float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
        float4 a0 = overwrite ? make_float4(0, 0, 0, 0) : a[0];
        float4 a1 = overwrite ? make_float4(0, 0, 0, 0) : a[1];
        a0.x += scale * f[0]; a0.y += scale * f[1]; a0.z += scale * f[2]; a0.w += scale * f[3];
        a1.x += scale * f[4]; a1.y += scale * f[5]; a1.z += scale * f[6]; a1.w += scale * f[7];
        a[0] = a0;
        a[1] = a1;
    }
    for (int64_t i = (nvec << 3) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float f = __bfloat162float(src[i]) * scale;
        acc[i] = overwrite ? f : acc[i] + f;
    }
}

// ---------------------------------------------------------------------------------------------
// Host wrappers
// ---------------------------------------------------------------------------------------------
static int grid_for(int64_t work_items, int threads = 256, int waves = 8) {
    int64_t g = ceil_div(work_items, threads);
    int64_t cap = (int64_t)kNumSMs * waves;
    return (int)std::max<int64_t>(1, std::min<int64_t>(g, cap));
}

std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps) {
    ATB_CHECK_CUDA(x); ATB_CHECK_CONTIG(x); ATB_CHECK_CONTIG(w);
    ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_DTYPE(w, at::kBFloat16);
    const int H = (int)x.size(-1);
    TORCH_CHECK(H % 8 == 0 && H <= 16384 && w.numel() == H, "rmsnorm: hidden size must be a multiple of 8, at most 16384, and match the weight");
    ATB_CHECK_ALIGNED16(x); ATB_CHECK_ALIGNED16(w);
    const int64_t T = x.numel() / H;
    c10::cuda::CUDAGuard guard(x.device());
    auto y = at::empty_like(x);
    auto rstd = at::empty({T}, x.options().dtype(at::kFloat));
    if (T > 0) {
        const int nvec = H / 8;
        const int vpt = (int)ceil_div(nvec, 128);
        const unsigned grid = (unsigned)std::min<int64_t>(T, (int64_t)kNumSMs * 16);
        auto launch = [&](auto tag) {
            constexpr int V = decltype(tag)::value;
            rmsnorm_fwd_kernel<V><<<grid, 128, 0, current_stream()>>>(
                (const bf16*)x.data_ptr(), (const bf16*)w.data_ptr(), (bf16*)y.data_ptr(), rstd.data_ptr<float>(), T, H,
                (float)eps);
        };
        if (vpt <= 1) launch(std::integral_constant<int, 1>{});
        else if (vpt <= 2) launch(std::integral_constant<int, 2>{});
        else if (vpt <= 4) launch(std::integral_constant<int, 4>{});
        else if (vpt <= 8) launch(std::integral_constant<int, 8>{});
        else launch(std::integral_constant<int, 16>{});
        ATB_LAUNCH_CHECK();
    }
    return {y, rstd};
}

std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w,
                                               const at::Tensor& rstd) {
    ATB_CHECK_CUDA(dy); ATB_CHECK_CONTIG(dy); ATB_CHECK_CONTIG(x);
    ATB_CHECK_DTYPE(dy, at::kBFloat16); ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_DTYPE(rstd, at::kFloat);
    const int H = (int)x.size(-1);
    const int64_t T = x.numel() / H;
    TORCH_CHECK(H % 8 == 0 && H <= 8 * 256 * 8, "rmsnorm_bwd: hidden size must be a multiple of 8 and <= 16384");
    ATB_CHECK_ALIGNED16(dy); ATB_CHECK_ALIGNED16(x);
    c10::cuda::CUDAGuard guard(x.device());
    auto dx = at::empty_like(x);
    const int nblk = (int)std::max<int64_t>(1, std::min<int64_t>(T, (int64_t)kNumSMs * 4));
    auto dwp = at::empty({nblk, H}, x.options().dtype(at::kFloat));
    if (T > 0) {
        const int nvec = H / 8;
        const int vpt = (int)ceil_div(nvec, 256);
        auto launch = [&](auto tag) {
            constexpr int V = decltype(tag)::value;
            rmsnorm_bwd_kernel<V><<<nblk, 256, 0, current_stream()>>>(
                (const bf16*)dy.data_ptr(), (const bf16*)x.data_ptr(), (const bf16*)w.data_ptr(),
                rstd.data_ptr<float>(), (bf16*)dx.data_ptr(), dwp.data_ptr<float>(), T, H);
        };
        if (vpt <= 1) launch(std::integral_constant<int, 1>{});
        else if (vpt <= 2) launch(std::integral_constant<int, 2>{});
        else if (vpt <= 4) launch(std::integral_constant<int, 4>{});
        else launch(std::integral_constant<int, 8>{});
        ATB_LAUNCH_CHECK();
    } else {
        dwp.zero_();
    }
    return {dx, dwp.sum(0)};
}

void rope_inplace(at::Tensor x, const at::Tensor& cosb, const at::Tensor& sinb, bool inverse) {
    // x: [T, NH, D] view whose last two dims are dense; the token stride may be larger (fused qkv buffer).
    ATB_CHECK_CUDA(x); ATB_CHECK_DTYPE(x, at::kBFloat16);
    ATB_CHECK_DTYPE(cosb, at::kFloat); ATB_CHECK_CONTIG(cosb); ATB_CHECK_CONTIG(sinb);
    TORCH_CHECK(x.dim() == 3, "rope: x must be [T, heads, head_dim]");
    const int64_t T = x.size(0);
    const int NH = (int)x.size(1), D = (int)x.size(2);
    TORCH_CHECK(x.stride(2) == 1 && x.stride(1) == D, "rope: heads must be dense");
    TORCH_CHECK(D % 16 == 0, "rope: head_dim must be a multiple of 16");
    TORCH_CHECK(x.stride(0) % 8 == 0, "rope: token stride must be a multiple of 8 elements");
    TORCH_CHECK(cosb.numel() == T * (D / 2) && sinb.numel() == T * (D / 2), "rope: cos/sin must be [T, D/2]");
    ATB_CHECK_ALIGNED16(x);
    if (T == 0) return;
    c10::cuda::CUDAGuard guard(x.device());
    rope_kernel<<<(unsigned)T, 256, 0, current_stream()>>>((bf16*)x.data_ptr(), x.stride(0), NH, D,
                                                           cosb.data_ptr<float>(), sinb.data_ptr<float>(),
                                                           inverse ? -1.f : 1.f);
    ATB_LAUNCH_CHECK();
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
    ATB_CHECK_CUDA(gu); ATB_CHECK_CONTIG(gu); ATB_CHECK_DTYPE(gu, at::kBFloat16); ATB_CHECK_ALIGNED16(gu);
    const int64_t two_i = gu.size(-1);
    TORCH_CHECK(two_i % 128 == 0, "swiglu: last dim must be a multiple of 128 (block-interleaved gate/up)");
    const int I = (int)(two_i / 2);
    const int64_t T = gu.numel() / two_i;
    auto sizes = gu.sizes().vec();
    sizes.back() = I;
    c10::cuda::CUDAGuard guard(gu.device());
    auto out = at::empty(sizes, gu.options());
    if (T > 0) {
        swiglu_fwd_kernel<<<grid_for(T * (I / 8)), 256, 0, current_stream()>>>((const bf16*)gu.data_ptr(),
                                                                                 (bf16*)out.data_ptr(), T, I);
        ATB_LAUNCH_CHECK();
    }
    return out;
}

at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& gu) {
    ATB_CHECK_CUDA(gu); ATB_CHECK_CONTIG(gu); ATB_CHECK_CONTIG(dout);
    ATB_CHECK_DTYPE(gu, at::kBFloat16); ATB_CHECK_DTYPE(dout, at::kBFloat16);
    ATB_CHECK_ALIGNED16(gu); ATB_CHECK_ALIGNED16(dout);
    const int64_t two_i = gu.size(-1);
    const int I = (int)(two_i / 2);
    const int64_t T = gu.numel() / two_i;
    TORCH_CHECK(dout.numel() == T * I, "swiglu_bwd: shape mismatch");
    c10::cuda::CUDAGuard guard(gu.device());
    auto dgu = at::empty_like(gu);
    if (T > 0) {
        swiglu_bwd_kernel<<<grid_for(T * (I / 8)), 256, 0, current_stream()>>>(
            (const bf16*)dout.data_ptr(), (const bf16*)gu.data_ptr(), (bf16*)dgu.data_ptr(), nullptr, T, I);
        ATB_LAUNCH_CHECK();
    }
    return dgu;
}

// Backward of the SwiGLU activation that also returns h = silu(gate) * up, for callers that did not keep it.
std::tuple<at::Tensor, at::Tensor> swiglu_bwd_recompute(const at::Tensor& dout, const at::Tensor& gu) {
    ATB_CHECK_CUDA(gu); ATB_CHECK_CONTIG(gu); ATB_CHECK_CONTIG(dout);
    ATB_CHECK_DTYPE(gu, at::kBFloat16); ATB_CHECK_DTYPE(dout, at::kBFloat16);
    TORCH_CHECK(gu.dim() == 2 && dout.dim() == 2 && gu.size(1) == 2 * dout.size(1) && gu.size(0) == dout.size(0) &&
                gu.size(1) % 128 == 0, "swiglu_bwd_recompute: shape mismatch");
    const int64_t T = gu.size(0);
    const int I = (int)dout.size(1);
    c10::cuda::CUDAGuard guard(gu.device());
    auto dgu = at::empty_like(gu);
    auto h = at::empty_like(dout);
    if (T > 0) {
        swiglu_bwd_kernel<<<grid_for(T * (I / 8)), 256, 0, current_stream()>>>(
            (const bf16*)dout.data_ptr(), (const bf16*)gu.data_ptr(), (bf16*)dgu.data_ptr(), (bf16*)h.data_ptr(), T, I);
        ATB_LAUNCH_CHECK();
    }
    return {dgu, h};
}

void adamw_step(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                const c10::optional<at::Tensor>& out_lp, double lr, double beta1, double beta2, double eps,
                double wd, int64_t step, const c10::optional<at::Tensor>& grad_scale) {
    ATB_CHECK_CUDA(master); ATB_CHECK_CONTIG(master); ATB_CHECK_CONTIG(grad); ATB_CHECK_CONTIG(m); ATB_CHECK_CONTIG(v);
    ATB_CHECK_DTYPE(master, at::kFloat);
    TORCH_CHECK(grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16, "adamw: gradient must be fp32 or bf16");
    ATB_CHECK_DTYPE(m, at::kFloat); ATB_CHECK_DTYPE(v, at::kFloat);
    const int64_t n = master.numel();
    TORCH_CHECK(grad.numel() == n && m.numel() == n && v.numel() == n, "adamw: size mismatch");
    ATB_CHECK_ALIGNED16(master); ATB_CHECK_ALIGNED16(m); ATB_CHECK_ALIGNED16(v);
    TORCH_CHECK((reinterpret_cast<uintptr_t>(grad.data_ptr()) & (grad.scalar_type() == at::kFloat ? 15 : 7)) == 0,
                "adamw: gradient pointer is not aligned for vector loads");
    bf16* lp = nullptr;
    if (out_lp.has_value()) {
        ATB_CHECK_DTYPE(*out_lp, at::kBFloat16); ATB_CHECK_CONTIG(*out_lp);
        TORCH_CHECK(out_lp->numel() == n, "adamw: low-precision output size mismatch");
        TORCH_CHECK((reinterpret_cast<uintptr_t>(out_lp->data_ptr()) & 7) == 0, "adamw: out_lp must be 8-byte aligned");
        lp = (bf16*)out_lp->data_ptr();
    }
    const float* gs = nullptr;
    if (grad_scale.has_value()) {
        ATB_CHECK_DTYPE(*grad_scale, at::kFloat);
        gs = grad_scale->data_ptr<float>();
    }
    if (n == 0) return;
    c10::cuda::CUDAGuard guard(master.device());
    const float bc1 = 1.f - (float)std::pow(beta1, (double)step);
    const float bc2 = 1.f - (float)std::pow(beta2, (double)step);
    if (grad.scalar_type() == at::kFloat)
        adamw_kernel<float><<<grid_for(n / 4 + 1), 256, 0, current_stream()>>>(
            master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), lp, n, (float)lr,
            (float)beta1, (float)beta2, (float)eps, (float)wd, bc1, bc2, gs);
    else
        adamw_kernel<bf16><<<grid_for(n / 4 + 1), 256, 0, current_stream()>>>(
            master.data_ptr<float>(), (const bf16*)grad.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), lp, n, (float)lr,
            (float)beta1, (float)beta2, (float)eps, (float)wd, bc1, bc2, gs);
    ATB_LAUNCH_CHECK();
}

at::Tensor sumsq(const at::Tensor& x) {
    ATB_CHECK_CUDA(x); ATB_CHECK_CONTIG(x);
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "sumsq: fp32 or bf16 input");
    c10::cuda::CUDAGuard guard(x.device());
    const int nblk = grid_for(x.numel() / 4 + 1, 256, 4);
    auto partial = at::empty({nblk}, x.options().dtype(at::kFloat));
    if (x.scalar_type() == at::kFloat)
        sumsq_kernel<float><<<nblk, 256, 0, current_stream()>>>(x.data_ptr<float>(), x.numel(), partial.data_ptr<float>());
    else
        sumsq_kernel<bf16><<<nblk, 256, 0, current_stream()>>>((const bf16*)x.data_ptr(), x.numel(), partial.data_ptr<float>());
    ATB_LAUNCH_CHECK();
    return partial.sum();
}

void accum_bf16(const at::Tensor& src, at::Tensor acc, double scale, bool overwrite) {
    ATB_CHECK_CUDA(src); ATB_CHECK_CONTIG(src); ATB_CHECK_CONTIG(acc);
    ATB_CHECK_DTYPE(src, at::kBFloat16); ATB_CHECK_DTYPE(acc, at::kFloat);
    TORCH_CHECK(src.numel() == acc.numel(), "accum_bf16: size mismatch");
    ATB_CHECK_ALIGNED16(src); ATB_CHECK_ALIGNED16(acc);
    if (src.numel() == 0) return;
    c10::cuda::CUDAGuard guard(src.device());
    accum_bf16_kernel<<<grid_for(src.numel() / 8 + 1), 256, 0, current_stream()>>>(
        (const bf16*)src.data_ptr(), acc.data_ptr<float>(), src.numel(), (float)scale, overwrite ? 1 : 0);
    ATB_LAUNCH_CHECK();
}

}  // namespace atb
