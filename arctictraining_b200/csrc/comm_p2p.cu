// SPDX-License-Identifier: Apache-2.0
// Collectives written as plain kernels over NVLink peer memory (symmetric buffers that every rank of the node has
// mapped).  Kernels receive a device table of peer base pointers; data moves with 16-byte peer loads / stores issued
// from the SMs, so the transfer is part of the same kernel as the arithmetic that consumes it:
//
//   p2p_barrier              : flag exchange through peer stores with release/acquire semantics and a bounded wait
//   p2p_all_gather           : pull every peer's shard into the local full buffer (ZeRO-3 parameter gather)
//   p2p_reduce_scatter_accum : read this rank's slice of every peer's bf16 gradient buffer, sum in fp32 in rank
//                              order (deterministic), scale, accumulate into the fp32 gradient shard and emit the
//                              squared-norm partials needed for clipping
//   p2p_reduce_scatter_adamw : the same reduction feeding AdamW directly (single pass when no clip factor is needed)
//   nvls_reduce_scatter_accum: the reduction done inside the NVSwitch (multimem.ld_reduce on the multicast mapping)
//   p2p_seq_to_head / p2p_head_to_seq : the Ulysses all-to-all as direct pushes into the owners' buffers
//   p2p_moe_dispatch / p2p_moe_combine: expert-parallel token exchange straight into / out of the expert-major,
//                              tile-aligned buffer of the owning rank (no intermediate send/receive staging)
//
// None of these kernels waits on another rank except p2p_barrier, whose wait is bounded (it records an error code
// and returns).  The reference reaches all of this through NCCL calls made by its engine dependency
// (arctic_training/trainer/trainer.py:195-202,315-322; arctic_training/model/moe/alltoall.py:20-46).

#include "common.cuh"

#include <cstdlib>
#include "ptx_sm100.cuh"

namespace atb {

constexpr int kMaxPeers = 16;

struct PeerTable {
    void* ptr[kMaxPeers];
};

static PeerTable make_table(const at::Tensor& ptrs_cpu, int64_t byte_offset) {
    TORCH_CHECK(ptrs_cpu.device().is_cpu() && ptrs_cpu.scalar_type() == at::kLong, "peer pointers: int64 CPU tensor");
    TORCH_CHECK(ptrs_cpu.numel() <= kMaxPeers, "at most 16 peers");
    PeerTable t{};
    for (int i = 0; i < ptrs_cpu.numel(); ++i)
        t.ptr[i] = reinterpret_cast<void*>(ptrs_cpu.data_ptr<int64_t>()[i] + byte_offset);
    return t;
}

at::Tensor& error_flag_for_comm(const at::Device& dev) {
    static std::vector<at::Tensor> flags(64);
    auto& f = flags[dev.index() < 0 ? 0 : dev.index()];
    if (!f.defined()) f = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
    return f;
}

// ------------------------------------------------------------------------------------------- barrier
// flags: per rank a symmetric array of uint32 [slots][P].  Rank r writes `epoch` into flags_of_peer[slot][r] for
// every peer, then waits until its own flags[slot][p] >= epoch for every p.  Epochs only grow.
__global__ void p2p_barrier_kernel(PeerTable flags, int rank, int P, int slot, uint32_t epoch, uint64_t limit_ns,
                                   int* error_flag) {
    const int p = threadIdx.x;
    if (p >= P) return;
    __threadfence_system();
    uint32_t* remote = reinterpret_cast<uint32_t*>(flags.ptr[p]) + slot * kMaxPeers + rank;
    ptx::st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + slot * kMaxPeers + p;
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::ld_acquire_sys(mine) < epoch) {
        if (ptx::globaltimer_ns() - t0 > limit_ns) {
            atomicCAS(error_flag, 0, (9 << 8) | (p + 1));
            break;
        }
    }
    __threadfence_system();
}

// ------------------------------------------------------------------------------------------- all-gather (pull)
__global__ void __launch_bounds__(512) p2p_all_gather_kernel(PeerTable shards, uint4* __restrict__ full,
                                                             int64_t shard_vec, int rank, int P) {
    // grid.y = peer index; every CTA row streams one peer's shard
    const int peer = blockIdx.y;
    const uint4* src = reinterpret_cast<const uint4*>(shards.ptr[peer]);
    uint4* dst = full + (int64_t)peer * shard_vec;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < shard_vec; i += (int64_t)gridDim.x * blockDim.x) {
        dst[i] = src[i];
    }
}

// ------------------------------------------------------------------------------------------- reduce-scatter
template <bool ADAM>
__global__ void __launch_bounds__(256) p2p_reduce_scatter_kernel(
    PeerTable grads,  // bf16 buffers, already offset to this rank's slice
    int P, int64_t n, float scale, float* __restrict__ acc, int overwrite, float* __restrict__ sumsq_partial,
    // AdamW part (ADAM == true): acc is unused, the reduced gradient feeds the update directly
    float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, bf16* __restrict__ out_lp, float lr,
    float beta1, float beta2, float eps, float wd, float bc1, float bc2) {
    __shared__ float scratch[32];
    const int64_t nvec = n >> 3;
    float ss = 0.f;
    const float inv_bc1 = ADAM ? 1.f / bc1 : 0.f, inv_sqrt_bc2 = ADAM ? rsqrtf(bc2) : 0.f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int p = 0; p < P; ++p) {  // fixed order: bit-identical results on every run
            float f[8];
            unpack8(reinterpret_cast<const bf16x8*>(grads.ptr[p])[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] += f[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] *= scale;
        if constexpr (!ADAM) {
            float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
            float4 a0 = overwrite ? make_float4(0, 0, 0, 0) : a[0];
            float4 a1 = overwrite ? make_float4(0, 0, 0, 0) : a[1];
            a0.x += sum[0]; a0.y += sum[1]; a0.z += sum[2]; a0.w += sum[3];
            a1.x += sum[4]; a1.y += sum[5]; a1.z += sum[6]; a1.w += sum[7];
            a[0] = a0;
            a[1] = a1;
            ss += a0.x * a0.x + a0.y * a0.y + a0.z * a0.z + a0.w * a0.w + a1.x * a1.x + a1.y * a1.y + a1.z * a1.z + a1.w * a1.w;
        } else {
            float pm[8], mm[8], vv[8];
            *reinterpret_cast<float4*>(&pm[0]) = reinterpret_cast<const float4*>(master)[2 * i];
            *reinterpret_cast<float4*>(&pm[4]) = reinterpret_cast<const float4*>(master)[2 * i + 1];
            *reinterpret_cast<float4*>(&mm[0]) = reinterpret_cast<const float4*>(m)[2 * i];
            *reinterpret_cast<float4*>(&mm[4]) = reinterpret_cast<const float4*>(m)[2 * i + 1];
            *reinterpret_cast<float4*>(&vv[0]) = reinterpret_cast<const float4*>(v)[2 * i];
            *reinterpret_cast<float4*>(&vv[4]) = reinterpret_cast<const float4*>(v)[2 * i + 1];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float g = sum[j];
                ss += g * g;
                mm[j] = beta1 * mm[j] + (1.f - beta1) * g;
                vv[j] = beta2 * vv[j] + (1.f - beta2) * g * g;
                pm[j] = pm[j] * (1.f - lr * wd) - lr * (mm[j] * inv_bc1) / (sqrtf(vv[j]) * inv_sqrt_bc2 + eps);
            }
            reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(&pm[0]);
            reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(&pm[4]);
            reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(&mm[0]);
            reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(&mm[4]);
            reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(&vv[0]);
            reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(&vv[4]);
            if (out_lp) reinterpret_cast<bf16x8*>(out_lp)[i] = pack8(pm);
        }
    }
    if (sumsq_partial) {
        ss = block_sum(ss, scratch);
        if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = ss;
    }
}

// in-switch reduction: one multimem.ld_reduce per 16 bytes returns the sum over all ranks (fp32 accumulation)
__global__ void __launch_bounds__(256) nvls_reduce_scatter_kernel(const bf16* __restrict__ mc_slice, int64_t n,
                                                                  float scale, float* __restrict__ acc, int overwrite,
                                                                  float* __restrict__ sumsq_partial) {
    __shared__ float scratch[32];
    const int64_t nvec = n >> 3;
    float ss = 0.f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        uint32_t r0, r1, r2, r3;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                     : "l"(mc_slice + i * 8)
                     : "memory");
        bf16x8 pk;
        *reinterpret_cast<uint4*>(&pk) = make_uint4(r0, r1, r2, r3);
        float f[8];
        unpack8(pk, f);
        float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
        float4 a0 = overwrite ? make_float4(0, 0, 0, 0) : a[0];
        float4 a1 = overwrite ? make_float4(0, 0, 0, 0) : a[1];
        a0.x += scale * f[0]; a0.y += scale * f[1]; a0.z += scale * f[2]; a0.w += scale * f[3];
        a1.x += scale * f[4]; a1.y += scale * f[5]; a1.z += scale * f[6]; a1.w += scale * f[7];
        a[0] = a0;
        a[1] = a1;
        ss += a0.x * a0.x + a0.y * a0.y + a0.z * a0.z + a0.w * a0.w + a1.x * a1.x + a1.y * a1.y + a1.z * a1.z + a1.w * a1.w;
    }
    if (sumsq_partial) {
        ss = block_sum(ss, scratch);
        if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = ss;
    }
}

// ------------------------------------------------------------------------------------------- Ulysses exchanges
// seq -> head: x [S_loc, H, D] (local tokens, all heads) ; destination on rank o = head / (H / P):
//   y_o [P * S_loc, H / P, D] at row rank * S_loc + s, head h % (H / P).   One CTA per (token, destination).
__global__ void __launch_bounds__(128) p2p_seq_to_head_kernel(const bf16* __restrict__ x, PeerTable dst, int S_loc,
                                                              int H, int D, int rank, int P) {
    const int s = blockIdx.x, o = blockIdx.y;
    const int Hl = H / P;
    const int vec_per_tok = Hl * D / 8;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + ((int64_t)s * H + (int64_t)o * Hl) * D);
    bf16x8* out = reinterpret_cast<bf16x8*>(reinterpret_cast<bf16*>(dst.ptr[o]) + ((int64_t)rank * S_loc + s) * Hl * D);
    for (int i = threadIdx.x; i < vec_per_tok; i += blockDim.x) out[i] = src[i];
}

// head -> seq: y [P * S_loc, Hl, D] (all tokens, my heads) ; destination on rank o (owner of sequence chunk o):
//   x_o [S_loc, H, D] at row s, heads rank * Hl ...
__global__ void __launch_bounds__(128) p2p_head_to_seq_kernel(const bf16* __restrict__ y, PeerTable dst, int S_loc,
                                                              int H, int D, int rank, int P) {
    const int s = blockIdx.x, o = blockIdx.y;
    const int Hl = H / P;
    const int vec_per_tok = Hl * D / 8;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(y + ((int64_t)o * S_loc + s) * Hl * D);
    bf16x8* out = reinterpret_cast<bf16x8*>(reinterpret_cast<bf16*>(dst.ptr[o]) + ((int64_t)s * H + (int64_t)rank * Hl) * D);
    for (int i = threadIdx.x; i < vec_per_tok; i += blockDim.x) out[i] = src[i];
}

// Fused Q/K/V exchange.  Source: this rank's tokens, all heads (q [S_loc, Hq, D], k / v [S_loc, Hkv, D], each with its
// own token stride, so views of one fused projection output are fine).  Destination on rank o: one fused buffer
// [P * S_loc, Hlq + 2 * Hlkv, D] (its q heads, then its k heads, then its v heads) at row rank * S_loc + s.  With
// fewer KV heads than ranks (rep = P / Hkv > 1) KV head h goes to the rep ranks h * rep ... and Hlkv = 1.
__global__ void __launch_bounds__(128) p2p_qkv_push_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                           const bf16* __restrict__ v, int64_t q_stride, int64_t k_stride,
                                                           int64_t v_stride, PeerTable dst, int S_loc, int Hq, int Hkv,
                                                           int D, int rank, int P) {
    const int s = blockIdx.x, o = blockIdx.y;
    const int Hlq = Hq / P;
    const int rep = Hkv >= P ? 1 : P / Hkv;
    const int Hlkv = Hkv >= P ? Hkv / P : 1;
    const int kv_head0 = Hkv >= P ? o * Hlkv : o / rep;
    const int W = (Hlq + 2 * Hlkv) * D;
    bf16* drow = reinterpret_cast<bf16*>(dst.ptr[o]) + ((int64_t)rank * S_loc + s) * W;
    const int nq = Hlq * D / 8, nkv = Hlkv * D / 8;
    const bf16x8* sq = reinterpret_cast<const bf16x8*>(q + s * q_stride + (int64_t)o * Hlq * D);
    const bf16x8* sk = reinterpret_cast<const bf16x8*>(k + s * k_stride + (int64_t)kv_head0 * D);
    const bf16x8* sv = reinterpret_cast<const bf16x8*>(v + s * v_stride + (int64_t)kv_head0 * D);
    bf16x8* dq = reinterpret_cast<bf16x8*>(drow);
    bf16x8* dk = reinterpret_cast<bf16x8*>(drow + Hlq * D);
    bf16x8* dv = reinterpret_cast<bf16x8*>(drow + (Hlq + Hlkv) * D);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) dq[i] = sq[i];
    for (int i = threadIdx.x; i < nkv; i += blockDim.x) dk[i] = sk[i];
    for (int i = threadIdx.x; i < nkv; i += blockDim.x) dv[i] = sv[i];
}

// Backward of the exchange above: every rank holds d(fused buffer) [P * S_loc, Hlq + 2 * Hlkv, D] in a symmetric
// buffer; the owner of a sequence chunk pulls its rows from every peer into out [S_loc, Hq + 2 * Hkv, D] and adds
// the replicas of a replicated KV head in fp32.
__global__ void __launch_bounds__(128) p2p_qkv_grad_pull_kernel(PeerTable src, bf16* __restrict__ out, int S_loc, int Hq,
                                                                int Hkv, int D, int rank, int P) {
    const int s = blockIdx.x, o = blockIdx.y;
    const int Hlq = Hq / P;
    const int rep = Hkv >= P ? 1 : P / Hkv;
    const int Hlkv = Hkv >= P ? Hkv / P : 1;
    const int W = (Hlq + 2 * Hlkv) * D;
    const int64_t row = (int64_t)rank * S_loc + s;
    bf16* orow = out + (int64_t)s * (Hq + 2 * Hkv) * D;
    const bf16* srow = reinterpret_cast<const bf16*>(src.ptr[o]) + row * W;
    const int nq = Hlq * D / 8, nkv = Hlkv * D / 8;
    {
        const bf16x8* a = reinterpret_cast<const bf16x8*>(srow);
        bf16x8* b = reinterpret_cast<bf16x8*>(orow + (int64_t)o * Hlq * D);
        for (int i = threadIdx.x; i < nq; i += blockDim.x) b[i] = a[i];
    }
    if (rep == 1) {
        const bf16x8* ak = reinterpret_cast<const bf16x8*>(srow + Hlq * D);
        const bf16x8* av = reinterpret_cast<const bf16x8*>(srow + (Hlq + Hlkv) * D);
        bf16x8* bk = reinterpret_cast<bf16x8*>(orow + (int64_t)(Hq + o * Hlkv) * D);
        bf16x8* bv = reinterpret_cast<bf16x8*>(orow + (int64_t)(Hq + Hkv + o * Hlkv) * D);
        for (int i = threadIdx.x; i < nkv; i += blockDim.x) { bk[i] = ak[i]; bv[i] = av[i]; }
    } else if (o % rep == 0) {
        const int head = o / rep;
        bf16x8* bk = reinterpret_cast<bf16x8*>(orow + (int64_t)(Hq + head) * D);
        bf16x8* bv = reinterpret_cast<bf16x8*>(orow + (int64_t)(Hq + Hkv + head) * D);
        for (int i = threadIdx.x; i < nkv; i += blockDim.x) {
            float sk[8] = {0, 0, 0, 0, 0, 0, 0, 0}, sv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j = 0; j < rep; ++j) {
                const bf16* prow = reinterpret_cast<const bf16*>(src.ptr[o + j]) + row * W;
                float f[8];
                unpack8(reinterpret_cast<const bf16x8*>(prow + Hlq * D)[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) sk[e] += f[e];
                unpack8(reinterpret_cast<const bf16x8*>(prow + (Hlq + 1) * D)[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) sv[e] += f[e];
            }
            bk[i] = pack8(sk);
            bv[i] = pack8(sv);
        }
    }
}

// ------------------------------------------------------------------------------------------- MoE exchanges
// dispatch: token t's k-th copy goes to expert e = experts[t, k], owned by rank e / El.  Its row in the owner's
// expert-major buffer is dest_row[t, k] (computed from the all-gathered counts, see moe_dest_rows_kernel).  With
// `pair_scale` the copy is multiplied by pair_scale[t, k] (the backward pass sends score * d_out this way).  A
// destination row beyond `capacity` is not written; the error word records it.
__global__ void __launch_bounds__(256) p2p_moe_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ experts,
                                                               const int* __restrict__ dest_row,
                                                               const float* __restrict__ pair_scale, PeerTable dst, int H,
                                                               int K, int El, int capacity, int* error_flag) {
    const int64_t t = blockIdx.x;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + t * H);
    const int nvec = H >> 3;
    for (int k = 0; k < K; ++k) {
        const int owner = experts[t * K + k] / El;
        const int row = dest_row[t * K + k];
        if (row < 0 || row >= capacity) {
            if (threadIdx.x == 0) atomicCAS(error_flag, 0, (0x31 << 8) | (owner + 1));
            continue;
        }
        bf16x8* out = reinterpret_cast<bf16x8*>(reinterpret_cast<bf16*>(dst.ptr[owner]) + (int64_t)row * H);
        if (pair_scale == nullptr) {
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) out[i] = src[i];
        } else {
            const float sc = pair_scale[t * K + k];
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
                float f[8];
                unpack8(src[i], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] *= sc;
                out[i] = pack8(f);
            }
        }
    }
}

// combine: the source rank pulls the expert outputs of its (token, k) pairs from the owners and reduces them:
//   out[t] = sum_k score[t, k] * y_owner[dest_row[t, k]]        (score = 1 without `scores`)
// `pair_dot` (optional, with `dout`): pair_dot[t, k] = < dout[t], y_owner[dest_row[t, k]] >, the gradient of the score.
__global__ void __launch_bounds__(256) p2p_moe_combine_kernel(PeerTable y, const int* __restrict__ experts,
                                                              const int* __restrict__ dest_row,
                                                              const float* __restrict__ scores, bf16* __restrict__ out,
                                                              const bf16* __restrict__ dout, float* __restrict__ pair_dot,
                                                              int H, int K, int El, int capacity) {
    __shared__ float scratch[32];
    const int64_t t = blockIdx.x;
    const int nvec = H >> 3;
    if (pair_dot != nullptr) {
        for (int k = 0; k < K; ++k) {
            const int owner = experts[t * K + k] / El;
            const int row = dest_row[t * K + k];
            float acc = 0.f;
            if (row >= 0 && row < capacity) {
                const bf16x8* yr = reinterpret_cast<const bf16x8*>(reinterpret_cast<const bf16*>(y.ptr[owner]) + (int64_t)row * H);
                for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
                    float a[8], b[8];
                    unpack8(yr[i], a);
                    unpack8(reinterpret_cast<const bf16x8*>(dout + t * H)[i], b);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc += a[j] * b[j];
                }
            }
            acc = block_sum(acc, scratch);
            if (threadIdx.x == 0) pair_dot[t * K + k] = acc;
            __syncthreads();
        }
        return;
    }
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < K; ++k) {
            const int owner = experts[t * K + k] / El;
            const int row = dest_row[t * K + k];
            if (row < 0 || row >= capacity) continue;
            const float s = scores ? scores[t * K + k] : 1.f;
            float f[8];
            unpack8(reinterpret_cast<const bf16x8*>(reinterpret_cast<const bf16*>(y.ptr[owner]) + (int64_t)row * H)[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += s * f[j];
        }
        reinterpret_cast<bf16x8*>(out + t * H)[i] = pack8(acc);
    }
}

// From the counts of every source rank (all_counts [P, E]) derive, for this rank's pairs, the row inside the owner's
// buffer: segment start of the expert on its owner (segments padded to `align` rows) + pairs of lower ranks for that
// expert + rank of the pair among this rank's pairs of that expert (local_slot - local_offset).  Also emits the
// owner-side segment offsets of this rank's own experts.
__global__ void moe_dest_rows_kernel(const int* __restrict__ all_counts, const int* __restrict__ experts,
                                     const int* __restrict__ local_slots, const int* __restrict__ local_offsets,
                                     int* __restrict__ dest_row, int* __restrict__ my_segment_offsets, int64_t n_pairs,
                                     int P, int E, int El, int rank, int align) {
    extern __shared__ int sh[];  // [E] base row of (this rank's pairs of expert e) on its owner
    int* base = sh;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int owner = e / El, first = owner * El;
        int seg = 0;
        for (int f = first; f < e; ++f) {
            int tot = 0;
            for (int s = 0; s < P; ++s) tot += all_counts[s * E + f];
            seg += (tot + align - 1) / align * align;
        }
        int before = 0;
        for (int s = 0; s < rank; ++s) before += all_counts[s * E + e];
        base[e] = seg + before;
        if (owner == rank && blockIdx.x == 0) {
            my_segment_offsets[e - first] = seg;
            if (e == first + El - 1) {
                int tot = 0;
                for (int s = 0; s < P; ++s) tot += all_counts[s * E + e];
                my_segment_offsets[El] = seg + (tot + align - 1) / align * align;
            }
        }
    }
    __syncthreads();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int e = experts[i];
        dest_row[i] = base[e] + (local_slots[i] - local_offsets[e]);
    }
}

// ------------------------------------------------------------------------------------------- host wrappers
static int grid_for_bytes(int64_t nvec, int threads, int max_waves = 8) {
    return (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(nvec, threads), (int64_t)kNumSMs * max_waves));
}

// CTAs of the bulk copy / reduction kernels that run beside the compute stream (parameter gathers, gradient
// reductions).  They share the SMs with persistent GEMM CTAs: enough of them to fill the NVLink ports, few enough to
// leave the issue slots and memory pipes to the math.  ATB200_COMM_CTAS lowers the default (4 per SM, the largest value
// these kernels have been run with; larger requests are clamped to it).
static int comm_cta_cap() {
    static const int cap = [] {
        const char* e = std::getenv("ATB200_COMM_CTAS");
        const int v = e ? std::atoi(e) : 0;
        return v > 0 ? std::min(v, kNumSMs * 4) : kNumSMs * 4;
    }();
    return cap;
}

void p2p_barrier(const at::Tensor& flag_ptrs, int64_t rank, int64_t slot, int64_t epoch, double timeout_s,
                 const at::Tensor& like) {
    const int P = (int)flag_ptrs.numel();
    TORCH_CHECK(slot >= 0 && slot < 64, "barrier slot out of range");
    c10::cuda::CUDAGuard guard(like.device());
    PeerTable t = make_table(flag_ptrs, 0);
    p2p_barrier_kernel<<<1, 32, 0, current_stream()>>>(t, (int)rank, P, (int)slot, (uint32_t)epoch,
                                                       (uint64_t)(timeout_s * 1e9),
                                                       error_flag_for_comm(like.device()).data_ptr<int>());
    ATB_LAUNCH_CHECK();
}

int64_t comm_read_and_clear_error(const at::Tensor& like) {
    auto& f = error_flag_for_comm(like.device());
    const int64_t v = f.item<int>();
    if (v != 0) f.zero_();
    return v;
}

void p2p_all_gather(const at::Tensor& shard_ptrs, int64_t shard_byte_offset, at::Tensor full, int64_t shard_numel,
                    int64_t rank) {
    ATB_CHECK_CUDA(full); ATB_CHECK_CONTIG(full); ATB_CHECK_ALIGNED16(full);
    const int P = (int)shard_ptrs.numel();
    const int64_t bytes = shard_numel * full.element_size();
    TORCH_CHECK(bytes % 16 == 0 && shard_byte_offset % 16 == 0, "all_gather: shards must be multiples of 16 bytes");
    TORCH_CHECK(full.numel() >= shard_numel * P, "all_gather: output too small");
    c10::cuda::CUDAGuard guard(full.device());
    PeerTable t = make_table(shard_ptrs, shard_byte_offset);
    const int64_t vec = bytes / 16;
    dim3 grid(std::max(1, std::min(grid_for_bytes(vec, 512, 4), comm_cta_cap()) / P), P);
    p2p_all_gather_kernel<<<grid, 512, 0, current_stream()>>>(t, reinterpret_cast<uint4*>(full.data_ptr()), vec, (int)rank, P);
    ATB_LAUNCH_CHECK();
}

// grad_ptrs: base pointers of every rank's flat bf16 gradient buffer; slice [elem_offset, elem_offset + n).
at::Tensor p2p_reduce_scatter_accum(const at::Tensor& grad_ptrs, int64_t elem_offset, int64_t n, at::Tensor acc,
                                    double scale, bool overwrite, bool want_sumsq) {
    ATB_CHECK_CUDA(acc); ATB_CHECK_DTYPE(acc, at::kFloat); ATB_CHECK_CONTIG(acc); ATB_CHECK_ALIGNED16(acc);
    TORCH_CHECK(n % 8 == 0 && elem_offset % 8 == 0 && acc.numel() >= n, "reduce_scatter: n and offset must be multiples of 8");
    c10::cuda::CUDAGuard guard(acc.device());
    PeerTable t = make_table(grad_ptrs, elem_offset * 2);
    const int grid = std::min(grid_for_bytes(n / 8, 256, 4), comm_cta_cap());
    at::Tensor partial = want_sumsq ? at::empty({grid}, acc.options()) : at::Tensor();
    p2p_reduce_scatter_kernel<false><<<grid, 256, 0, current_stream()>>>(
        t, (int)grad_ptrs.numel(), n, (float)scale, acc.data_ptr<float>(), overwrite ? 1 : 0,
        want_sumsq ? partial.data_ptr<float>() : nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 1, 1);
    ATB_LAUNCH_CHECK();
    return want_sumsq ? partial.sum() : at::zeros({}, acc.options());
}

at::Tensor p2p_reduce_scatter_adamw(const at::Tensor& grad_ptrs, int64_t elem_offset, int64_t n, double scale,
                                    at::Tensor master, at::Tensor m, at::Tensor v, const c10::optional<at::Tensor>& out_lp,
                                    double lr, double beta1, double beta2, double eps, double wd, int64_t step) {
    ATB_CHECK_CUDA(master); ATB_CHECK_DTYPE(master, at::kFloat); ATB_CHECK_DTYPE(m, at::kFloat); ATB_CHECK_DTYPE(v, at::kFloat);
    ATB_CHECK_ALIGNED16(master); ATB_CHECK_ALIGNED16(m); ATB_CHECK_ALIGNED16(v);
    TORCH_CHECK(n % 8 == 0 && elem_offset % 8 == 0 && master.numel() >= n && m.numel() >= n && v.numel() >= n,
                "reduce_scatter_adamw: sizes must be multiples of 8 and cover n");
    bf16* lp = nullptr;
    if (out_lp.has_value()) {
        ATB_CHECK_DTYPE(*out_lp, at::kBFloat16); ATB_CHECK_ALIGNED16(*out_lp);
        lp = (bf16*)out_lp->data_ptr();
    }
    c10::cuda::CUDAGuard guard(master.device());
    PeerTable t = make_table(grad_ptrs, elem_offset * 2);
    const int grid = grid_for_bytes(n / 8, 256, 4);
    auto partial = at::empty({grid}, master.options());
    const float bc1 = 1.f - (float)std::pow(beta1, (double)step), bc2 = 1.f - (float)std::pow(beta2, (double)step);
    p2p_reduce_scatter_kernel<true><<<grid, 256, 0, current_stream()>>>(
        t, (int)grad_ptrs.numel(), n, (float)scale, nullptr, 0, partial.data_ptr<float>(), master.data_ptr<float>(),
        m.data_ptr<float>(), v.data_ptr<float>(), lp, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, bc1, bc2);
    ATB_LAUNCH_CHECK();
    return partial.sum();
}

at::Tensor nvls_reduce_scatter_accum(int64_t multicast_ptr, int64_t elem_offset, int64_t n, at::Tensor acc, double scale,
                                     bool overwrite, bool want_sumsq) {
    ATB_CHECK_CUDA(acc); ATB_CHECK_DTYPE(acc, at::kFloat); ATB_CHECK_ALIGNED16(acc);
    TORCH_CHECK(multicast_ptr != 0, "NVLS reduce-scatter needs a multicast mapping");
    TORCH_CHECK(n % 8 == 0 && elem_offset % 8 == 0 && acc.numel() >= n, "nvls reduce_scatter: n and offset multiples of 8");
    c10::cuda::CUDAGuard guard(acc.device());
    const int grid = grid_for_bytes(n / 8, 256, 4);
    at::Tensor partial = want_sumsq ? at::empty({grid}, acc.options()) : at::Tensor();
    nvls_reduce_scatter_kernel<<<grid, 256, 0, current_stream()>>>(
        reinterpret_cast<const bf16*>(multicast_ptr) + elem_offset, n, (float)scale, acc.data_ptr<float>(), overwrite ? 1 : 0,
        want_sumsq ? partial.data_ptr<float>() : nullptr);
    ATB_LAUNCH_CHECK();
    return want_sumsq ? partial.sum() : at::zeros({}, acc.options());
}

void p2p_seq_to_head(const at::Tensor& x, const at::Tensor& dst_ptrs, int64_t rank, bool reverse, int64_t dst_byte_offset) {
    // forward: x [S_loc, H, D] -> peers' [P * S_loc, H / P, D];  reverse: x [P * S_loc, H / P, D] -> peers' [S_loc, H, D]
    ATB_CHECK_CUDA(x); ATB_CHECK_CONTIG(x); ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_ALIGNED16(x);
    TORCH_CHECK(x.dim() == 3, "ulysses exchange: x must be [tokens, heads, head_dim]");
    const int P = (int)dst_ptrs.numel();
    const int D = (int)x.size(2);
    int S_loc, H;
    if (!reverse) { S_loc = (int)x.size(0); H = (int)x.size(1); }
    else { S_loc = (int)(x.size(0) / P); H = (int)x.size(1) * P; }
    TORCH_CHECK(H % P == 0 && ((H / P) * D) % 8 == 0, "ulysses exchange: heads must divide by the group size");
    if (S_loc == 0) return;
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(dst_byte_offset % 16 == 0, "ulysses exchange: misaligned destination offset");
    PeerTable t = make_table(dst_ptrs, dst_byte_offset);
    dim3 grid(S_loc, P);
    if (!reverse)
        p2p_seq_to_head_kernel<<<grid, 128, 0, current_stream()>>>((const bf16*)x.data_ptr(), t, S_loc, H, D, (int)rank, P);
    else
        p2p_head_to_seq_kernel<<<grid, 128, 0, current_stream()>>>((const bf16*)x.data_ptr(), t, S_loc, H, D, (int)rank, P);
    ATB_LAUNCH_CHECK();
}

static void check_qkv_heads(int Hq, int Hkv, int D, int P) {
    TORCH_CHECK(Hq % P == 0, "ulysses exchange: query heads must divide by the group size");
    TORCH_CHECK(Hkv >= P ? Hkv % P == 0 : P % Hkv == 0, "ulysses exchange: KV heads and group size must divide one another");
    TORCH_CHECK(D % 8 == 0, "ulysses exchange: head_dim must be a multiple of 8");
}

// q [S_loc, Hq, D], k / v [S_loc, Hkv, D] (dense heads, any token stride that is a multiple of 8 elements).
void p2p_qkv_push(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& dst_ptrs,
                  int64_t dst_byte_offset, int64_t rank) {
    ATB_CHECK_CUDA(q); ATB_CHECK_DTYPE(q, at::kBFloat16); ATB_CHECK_DTYPE(k, at::kBFloat16); ATB_CHECK_DTYPE(v, at::kBFloat16);
    TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "ulysses exchange: [tokens, heads, head_dim] tensors");
    const int P = (int)dst_ptrs.numel(), S_loc = (int)q.size(0), Hq = (int)q.size(1), Hkv = (int)k.size(1), D = (int)q.size(2);
    check_qkv_heads(Hq, Hkv, D, P);
    for (const at::Tensor* t : {&q, &k, &v}) {
        TORCH_CHECK(t->size(0) == S_loc && t->size(2) == D && t->stride(2) == 1 && t->stride(1) == D && t->stride(0) % 8 == 0,
                    "ulysses exchange: dense heads and a token stride that is a multiple of 8");
        TORCH_CHECK((reinterpret_cast<uintptr_t>(t->data_ptr()) & 15) == 0, "ulysses exchange: 16-byte aligned operands");
    }
    TORCH_CHECK(v.size(1) == Hkv && dst_byte_offset % 16 == 0, "ulysses exchange: inconsistent arguments");
    if (S_loc == 0) return;
    c10::cuda::CUDAGuard guard(q.device());
    PeerTable t = make_table(dst_ptrs, dst_byte_offset);
    p2p_qkv_push_kernel<<<dim3(S_loc, P), 128, 0, current_stream()>>>(
        (const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
        t, S_loc, Hq, Hkv, D, (int)rank, P);
    ATB_LAUNCH_CHECK();
}

// Returns d(qkv) [S_loc, Hq + 2 * Hkv, D] for this rank's tokens from the peers' symmetric gradient buffers.
at::Tensor p2p_qkv_grad_pull(const at::Tensor& src_ptrs, int64_t src_byte_offset, const at::Tensor& like, int64_t S_loc,
                             int64_t Hq, int64_t Hkv, int64_t D, int64_t rank) {
    ATB_CHECK_CUDA(like); ATB_CHECK_DTYPE(like, at::kBFloat16);
    const int P = (int)src_ptrs.numel();
    check_qkv_heads((int)Hq, (int)Hkv, (int)D, P);
    TORCH_CHECK(src_byte_offset % 16 == 0, "ulysses exchange: misaligned source offset");
    c10::cuda::CUDAGuard guard(like.device());
    auto out = at::empty({S_loc, Hq + 2 * Hkv, D}, like.options());
    if (S_loc == 0) return out;
    PeerTable t = make_table(src_ptrs, src_byte_offset);
    p2p_qkv_grad_pull_kernel<<<dim3((unsigned)S_loc, P), 128, 0, current_stream()>>>(t, (bf16*)out.data_ptr(), (int)S_loc, (int)Hq,
                                                                                     (int)Hkv, (int)D, (int)rank, P);
    ATB_LAUNCH_CHECK();
    return out;
}

std::tuple<at::Tensor, at::Tensor> moe_dest_rows(const at::Tensor& all_counts, const at::Tensor& experts,
                                                 const at::Tensor& local_slots, const at::Tensor& local_offsets,
                                                 int64_t rank, int64_t align) {
    ATB_CHECK_CUDA(all_counts); ATB_CHECK_DTYPE(all_counts, at::kInt); ATB_CHECK_CONTIG(all_counts);
    ATB_CHECK_DTYPE(experts, at::kInt); ATB_CHECK_CONTIG(experts); ATB_CHECK_CONTIG(local_slots); ATB_CHECK_CONTIG(local_offsets);
    const int P = (int)all_counts.size(0), E = (int)all_counts.size(1), El = E / P;
    TORCH_CHECK(E % P == 0 && E <= 1024, "moe_dest_rows: experts must divide by ranks, at most 1024 experts");
    c10::cuda::CUDAGuard guard(experts.device());
    auto dest = at::empty_like(experts);
    auto seg = at::empty({El + 1}, experts.options());
    const int64_t n = experts.numel();
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n, 256), kNumSMs));
    moe_dest_rows_kernel<<<grid, 256, E * sizeof(int), current_stream()>>>(
        all_counts.data_ptr<int>(), experts.data_ptr<int>(), local_slots.data_ptr<int>(), local_offsets.data_ptr<int>(),
        dest.data_ptr<int>(), seg.data_ptr<int>(), n, P, E, El, (int)rank, (int)align);
    ATB_LAUNCH_CHECK();
    return {dest, seg};
}

void p2p_moe_dispatch(const at::Tensor& x, const at::Tensor& experts, const at::Tensor& dest_row,
                      const at::Tensor& dst_ptrs, int64_t dst_byte_offset, int64_t experts_per_rank, int64_t capacity,
                      const c10::optional<at::Tensor>& pair_scale) {
    ATB_CHECK_CUDA(x); ATB_CHECK_CONTIG(x); ATB_CHECK_DTYPE(x, at::kBFloat16); ATB_CHECK_ALIGNED16(x);
    ATB_CHECK_DTYPE(experts, at::kInt); ATB_CHECK_DTYPE(dest_row, at::kInt); ATB_CHECK_CONTIG(experts); ATB_CHECK_CONTIG(dest_row);
    const int64_t T = x.size(0);
    const int H = (int)x.size(1), K = (int)experts.size(1);
    TORCH_CHECK(H % 8 == 0 && dst_byte_offset % 16 == 0, "moe dispatch: hidden size must be a multiple of 8");
    const float* ps = nullptr;
    if (pair_scale.has_value()) {
        ATB_CHECK_DTYPE(*pair_scale, at::kFloat); ATB_CHECK_CONTIG(*pair_scale);
        TORCH_CHECK(pair_scale->numel() == experts.numel(), "moe dispatch: one scale per (token, k) pair");
        ps = pair_scale->data_ptr<float>();
    }
    if (T == 0) return;
    c10::cuda::CUDAGuard guard(x.device());
    PeerTable t = make_table(dst_ptrs, dst_byte_offset);
    p2p_moe_dispatch_kernel<<<(unsigned)T, 256, 0, current_stream()>>>(
        (const bf16*)x.data_ptr(), experts.data_ptr<int>(), dest_row.data_ptr<int>(), ps, t, H, K, (int)experts_per_rank,
        (int)capacity, error_flag_for_comm(x.device()).data_ptr<int>());
    ATB_LAUNCH_CHECK();
}

at::Tensor p2p_moe_combine(const at::Tensor& y_ptrs, int64_t y_byte_offset, const at::Tensor& experts, const at::Tensor& dest_row,
                           const c10::optional<at::Tensor>& scores, int64_t hidden, int64_t experts_per_rank, int64_t capacity) {
    ATB_CHECK_CUDA(experts); ATB_CHECK_DTYPE(experts, at::kInt); ATB_CHECK_DTYPE(dest_row, at::kInt);
    ATB_CHECK_CONTIG(experts); ATB_CHECK_CONTIG(dest_row);
    const float* sc = nullptr;
    if (scores.has_value()) { ATB_CHECK_DTYPE(*scores, at::kFloat); ATB_CHECK_CONTIG(*scores); sc = scores->data_ptr<float>(); }
    const int64_t T = experts.size(0);
    const int K = (int)experts.size(1);
    TORCH_CHECK(hidden % 8 == 0 && y_byte_offset % 16 == 0, "moe combine: hidden size must be a multiple of 8");
    c10::cuda::CUDAGuard guard(experts.device());
    auto out = at::empty({T, hidden}, experts.options().dtype(at::kBFloat16));
    if (T == 0) return out;
    PeerTable t = make_table(y_ptrs, y_byte_offset);
    p2p_moe_combine_kernel<<<(unsigned)T, 256, 0, current_stream()>>>(t, experts.data_ptr<int>(), dest_row.data_ptr<int>(), sc,
                                                                      (bf16*)out.data_ptr(), nullptr, nullptr, (int)hidden, K,
                                                                      (int)experts_per_rank, (int)capacity);
    ATB_LAUNCH_CHECK();
    return out;
}

// pair_dot[t, k] = < dout[t], y_owner[dest_row[t, k]] > : the gradient of the combine weights.
at::Tensor p2p_moe_pair_dot(const at::Tensor& y_ptrs, int64_t y_byte_offset, const at::Tensor& experts, const at::Tensor& dest_row,
                            const at::Tensor& dout, int64_t experts_per_rank, int64_t capacity) {
    ATB_CHECK_CUDA(dout); ATB_CHECK_CONTIG(dout); ATB_CHECK_DTYPE(dout, at::kBFloat16); ATB_CHECK_ALIGNED16(dout);
    ATB_CHECK_DTYPE(experts, at::kInt); ATB_CHECK_DTYPE(dest_row, at::kInt); ATB_CHECK_CONTIG(experts); ATB_CHECK_CONTIG(dest_row);
    const int64_t T = experts.size(0);
    const int K = (int)experts.size(1);
    const int H = (int)dout.size(1);
    TORCH_CHECK(H % 8 == 0 && y_byte_offset % 16 == 0 && dout.size(0) == T, "moe pair_dot: shape mismatch");
    c10::cuda::CUDAGuard guard(dout.device());
    auto dots = at::zeros({T, K}, dout.options().dtype(at::kFloat));
    if (T == 0) return dots;
    PeerTable t = make_table(y_ptrs, y_byte_offset);
    p2p_moe_combine_kernel<<<(unsigned)T, 256, 0, current_stream()>>>(t, experts.data_ptr<int>(), dest_row.data_ptr<int>(), nullptr,
                                                                      nullptr, (const bf16*)dout.data_ptr(), dots.data_ptr<float>(),
                                                                      H, K, (int)experts_per_rank, (int)capacity);
    ATB_LAUNCH_CHECK();
    return dots;
}

}  // namespace atb
