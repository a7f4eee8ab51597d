// SPDX-License-Identifier: Apache-2.0
// Operator registration: every kernel of the library is reachable as torch.ops.atb200.<name>.
#include <ATen/ATen.h>
#include <torch/library.h>

#include <tuple>

namespace atb {
std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps);
std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w,
                                               const at::Tensor& rstd);
void rope_inplace(at::Tensor x, const at::Tensor& cosb, const at::Tensor& sinb, bool inverse);
at::Tensor swiglu_fwd(const at::Tensor& gu);
at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& gu);
std::tuple<at::Tensor, at::Tensor> swiglu_bwd_recompute(const at::Tensor& dout, const at::Tensor& gu);
void adamw_step(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                const c10::optional<at::Tensor>& out_lp, double lr, double beta1, double beta2, double eps, double wd,
                int64_t step, const c10::optional<at::Tensor>& grad_scale);
at::Tensor sumsq(const at::Tensor& x);
void accum_bf16(const at::Tensor& src, at::Tensor acc, double scale, bool overwrite);
std::tuple<at::Tensor, at::Tensor> ce_fwd_bwd(at::Tensor logits, const at::Tensor& labels,
                                              const c10::optional<at::Tensor>& grad_scale,
                                              const c10::optional<at::Tensor>& row_scale, bool write_grad);
at::Tensor kl_fwd_bwd(at::Tensor student, const at::Tensor& teacher, const c10::optional<at::Tensor>& row_weight,
                      double temperature, const c10::optional<at::Tensor>& grad_scale, bool write_grad);
at::Tensor gemm_bf16(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, int64_t epilogue,
                     const c10::optional<at::Tensor>& out, int64_t max_ctas, const c10::optional<at::Tensor>& residual);
int64_t read_and_clear_error_flag(const at::Tensor& like);
void gemm_bf16_push_heads(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dst_ptrs, int64_t dst_byte_offset,
                          int64_t rank, int64_t Hq, int64_t Hkv, int64_t D);
std::tuple<at::Tensor, at::Tensor> gemm_bf16_peer_a(const at::Tensor& a_ptrs, int64_t a_byte_offset, int64_t rows_total,
                                                    int64_t seg_cols, int64_t row0, int64_t M, const at::Tensor& b,
                                                    const c10::optional<at::Tensor>& residual, int64_t stage_ctas);
#ifdef ATB_ATTN_PROFILE
at::Tensor fmha_read_profile();
#endif
std::tuple<at::Tensor, at::Tensor> fmha_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                            const at::Tensor& cu_seqlens, int64_t max_blocks, double softmax_scale);
std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                                         const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                                         const at::Tensor& cu_seqlens, int64_t max_blocks, double softmax_scale,
                                                         bool packed);
at::Tensor fmha_bwd_read_profile(const at::Tensor& like);
at::Tensor gemm_bf16_gather_b(const at::Tensor& x, const at::Tensor& shard_ptrs, int64_t shard_byte_offset, int64_t shard_elems,
                              at::Tensor flat, int64_t w_elem_offset, int64_t N, int64_t stage_ctas);
bool set_gemm_cta_pairs(bool on);
at::Tensor gemm_bf16_grouped(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets, int64_t mode, bool b_mn,
                             int64_t epilogue, const c10::optional<at::Tensor>& out);
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_topk_gating_fwd(const at::Tensor& logits, int64_t K, bool normalize);
at::Tensor moe_topk_gating_bwd(const at::Tensor& dscores, const at::Tensor& probs, const at::Tensor& experts,
                               const c10::optional<at::Tensor>& dprobs_extra, bool normalize);
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_assign_slots(const at::Tensor& experts, int64_t E, int64_t align);
at::Tensor moe_scatter_fwd(const at::Tensor& x, const at::Tensor& slots, int64_t out_rows);
at::Tensor moe_scatter_bwd(const at::Tensor& dout, const at::Tensor& slots);
at::Tensor moe_gather_fwd(const at::Tensor& y, const at::Tensor& slots, const at::Tensor& scores);
std::tuple<at::Tensor, at::Tensor> moe_gather_bwd(const at::Tensor& dout, const at::Tensor& y, const at::Tensor& slots,
                                                  const at::Tensor& scores);
void p2p_barrier(const at::Tensor& flag_ptrs, int64_t rank, int64_t slot, int64_t epoch, double timeout_s, const at::Tensor& like);
int64_t comm_read_and_clear_error(const at::Tensor& like);
void p2p_all_gather(const at::Tensor& shard_ptrs, int64_t shard_byte_offset, at::Tensor full, int64_t shard_numel, int64_t rank);
at::Tensor p2p_reduce_scatter_accum(const at::Tensor& grad_ptrs, int64_t elem_offset, int64_t n, at::Tensor acc, double scale,
                                    bool overwrite, bool want_sumsq);
at::Tensor p2p_reduce_scatter_adamw(const at::Tensor& grad_ptrs, int64_t elem_offset, int64_t n, double scale, at::Tensor master,
                                    at::Tensor m, at::Tensor v, const c10::optional<at::Tensor>& out_lp, double lr, double beta1,
                                    double beta2, double eps, double wd, int64_t step);
at::Tensor nvls_reduce_scatter_accum(int64_t multicast_ptr, int64_t elem_offset, int64_t n, at::Tensor acc, double scale,
                                     bool overwrite, bool want_sumsq);
void p2p_seq_to_head(const at::Tensor& x, const at::Tensor& dst_ptrs, int64_t rank, bool reverse, int64_t dst_byte_offset);
void p2p_qkv_push(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& dst_ptrs,
                  int64_t dst_byte_offset, int64_t rank);
at::Tensor p2p_qkv_grad_pull(const at::Tensor& src_ptrs, int64_t src_byte_offset, const at::Tensor& like, int64_t S_loc,
                             int64_t Hq, int64_t Hkv, int64_t D, int64_t rank);
std::tuple<at::Tensor, at::Tensor> moe_dest_rows(const at::Tensor& all_counts, const at::Tensor& experts,
                                                 const at::Tensor& local_slots, const at::Tensor& local_offsets, int64_t rank,
                                                 int64_t align);
void p2p_moe_dispatch(const at::Tensor& x, const at::Tensor& experts, const at::Tensor& dest_row,
                      const at::Tensor& dst_ptrs, int64_t dst_byte_offset, int64_t experts_per_rank, int64_t capacity,
                      const c10::optional<at::Tensor>& pair_scale);
at::Tensor p2p_moe_combine(const at::Tensor& y_ptrs, int64_t y_byte_offset, const at::Tensor& experts, const at::Tensor& dest_row,
                           const c10::optional<at::Tensor>& scores, int64_t hidden, int64_t experts_per_rank, int64_t capacity);
at::Tensor p2p_moe_pair_dot(const at::Tensor& y_ptrs, int64_t y_byte_offset, const at::Tensor& experts, const at::Tensor& dest_row,
                            const at::Tensor& dout, int64_t experts_per_rank, int64_t capacity);
}  // namespace atb

TORCH_LIBRARY(atb200, m) {
    m.def("rmsnorm_fwd(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)", &atb::rmsnorm_fwd);
    m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd) -> (Tensor, Tensor)", &atb::rmsnorm_bwd);
    m.def("rope_inplace(Tensor(a!) x, Tensor cos, Tensor sin, bool inverse) -> ()", &atb::rope_inplace);
    m.def("swiglu_fwd(Tensor gu) -> Tensor", &atb::swiglu_fwd);
    m.def("swiglu_bwd(Tensor dout, Tensor gu) -> Tensor", &atb::swiglu_bwd);
    m.def("swiglu_bwd_recompute(Tensor dout, Tensor gu) -> (Tensor, Tensor)", &atb::swiglu_bwd_recompute);
    m.def(
        "adamw_step(Tensor(a!) master, Tensor grad, Tensor(b!) m, Tensor(c!) v, Tensor? out_lp, float lr, float beta1, "
        "float beta2, float eps, float wd, int step, Tensor? grad_scale) -> ()",
        &atb::adamw_step);
    m.def("sumsq(Tensor x) -> Tensor", &atb::sumsq);
    m.def("accum_bf16(Tensor src, Tensor(a!) acc, float scale, bool overwrite) -> ()", &atb::accum_bf16);
    m.def("ce_fwd_bwd(Tensor(a!) logits, Tensor labels, Tensor? grad_scale, Tensor? row_scale, bool write_grad) -> (Tensor, Tensor)",
          &atb::ce_fwd_bwd);
    m.def("kl_fwd_bwd(Tensor(a!) student, Tensor teacher, Tensor? row_weight, float temperature, Tensor? grad_scale, bool write_grad) -> Tensor",
          &atb::kl_fwd_bwd);
    m.def("gemm_bf16(Tensor a, Tensor b, bool a_mn, bool b_mn, int epilogue, Tensor? out, int max_ctas, Tensor? residual=None) -> Tensor",
          &atb::gemm_bf16);
    m.def("read_and_clear_error_flag(Tensor like) -> int", &atb::read_and_clear_error_flag);
    m.def("gemm_bf16_push_heads(Tensor x, Tensor w, Tensor dst_ptrs, int dst_byte_offset, int rank, int Hq, int Hkv, int D) -> ()", &atb::gemm_bf16_push_heads);
    m.def("gemm_bf16_peer_a(Tensor a_ptrs, int a_byte_offset, int rows_total, int seg_cols, int row0, int M, Tensor b, Tensor? residual=None, int stage_ctas=16) -> (Tensor, Tensor)", &atb::gemm_bf16_peer_a);
#ifdef ATB_ATTN_PROFILE
    m.def("fmha_read_profile() -> Tensor", &atb::fmha_read_profile);
#endif
    m.def("fmha_fwd(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens, int max_blocks, float softmax_scale) -> (Tensor, Tensor)", &atb::fmha_fwd);
    m.def("gemm_bf16_gather_b(Tensor x, Tensor shard_ptrs, int shard_byte_offset, int shard_elems, Tensor(a!) flat, "
          "int w_elem_offset, int N, int stage_ctas) -> Tensor", &atb::gemm_bf16_gather_b);
    m.def("fmha_bwd_read_profile(Tensor like) -> Tensor", &atb::fmha_bwd_read_profile);
    m.def("fmha_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, Tensor cu_seqlens, int max_blocks, float softmax_scale, bool packed=False) -> (Tensor, Tensor, Tensor)", &atb::fmha_bwd);
    m.def("set_gemm_cta_pairs(bool on) -> bool", &atb::set_gemm_cta_pairs);
    m.def("p2p_barrier(Tensor flag_ptrs, int rank, int slot, int epoch, float timeout_s, Tensor like) -> ()", &atb::p2p_barrier);
    m.def("comm_read_and_clear_error(Tensor like) -> int", &atb::comm_read_and_clear_error);
    m.def("p2p_all_gather(Tensor shard_ptrs, int shard_byte_offset, Tensor(a!) full, int shard_numel, int rank) -> ()",
          &atb::p2p_all_gather);
    m.def("p2p_reduce_scatter_accum(Tensor grad_ptrs, int elem_offset, int n, Tensor(a!) acc, float scale, bool overwrite, "
          "bool want_sumsq) -> Tensor", &atb::p2p_reduce_scatter_accum);
    m.def("p2p_reduce_scatter_adamw(Tensor grad_ptrs, int elem_offset, int n, float scale, Tensor(a!) master, Tensor(b!) m, "
          "Tensor(c!) v, Tensor? out_lp, float lr, float beta1, float beta2, float eps, float wd, int step) -> Tensor",
          &atb::p2p_reduce_scatter_adamw);
    m.def("nvls_reduce_scatter_accum(int multicast_ptr, int elem_offset, int n, Tensor(a!) acc, float scale, bool overwrite, "
          "bool want_sumsq) -> Tensor", &atb::nvls_reduce_scatter_accum);
    m.def("p2p_seq_to_head(Tensor x, Tensor dst_ptrs, int rank, bool reverse, int dst_byte_offset=0) -> ()", &atb::p2p_seq_to_head);
    m.def("p2p_qkv_push(Tensor q, Tensor k, Tensor v, Tensor dst_ptrs, int dst_byte_offset, int rank) -> ()", &atb::p2p_qkv_push);
    m.def("p2p_qkv_grad_pull(Tensor src_ptrs, int src_byte_offset, Tensor like, int S_loc, int Hq, int Hkv, int D, int rank) -> Tensor", &atb::p2p_qkv_grad_pull);
    m.def("moe_dest_rows(Tensor all_counts, Tensor experts, Tensor local_slots, Tensor local_offsets, int rank, int align) -> "
          "(Tensor, Tensor)", &atb::moe_dest_rows);
    m.def("p2p_moe_dispatch(Tensor x, Tensor experts, Tensor dest_row, Tensor dst_ptrs, int dst_byte_offset, int experts_per_rank, int capacity, Tensor? pair_scale=None) -> ()", &atb::p2p_moe_dispatch);
    m.def("p2p_moe_combine(Tensor y_ptrs, int y_byte_offset, Tensor experts, Tensor dest_row, Tensor? scores, int hidden, int experts_per_rank, int capacity) -> Tensor", &atb::p2p_moe_combine);
    m.def("p2p_moe_pair_dot(Tensor y_ptrs, int y_byte_offset, Tensor experts, Tensor dest_row, Tensor dout, int experts_per_rank, int capacity) -> Tensor", &atb::p2p_moe_pair_dot);
    m.def("gemm_bf16_grouped(Tensor a, Tensor b, Tensor offsets, int mode, bool b_mn, int epilogue, Tensor? out) -> Tensor",
          &atb::gemm_bf16_grouped);
    m.def("moe_topk_gating_fwd(Tensor logits, int K, bool normalize) -> (Tensor, Tensor, Tensor)", &atb::moe_topk_gating_fwd);
    m.def("moe_topk_gating_bwd(Tensor dscores, Tensor probs, Tensor experts, Tensor? dprobs_extra, bool normalize) -> Tensor",
          &atb::moe_topk_gating_bwd);
    m.def("moe_assign_slots(Tensor experts, int E, int align) -> (Tensor, Tensor, Tensor)", &atb::moe_assign_slots);
    m.def("moe_scatter_fwd(Tensor x, Tensor slots, int out_rows) -> Tensor", &atb::moe_scatter_fwd);
    m.def("moe_scatter_bwd(Tensor dout, Tensor slots) -> Tensor", &atb::moe_scatter_bwd);
    m.def("moe_gather_fwd(Tensor y, Tensor slots, Tensor scores) -> Tensor", &atb::moe_gather_fwd);
    m.def("moe_gather_bwd(Tensor dout, Tensor y, Tensor slots, Tensor scores) -> (Tensor, Tensor)", &atb::moe_gather_bwd);
}
