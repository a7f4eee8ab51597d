# SPDX-License-Identifier: Apache-2.0
"""ArcticMoE: a mixture-of-experts feed-forward block with expert parallelism.

Behaviour parity: arctic_training/model/moe/moe.py:33-509 — softmax-then-top-k routing with optional
renormalisation, load-balancing loss applied as an analytic gradient on the router probabilities
(``grad += freq * loss_coeff / tokens / ep_size``), expert-major token permutation, variable-split
all-to-all over the expert-parallel group, grouped gate/up GEMM -> SwiGLU -> grouped down GEMM, the inverse
exchange and a score-weighted combine; optional sigmoid-gated shared expert; routing replay.

Differences by design: slot assignment is deterministic (no atomics), expert segments are padded to
128-row tiles instead of a globally all-reduced capacity, weights are stored ``[experts, out, in]`` with
gate/up rows block-interleaved so the grouped GEMM can apply SwiGLU in its epilogue, and token counts stay
on the device except for the one exchange of split sizes that the NCCL baseline path needs.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..models.arch import ArchConfig
from ..ops import reference as ref
from . import ops as mops
from .alltoall import all_to_all_v
from .grouped import grouped_mlp

SEGMENT_ALIGN = 128

# Expert-parallel layout with which MoE blocks are built while a model is being constructed (set by the model factory
# from the trainer's process groups), so that every rank allocates only its own experts from the start.
_BUILD_LAYOUT = {"ep_size": 1, "ep_rank": 0, "ep_group": None}


class expert_parallel_layout:
    """``with expert_parallel_layout(size, rank, group): model = CausalLM(cfg)`` builds every MoE block of the model
    with ``num_experts / size`` local experts (the reference creates its blocks on the meta device and fills in the
    local experts only, arctic_training/model/moe/utils.py:76-200)."""

    def __init__(self, ep_size: int, ep_rank: int, ep_group: Any) -> None:
        self.new = {"ep_size": int(ep_size), "ep_rank": int(ep_rank), "ep_group": ep_group}

    def __enter__(self):
        self.old = dict(_BUILD_LAYOUT)
        _BUILD_LAYOUT.update(self.new)
        return self

    def __exit__(self, *exc):
        _BUILD_LAYOUT.update(self.old)
        return False


@dataclass
class MoEConfig:
    model_dim: int
    intermediate_dim: int
    num_experts: int
    top_k: int
    normalize_topk_scores: bool = True
    loss_coeff: float = 0.01
    act_fn: str = "silu"  # "silu", or "silu_alpha" = x * sigmoid(1.702 x) (the gated activation of gpt-oss)
    is_gated: bool = True
    use_shared_expert: bool = False
    shared_intermediate_dim: int = 0
    shared_expert_gated: bool = True
    """ Qwen2-MoE multiplies the shared expert by a sigmoid gate of the token; DeepSeek adds it as it is. """
    routed_scaling_factor: float = 1.0
    """ Factor on the routed experts' scores (DeepSeek). """
    n_group: int = 1
    topk_group: int = 1
    """ Group-limited routing (DeepSeek): the experts form ``n_group`` groups, a token may only use experts of its
    ``topk_group`` best groups (a group's score is its best expert's probability). """
    ep_size: int = 1
    ep_rank: int = 0
    ep_group: Any = None
    input_dtype: torch.dtype = torch.bfloat16
    return_router_scores: bool = False
    use_fused_kernels: bool = True
    enable_routing_replay: bool = False


class ArcticMoE(nn.Module):
    def __init__(self, config: MoEConfig, dtype=None, device=None) -> None:
        super().__init__()
        c = self._config = config
        assert c.num_experts % c.ep_size == 0, "num_experts must be divisible by the expert-parallel size"
        self.num_experts, self.top_k = c.num_experts, c.top_k
        self.ep_size, self.ep_rank, self.ep_group = c.ep_size, c.ep_rank, c.ep_group
        self.num_local_experts = c.num_experts // c.ep_size
        H, I, El = c.model_dim, c.intermediate_dim, self.num_local_experts
        self.router_gate = nn.Parameter(torch.empty(c.num_experts, H, dtype=dtype, device=device))
        self.expert_gate_up = nn.Parameter(torch.empty(El, 2 * I, H, dtype=dtype, device=device))
        self.expert_down = nn.Parameter(torch.empty(El, H, I, dtype=dtype, device=device))
        for p in (self.expert_gate_up, self.expert_down):
            p.is_expert_param = True
            p._first_expert = c.ep_rank * El     # global index of this rank's first expert
            p._num_experts = c.num_experts
        if c.use_shared_expert:
            Is = c.shared_intermediate_dim or I
            self.shared_expert_gate_up = nn.Parameter(torch.empty(2 * Is, H, dtype=dtype, device=device))
            self.shared_expert_down = nn.Parameter(torch.empty(H, Is, dtype=dtype, device=device))
            if c.shared_expert_gated:
                self.shared_expert_output_gate = nn.Parameter(torch.empty(1, H, dtype=dtype, device=device))
        from .timers import StageTimers

        self.timers = StageTimers()
        self.replay_assignments: Optional[torch.Tensor] = None
        self.recorded_assignments: Optional[torch.Tensor] = None
        self.last_expert_counts: Optional[torch.Tensor] = None
        self.pending_aux_loss = None

    @property
    def local_expert_indices(self) -> range:
        return range(self.ep_rank * self.num_local_experts, (self.ep_rank + 1) * self.num_local_experts)

    # ------------------------------------------------------------------ routing
    def route(self, x: torch.Tensor):
        c = self._config
        logits = F.linear(x, self.router_gate).float()
        T = x.shape[0]
        if c.enable_routing_replay and self.replay_assignments is not None:
            experts = self.replay_assignments.to(torch.int32)
            probs = torch.softmax(logits, dim=-1)
            scores = torch.gather(probs, 1, experts.long())
            if c.normalize_topk_scores:
                scores = scores / scores.sum(-1, keepdim=True)
            lb = None
        else:
            # load-balancing term: d(sum_e mean_t(p_te) * freq_e)/dp = freq / T, with freq taken from this routing
            # inside the gating op (one top-k pass)
            coeff = 0.0
            if self.training and c.loss_coeff > 0 and torch.is_grad_enabled():
                coeff = c.loss_coeff / T / self.ep_size
            if c.n_group > 1 and c.topk_group < c.n_group:
                scores, experts = self._route_group_limited(logits, coeff)
            else:
                scores, experts, probs = mops.topk_gating(logits, self.top_k, c.normalize_topk_scores, None, coeff)
        if c.routed_scaling_factor != 1.0:
            scores = scores * c.routed_scaling_factor
        if c.enable_routing_replay:
            self.recorded_assignments = experts.detach()
        return scores, experts

    def _route_group_limited(self, logits: torch.Tensor, lb_coeff: float):
        """Softmax over all experts, keep the ``topk_group`` groups whose best expert scores highest, top-k among the
        experts of those groups.  Scores stay the full-softmax probabilities (no renormalisation over the groups)."""
        c = self._config
        T, E = logits.shape
        probs = torch.softmax(logits, dim=-1)
        group_best = probs.detach().view(T, c.n_group, E // c.n_group).max(-1).values
        keep = torch.zeros_like(group_best, dtype=torch.bool).scatter_(
            1, torch.topk(group_best, c.topk_group, dim=-1, sorted=False).indices, True)
        allowed = keep.unsqueeze(-1).expand(T, c.n_group, E // c.n_group).reshape(T, E)
        masked = probs.detach().masked_fill(~allowed, 0.0)
        experts = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, : self.top_k]
        if lb_coeff and probs.requires_grad:
            lb = mops._load_balance_grad(experts, E, lb_coeff)
            probs.register_hook(lambda g: g + lb.unsqueeze(0))
        scores = torch.gather(probs, 1, experts)
        if c.normalize_topk_scores:
            scores = scores / scores.sum(-1, keepdim=True)
        return scores, experts.to(torch.int32)

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states: torch.Tensor, *_: Any) -> torch.Tensor:
        shp = hidden_states.shape
        x = hidden_states.reshape(-1, shp[-1])
        T = x.shape[0]
        tm, gpu = self.timers, x.is_cuda
        tm.start("amoe e2e", gpu)
        tm.start("router", gpu)
        scores, experts = self.route(x)
        tm.stop("router", gpu)
        if self.ep_size == 1:
            tm.start("dispatch", gpu)
            slots, counts, offsets = mops.assign_slots(experts, self.num_experts, SEGMENT_ALIGN)
            rows = T * self.top_k + self.num_experts * (SEGMENT_ALIGN - 1)
            rows = (rows + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
            permuted = mops.scatter_rows(x, slots, rows)
            tm.stop("dispatch", gpu)
            tm.start("experts", gpu)
            y = grouped_mlp(permuted, offsets, self.expert_gate_up, self.expert_down, self._config.act_fn)
            tm.stop("experts", gpu)
            tm.start("combine", gpu)
            out = mops.gather_rows(y, slots, scores)
            tm.stop("combine", gpu)
        else:
            out = self._forward_ep(x, scores, experts)
        self.last_expert_counts = None
        if self._config.use_shared_expert:
            tm.start("shared-expert", gpu)
            sh = F.linear(ops.swiglu_interleaved(F.linear(x, self.shared_expert_gate_up)), self.shared_expert_down)
            if self._config.shared_expert_gated:
                sh = torch.sigmoid(F.linear(x, self.shared_expert_output_gate)) * sh
            out = out + sh
            tm.stop("shared-expert", gpu)
        tm.stop("amoe e2e", gpu)
        return out.view(shp)

    def _forward_ep(self, x: torch.Tensor, scores: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
        """Expert parallel path over NCCL: send buffer is (destination rank, local expert)-major, i.e. plain
        global-expert-major; the receiver regroups rank-major chunks into expert-major tile-aligned segments."""
        P, El, K = self.ep_size, self.num_local_experts, self.top_k
        T = x.shape[0]
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and self.num_experts <= 1024:
            from .peer import exchange_for
            from .peer import peer_expert_forward

            ex = exchange_for(self.ep_group)
            if ex is not None:
                tm = self.timers

                def run_experts(tokens, seg):
                    # the dispatch ends and the combine starts where the local experts run
                    tm.stop("dispatch", True)
                    tm.start("experts", True)
                    y = grouped_mlp(tokens, seg, self.expert_gate_up, self.expert_down, self._config.act_fn)
                    tm.stop("experts", True)
                    tm.start("combine", True)
                    return y

                tm.start("dispatch", True)
                out = peer_expert_forward(x, scores, experts, self.num_experts, ex, SEGMENT_ALIGN, run_experts).to(x.dtype)
                tm.stop("combine", True)
                return out
        slots, counts, _ = mops.assign_slots(experts, self.num_experts, 1)
        send = mops.scatter_rows(x, slots, T * K)
        # counts[src][e] for my local experts from every source rank
        gathered = [torch.empty_like(counts) for _ in range(P)]
        dist.all_gather(gathered, counts, group=self.ep_group)
        # [P * El]: (source rank, my local expert)
        recv_counts = torch.stack(gathered)[:, self.ep_rank * El : (self.ep_rank + 1) * El].reshape(-1).contiguous()
        send_splits = counts.view(P, El).sum(1)
        recv_splits = recv_counts.view(P, El).sum(1)
        splits = torch.stack([send_splits, recv_splits]).tolist()  # the one host sync of the baseline path
        self.timers.record_token_counts(splits[1], splits[0])
        recv = all_to_all_v(send, splits[0], splits[1], self.ep_group)
        # regroup: received rows are ordered (src, expert); build expert-major aligned slots for them
        n_recv = recv.shape[0]
        src_expert = torch.repeat_interleave(
            torch.arange(P * El, device=x.device, dtype=torch.int32) % El, recv_counts.long(), output_size=n_recv
        )
        r_slots, r_counts, r_offsets = mops.assign_slots(src_expert.view(-1, 1), El, SEGMENT_ALIGN)
        rows = n_recv + El * (SEGMENT_ALIGN - 1)
        rows = max(SEGMENT_ALIGN, (rows + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN)
        permuted = mops.scatter_rows(recv, r_slots, rows)
        y = grouped_mlp(permuted, r_offsets, self.expert_gate_up, self.expert_down)
        ones = torch.ones(n_recv, 1, dtype=torch.float32, device=x.device)
        back = mops.gather_rows(y, r_slots, ones)  # undo the regrouping (one source row per received row)
        returned = all_to_all_v(back, splits[1], splits[0], self.ep_group)
        return mops.gather_rows(returned, slots, scores)


def build_moe_block(cfg: ArchConfig, dtype=None, device=None, ep_size: Optional[int] = None, ep_rank: Optional[int] = None,
                    ep_group=None) -> ArcticMoE:
    """ArcticMoE configured from a Hugging Face style architecture dict (Qwen3-MoE naming).  Without explicit
    arguments the expert-parallel layout is the one of the enclosing :class:`expert_parallel_layout` block."""
    if ep_size is None:
        ep_size, ep_rank, ep_group = _BUILD_LAYOUT["ep_size"], _BUILD_LAYOUT["ep_rank"], _BUILD_LAYOUT["ep_group"]
    if cfg.get("n_routed_experts"):  # DeepSeek naming
        moe_i = int(cfg["moe_intermediate_size"])
        group_limited = cfg.get("topk_method") == "group_limited_greedy" and (cfg.get("n_group") or 1) > 1
        mc = MoEConfig(
            model_dim=cfg["hidden_size"], intermediate_dim=moe_i, num_experts=int(cfg["n_routed_experts"]),
            top_k=int(cfg.get("num_experts_per_tok") or 1), normalize_topk_scores=bool(cfg.get("norm_topk_prob", False)),
            loss_coeff=float(cfg.get("aux_loss_alpha", 0.001) or 0.0),
            use_shared_expert=bool(cfg.get("n_shared_experts")), shared_expert_gated=False,
            shared_intermediate_dim=moe_i * int(cfg.get("n_shared_experts") or 0),
            routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0) or 1.0),
            n_group=int(cfg.get("n_group") or 1) if group_limited else 1,
            topk_group=int(cfg.get("topk_group") or 1) if group_limited else 1,
            ep_size=ep_size, ep_rank=ep_rank, ep_group=ep_group, input_dtype=dtype or torch.bfloat16,
        )
        return ArcticMoE(mc, dtype=dtype, device=device)
    mc = MoEConfig(
        model_dim=cfg["hidden_size"],
        intermediate_dim=cfg.get("moe_intermediate_size") or cfg["intermediate_size"],
        num_experts=cfg.get("num_experts") or cfg.get("num_local_experts"),
        top_k=cfg.get("num_experts_per_tok", 2),
        normalize_topk_scores=bool(cfg.get("norm_topk_prob", True)),
        loss_coeff=float(cfg.get("router_aux_loss_coef", 0.01) or 0.0),
        act_fn="silu_alpha" if cfg.get("model_type") == "gpt_oss" else "silu",
        use_shared_expert=bool(cfg.get("shared_expert_intermediate_size")),
        shared_intermediate_dim=int(cfg.get("shared_expert_intermediate_size") or 0),
        ep_size=ep_size, ep_rank=ep_rank, ep_group=ep_group,
        input_dtype=dtype or torch.bfloat16,
    )
    return ArcticMoE(mc, dtype=dtype, device=device)
