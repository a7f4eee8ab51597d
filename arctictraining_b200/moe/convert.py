# SPDX-License-Identifier: Apache-2.0
"""Hugging Face <-> ArcticMoE parameter layouts, model conversion and expert checkpoint files.

Behaviour parity: arctic_training/model/moe/utils.py:75-666.
* HF Qwen3-MoE keeps one ``nn.Linear`` triple per expert (``mlp.experts.<i>.{gate,up,down}_proj.weight``) and
  ``mlp.gate.weight`` for the router.  ArcticMoE stacks this rank's experts into ``expert_gate_up
  [E_local, 2I, H]`` (gate/up rows block-interleaved) and ``expert_down [E_local, H, I]``.
* The model factory builds MoE blocks inside ``expert_parallel_layout`` so that a rank only ever allocates its own
  experts; ``convert_to_arctic_moe`` sets the run-time switches and re-shards blocks that were built unsharded.
* export (``checkpoint/hf.py``) gathers the experts of all expert-parallel ranks back into HF names
  (``gather_expert_tensor``).
* expert state is also written per (expert-parallel rank, layer) in ``ep_rank_<r>_moe_layer_<l>_model_states.pt``
  files beside the engine's own shard files (``save_moe_states`` / ``load_moe_states``).
"""

from __future__ import annotations

import re
from pathlib import Path
from typing import Any
from typing import Dict
from typing import List
from typing import Optional
from typing import Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models import hf_io
from ..models.arch import ArchConfig
from ..ops import reference as ref
from .layer import ArcticMoE

_EXPERT_RE = re.compile(r"^(.*mlp\.)experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def detect_if_moe_model(model: nn.Module) -> bool:
    cfg = getattr(model, "config", {})
    get = cfg.get if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
    return bool(get("num_experts") or get("num_local_experts") or get("n_routed_experts"))


# ------------------------------------------------------------------ state-dict converters (registered in hf_io)
def _stacked_expert_layout(cfg: Any) -> bool:
    """gpt-oss keeps all experts of a block in two stacked tensors (``mlp.experts.gate_up_proj [E, H, 2I]`` with gate
    and up interleaved element-wise on the last dimension, ``mlp.experts.down_proj [E, I, H]``) and names its router
    ``mlp.router``; Qwen keeps one ``nn.Linear`` triple per expert.  Reference:
    arctic_training/model/moe/utils.py:118-137,198-232."""
    get = cfg.get if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
    return get("model_type") == "gpt_oss"


def _native_to_hf(name: str, tensor: torch.Tensor, cfg: ArchConfig):
    if _stacked_expert_layout(cfg):
        if name.endswith("mlp.router_gate"):
            return [(name[: -len("router_gate")] + "router.weight", tensor)]
        if name.endswith("mlp.expert_gate_up"):
            E, two_i, H = tensor.shape
            g, u = zip(*(ref.deinterleave_gate_up_rows(tensor[i]) for i in range(E)))  # [I, H] each
            gu = torch.stack([torch.stack((gi.t(), ui.t()), dim=-1).reshape(H, two_i) for gi, ui in zip(g, u)])
            return [(name[: -len("expert_gate_up")] + "experts.gate_up_proj", gu)]
        if name.endswith("mlp.expert_down"):
            return [(name[: -len("expert_down")] + "experts.down_proj", tensor.transpose(1, 2).contiguous())]
    if name.endswith("mlp.router_gate"):
        return [(name[: -len("router_gate")] + "gate.weight", tensor)]
    if name.endswith("mlp.expert_gate_up"):
        pre = name[: -len("expert_gate_up")]
        first = getattr(tensor, "_first_expert", 0)
        out = []
        for i in range(tensor.shape[0]):
            g, u = ref.deinterleave_gate_up_rows(tensor[i])
            out += [(f"{pre}experts.{first + i}.gate_proj.weight", g), (f"{pre}experts.{first + i}.up_proj.weight", u)]
        return out
    if name.endswith("mlp.expert_down"):
        pre = name[: -len("expert_down")]
        first = getattr(tensor, "_first_expert", 0)
        return [(f"{pre}experts.{first + i}.down_proj.weight", tensor[i]) for i in range(tensor.shape[0])]
    shared = "shared_experts" if cfg.get("n_routed_experts") else "shared_expert"  # DeepSeek uses the plural
    if name.endswith("mlp.shared_expert_gate_up"):
        pre = name[: -len("shared_expert_gate_up")]
        g, u = ref.deinterleave_gate_up_rows(tensor)
        return [(f"{pre}{shared}.gate_proj.weight", g), (f"{pre}{shared}.up_proj.weight", u)]
    if name.endswith("mlp.shared_expert_down"):
        return [(name[: -len("shared_expert_down")] + f"{shared}.down_proj.weight", tensor)]
    if name.endswith("mlp.shared_expert_output_gate"):
        return [(name[: -len("shared_expert_output_gate")] + "shared_expert_gate.weight", tensor)]
    return None


def _hf_to_native(hf: Dict[str, torch.Tensor], out: Dict[str, torch.Tensor], cfg: ArchConfig) -> None:
    groups: Dict[str, Dict[int, Dict[str, torch.Tensor]]] = {}
    for name in list(hf):
        m = _EXPERT_RE.match(name)
        if m:
            groups.setdefault(m.group(1), {}).setdefault(int(m.group(2)), {})[m.group(3)] = hf.pop(name)
    for pre, experts in groups.items():
        idx = sorted(experts)
        out[f"{pre}expert_gate_up"] = torch.stack(
            [ref.interleave_gate_up_rows(experts[i]["gate_proj"], experts[i]["up_proj"]) for i in idx]
        )
        out[f"{pre}expert_down"] = torch.stack([experts[i]["down_proj"] for i in idx])
    for name in list(hf):
        if name not in hf:
            continue
        if name.endswith("mlp.experts.gate_up_proj"):  # gpt-oss: [E, H, 2I], gate = [..., 0::2], up = [..., 1::2]
            gu = hf.pop(name)
            out[name[: -len("experts.gate_up_proj")] + "expert_gate_up"] = torch.stack(
                [ref.interleave_gate_up_rows(gu[e][:, 0::2].t().contiguous(), gu[e][:, 1::2].t().contiguous())
                 for e in range(gu.shape[0])]
            )
        elif name.endswith("mlp.experts.down_proj"):   # gpt-oss: [E, I, H]
            out[name[: -len("experts.down_proj")] + "expert_down"] = hf.pop(name).transpose(1, 2).contiguous()
        elif name.endswith("mlp.router.weight"):
            out[name[: -len("router.weight")] + "router_gate"] = hf.pop(name)
        elif name.endswith(("mlp.experts.gate_up_proj_bias", "mlp.experts.down_proj_bias", "mlp.router.bias")):
            b = hf.pop(name)
            if float(b.abs().max()) != 0.0:
                import warnings

                warnings.warn(f"{name}: expert / router biases are not carried by ArcticMoE and are dropped", stacklevel=2)
    for name in list(hf):
        if name.endswith("mlp.gate.weight"):
            out[name[: -len("gate.weight")] + "router_gate"] = hf.pop(name)
        elif name.endswith("mlp.shared_expert_gate.weight"):
            out[name[: -len("shared_expert_gate.weight")] + "shared_expert_output_gate"] = hf.pop(name)
        elif name.endswith(("mlp.shared_expert.down_proj.weight", "mlp.shared_experts.down_proj.weight")):
            out[name.rsplit("shared_expert", 1)[0] + "shared_expert_down"] = hf.pop(name)
        elif name.endswith(("mlp.shared_expert.gate_proj.weight", "mlp.shared_experts.gate_proj.weight")):
            up = hf.pop(name.replace("gate_proj.weight", "up_proj.weight"))
            out[name.rsplit("shared_expert", 1)[0] + "shared_expert_gate_up"] = ref.interleave_gate_up_rows(hf.pop(name), up)


if _native_to_hf not in hf_io._EXTRA_NATIVE_TO_HF:
    hf_io._EXTRA_NATIVE_TO_HF.append(_native_to_hf)
    hf_io._EXTRA_HF_TO_NATIVE.append(_hf_to_native)


# ------------------------------------------------------------------ model conversion
def moe_layers(model: nn.Module) -> List[Tuple[int, nn.Module, ArcticMoE]]:
    out = []
    layers = getattr(getattr(model, "model", model), "layers", [])
    for i, layer in enumerate(layers):
        if isinstance(getattr(layer, "mlp", None), ArcticMoE):
            out.append((i, layer, layer.mlp))
    return out


def convert_to_arctic_moe(model: nn.Module, groups: Any, is_resume: bool = False, use_fused_kernels: bool = True,
                          routing_replay: bool = False) -> int:
    """Re-shard the experts of every MoE block for the run's expert-parallel degree: each rank keeps the
    experts ``[ep_rank * E/ep, (ep_rank + 1) * E/ep)``.  Returns the number of blocks converted."""
    ep_size, ep_rank, ep_group = groups.ep_size, groups.ep_rank, groups.ep_group
    n = 0
    for _, layer, moe in moe_layers(model):
        moe._config.use_fused_kernels = use_fused_kernels
        moe._config.enable_routing_replay = routing_replay
        if ep_size == 1 or moe.ep_size == ep_size:
            n += 1
            continue
        assert moe.ep_size == 1, "experts can only be re-sharded from an unsharded block"
        cfg = moe._config
        new_cfg = type(cfg)(**{**cfg.__dict__, "ep_size": ep_size, "ep_rank": ep_rank, "ep_group": ep_group})
        new = ArcticMoE(new_cfg, dtype=moe.router_gate.dtype, device=moe.router_gate.device)
        lo, hi = new.local_expert_indices.start, new.local_expert_indices.stop
        with torch.no_grad():
            new.router_gate.copy_(moe.router_gate)
            new.expert_gate_up.copy_(moe.expert_gate_up[lo:hi])
            new.expert_down.copy_(moe.expert_down[lo:hi])
            if cfg.use_shared_expert:
                new.shared_expert_gate_up.copy_(moe.shared_expert_gate_up)
                new.shared_expert_down.copy_(moe.shared_expert_down)
                if cfg.shared_expert_gated:
                    new.shared_expert_output_gate.copy_(moe.shared_expert_output_gate)
        layer.mlp = new
        del moe
        n += 1
    return n


# ------------------------------------------------------------------ Hugging Face sparse blocks -> ArcticMoE
def _is_hf_sparse_block(m: nn.Module) -> bool:
    experts, gate = getattr(m, "experts", None), getattr(m, "gate", None)
    return (experts is not None and gate is not None and not isinstance(m, ArcticMoE)
            and hasattr(experts, "gate_up_proj") and hasattr(experts, "down_proj") and hasattr(gate, "weight"))


def arctic_moe_from_hf_block(block: nn.Module, ep_size: int = 1, ep_rank: int = 0, ep_group: Any = None,
                             loss_coeff: float = 0.0) -> ArcticMoE:
    """ArcticMoE with the weights of a ``transformers`` sparse MoE block of the Qwen family (Qwen2-MoE, Qwen3-MoE,
    Qwen3-Next: ``gate.weight [E, H]``, ``experts.gate_up_proj [E, 2I, H]`` with the gate rows first,
    ``experts.down_proj [E, H, I]``, optionally ``shared_expert`` + ``shared_expert_gate``).  With ``ep_size > 1`` the
    new block holds this rank's experts only.  Reference: arctic_training/model/moe/utils.py:75-232."""
    from .layer import MoEConfig

    experts, gate = block.experts, block.gate
    gu, down = experts.gate_up_proj.data, experts.down_proj.data
    E, two_i, H = gu.shape
    shared = getattr(block, "shared_expert", None)
    cfg = MoEConfig(
        model_dim=H, intermediate_dim=two_i // 2, num_experts=E, top_k=int(gate.top_k),
        normalize_topk_scores=bool(getattr(gate, "norm_topk_prob", True)), loss_coeff=float(loss_coeff),
        use_shared_expert=shared is not None,
        shared_intermediate_dim=int(shared.gate_proj.weight.shape[0]) if shared is not None else 0,
        shared_expert_gated=hasattr(block, "shared_expert_gate"),
        ep_size=ep_size, ep_rank=ep_rank, ep_group=ep_group, input_dtype=gu.dtype,
    )
    moe = ArcticMoE(cfg, dtype=gu.dtype, device=gu.device)
    lo, hi = moe.local_expert_indices.start, moe.local_expert_indices.stop
    with torch.no_grad():
        moe.router_gate.copy_(gate.weight.data)
        for i, e in enumerate(range(lo, hi)):
            g, u = gu[e].chunk(2, dim=0)
            moe.expert_gate_up[i].copy_(ref.interleave_gate_up_rows(g, u))
        moe.expert_down.copy_(down[lo:hi])
        if shared is not None:
            moe.shared_expert_gate_up.copy_(ref.interleave_gate_up_rows(shared.gate_proj.weight.data, shared.up_proj.weight.data))
            moe.shared_expert_down.copy_(shared.down_proj.weight.data)
            if cfg.shared_expert_gated:
                moe.shared_expert_output_gate.copy_(block.shared_expert_gate.weight.data)
    return moe


def convert_hf_blocks_to_arctic_moe(model: nn.Module, groups: Any = None, loss_coeff: float = 0.0) -> int:
    """Replace every ``transformers`` sparse MoE block of ``model`` (a model built by the ``transformers`` fallback of
    the model factory, e.g. Qwen3-Next) by an :class:`ArcticMoE` with the same weights, sharded for the run's
    expert-parallel degree.  Returns the number of blocks replaced."""
    ep_size = getattr(groups, "ep_size", 1) if groups is not None else 1
    ep_rank = getattr(groups, "ep_rank", 0) if groups is not None else 0
    ep_group = getattr(groups, "ep_group", None) if groups is not None else None
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if _is_hf_sparse_block(child):
                setattr(parent, name, arctic_moe_from_hf_block(child, ep_size, ep_rank, ep_group, loss_coeff))
                n += 1
    return n


def gather_expert_tensor(local: torch.Tensor, ep_size: int, ep_group: Any, keep: bool) -> Optional[torch.Tensor]:
    """Stack of all experts ``[E, ...]`` from the ``[E / ep_size, ...]`` stacks of an expert-parallel group, in expert
    order (expert-parallel rank r holds experts ``[r E / ep, (r + 1) E / ep)``).  A collective of the group; the result
    is kept only where ``keep`` is true (the rank that writes the export).  Reference: the expert gather before an
    export, arctic_training/model/moe/utils.py:331-422."""
    if ep_size == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(ep_size)]
    dist.all_gather(parts, local.contiguous(), group=ep_group)
    return torch.cat(parts, dim=0) if keep else None


def expert_parallel_of(model: nn.Module) -> Tuple[int, Any]:
    """``(ep_size, ep_group)`` of the model's MoE blocks (``(1, None)`` for dense models)."""
    for _, _, moe in moe_layers(model):
        return moe.ep_size, moe.ep_group
    return 1, None


# ------------------------------------------------------------------ expert checkpoint files
_LAYER_RE = re.compile(r"layers\.(\d+)\.mlp\.(expert_gate_up|expert_down)$")


def moe_state_file(directory: Path, ep_rank: int, layer_idx: int) -> Path:
    return Path(directory) / f"ep_rank_{ep_rank}_moe_layer_{layer_idx}_model_states.pt"


def save_moe_states(engine: Any, directory: Path) -> List[Path]:
    """One file per (expert-parallel rank, MoE layer) with that rank's expert stacks, next to the engine's own
    shard files (naming of the reference, arctic_training/model/moe/utils.py:541-666).  Expert units that are
    ZeRO-sharded over the expert-data-parallel group are gathered first (every rank takes part); the first replica of
    each expert-parallel rank writes."""
    module = engine.module
    blocks = {idx: moe for idx, _, moe in moe_layers(module)}
    if not blocks:
        return []
    writer = engine.expert_dp_group is None or dist.get_rank(engine.expert_dp_group) == 0
    if engine.expert_dp_group is None and dist.is_initialized():
        ep_size = next(iter(blocks.values())).ep_size
        writer = ep_size > 1 or dist.get_rank() == 0  # without expert parallelism every rank holds the same experts
    per_layer: Dict[int, Dict[str, torch.Tensor]] = {}
    for u in engine.units:
        names = [n for n in u.param_names if _LAYER_RE.search(n)]
        if not names:
            continue
        with engine.gathered_unit(u):
            for n, p in zip(u.param_names, u.params):
                m = _LAYER_RE.search(n)
                if m and writer:
                    per_layer.setdefault(int(m.group(1)), {})[m.group(2)] = p.data.detach().cpu().clone()
    written = []
    for idx, tensors in sorted(per_layer.items()):
        moe = blocks[idx]
        f = moe_state_file(directory, moe.ep_rank, idx)
        torch.save({**tensors, "num_experts": moe.num_experts, "ep_size": moe.ep_size, "ep_rank": moe.ep_rank}, f)
        written.append(f)
    return written


def load_moe_states(engine: Any, directory: Path) -> int:
    """Fill the expert stacks of this rank from the per-(rank, layer) files (e.g. into a run whose expert-data-parallel
    replication differs from the run that wrote them; the expert-parallel degree must be the same).  Returns the number
    of layers loaded."""
    module = engine.module
    blocks = {idx: moe for idx, _, moe in moe_layers(module)}
    n = 0
    for u in engine.units:
        if not any(_LAYER_RE.search(x) for x in u.param_names):
            continue
        with engine.gathered_unit(u):
            touched = False
            for name, p in zip(u.param_names, u.params):
                m = _LAYER_RE.search(name)
                if not m:
                    continue
                idx = int(m.group(1))
                f = moe_state_file(directory, blocks[idx].ep_rank, idx)
                if not f.exists():
                    continue
                st = torch.load(f, map_location="cpu", weights_only=True)
                assert st["ep_size"] == blocks[idx].ep_size, "expert files were written with another expert-parallel degree"
                with torch.no_grad():
                    p.data.copy_(st[m.group(2)].to(p.dtype))
                touched = True
                n += m.group(2) == "expert_down"
            if touched:
                engine.refresh_unit_from_full(u)
    return n
