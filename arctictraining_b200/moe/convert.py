"""Hugging Face <-> ArcticMoE parameter layouts, model conversion and expert checkpoint files.

Behaviour parity: arctic_training/model/moe/utils.py:75-666.
* HF Qwen3-MoE keeps one ``nn.Linear`` triple per expert (``mlp.experts.<i>.{gate,up,down}_proj.weight``) and
  ``mlp.gate.weight`` for the router.  ArcticMoE stacks this rank's experts into ``expert_gate_up
  [E_local, 2I, H]`` (gate/up rows block-interleaved) and ``expert_down [E_local, H, I]``.
* ``convert_to_arctic_moe`` re-creates every MoE block of a native model for the run's expert-parallel layout
  (each rank keeps only its own experts) — skipped weights are never materialised twice.
* export gathers the experts of all expert-parallel ranks back into HF names.
* expert state is checkpointed per (expert-parallel rank, layer) in
  ``ep_rank_<r>_moe_layer_<l>_model_states.pt`` files, the dense remainder only by expert-parallel rank 0.
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
from .layer import build_moe_block

_EXPERT_RE = re.compile(r"^(.*mlp\.)experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def detect_if_moe_model(model: nn.Module) -> bool:
    cfg = getattr(model, "config", {})
    get = cfg.get if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
    return bool(get("num_experts") or get("num_local_experts"))


# ------------------------------------------------------------------ state-dict converters (registered in hf_io)
def _native_to_hf(name: str, tensor: torch.Tensor, cfg: ArchConfig):
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
    if name.endswith("mlp.shared_expert_gate_up"):
        pre = name[: -len("shared_expert_gate_up")]
        g, u = ref.deinterleave_gate_up_rows(tensor)
        return [(f"{pre}shared_expert.gate_proj.weight", g), (f"{pre}shared_expert.up_proj.weight", u)]
    if name.endswith("mlp.shared_expert_down"):
        return [(name[: -len("shared_expert_down")] + "shared_expert.down_proj.weight", tensor)]
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
        if name.endswith("mlp.gate.weight"):
            out[name[: -len("gate.weight")] + "router_gate"] = hf.pop(name)
        elif name.endswith("mlp.shared_expert_gate.weight"):
            out[name[: -len("shared_expert_gate.weight")] + "shared_expert_output_gate"] = hf.pop(name)
        elif name.endswith("mlp.shared_expert.down_proj.weight"):
            out[name[: -len("shared_expert.down_proj.weight")] + "shared_expert_down"] = hf.pop(name)
        elif name.endswith("mlp.shared_expert.gate_proj.weight"):
            pre = name[: -len("shared_expert.gate_proj.weight")]
            up = hf.pop(f"{pre}shared_expert.up_proj.weight")
            out[f"{pre}shared_expert_gate_up"] = ref.interleave_gate_up_rows(hf.pop(name), up)


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
                new.shared_expert_output_gate.copy_(moe.shared_expert_output_gate)
        layer.mlp = new
        del moe
        n += 1
    return n


def gather_experts_for_export(moe: ArcticMoE) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """All experts of a block on expert-parallel rank 0 (``None`` elsewhere)."""
    if moe.ep_size == 1:
        return moe.expert_gate_up.data, moe.expert_down.data
    outs = []
    for p in (moe.expert_gate_up.data, moe.expert_down.data):
        parts = [torch.empty_like(p) for _ in range(moe.ep_size)]
        dist.all_gather(parts, p.contiguous(), group=moe.ep_group)
        outs.append(torch.cat(parts, dim=0) if moe.ep_rank == 0 else None)
    return outs[0], outs[1]


# ------------------------------------------------------------------ expert checkpoint files
def moe_state_file(directory: Path, ep_rank: int, layer_idx: int) -> Path:
    return Path(directory) / f"ep_rank_{ep_rank}_moe_layer_{layer_idx}_model_states.pt"


def save_moe_states(model: nn.Module, directory: Path, expert_dp_rank: int = 0) -> List[Path]:
    """Every expert-parallel rank (first expert-data-parallel replica only) writes its experts, one file per layer."""
    written = []
    if expert_dp_rank != 0:
        return written
    for idx, _, moe in moe_layers(model):
        f = moe_state_file(directory, moe.ep_rank, idx)
        torch.save({"expert_gate_up": moe.expert_gate_up.detach().cpu(), "expert_down": moe.expert_down.detach().cpu(),
                    "num_experts": moe.num_experts, "ep_size": moe.ep_size}, f)
        written.append(f)
    return written


def load_moe_states(model: nn.Module, directory: Path) -> int:
    n = 0
    for idx, _, moe in moe_layers(model):
        f = moe_state_file(directory, moe.ep_rank, idx)
        if not f.exists():
            continue
        st = torch.load(f, map_location="cpu", weights_only=True)
        assert st["ep_size"] == moe.ep_size, "expert checkpoint was written with another expert-parallel degree"
        with torch.no_grad():
            moe.expert_gate_up.copy_(st["expert_gate_up"])
            moe.expert_down.copy_(st["expert_down"])
        n += 1
    return n
