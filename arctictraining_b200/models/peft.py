# SPDX-License-Identifier: Apache-2.0
"""Parameter-efficient fine-tuning: LoRA adapters on the native ``Linear`` modules, exported in the PEFT layout.

The reference delegates to the ``peft`` package (arctic_training/config/model.py:62-82,
arctic_training/model/hf_factory.py:77-84) and saves adapters with ``save_pretrained(state_dict=trainable)``
(arctic_training/checkpoint/hf_engine.py:143-154).  This is an own, small implementation with the same recipe keys
(``peft_type``, ``r``, ``lora_alpha``, ``lora_dropout``, ``target_modules``) and the same semantics:

* a Hugging Face target name (``q_proj``, ``gate_proj`` ...) that lives inside a fused native projection (``qkv_proj``,
  ``gate_up_proj``) gets an adapter of its own — its own ``A [r, in]`` and its own ``B [rows of that projection, r]`` —
  which only touches that projection's rows of the fused output; projections that were not asked for stay untouched;
* the export is ``adapter_model.safetensors`` with ``base_model.model.<hf module>.lora_{A,B}.weight`` keys plus
  ``adapter_config.json``, which the ``peft`` package loads onto the Hugging Face base model.
"""

from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any
from typing import Dict
from typing import Iterable
from typing import List
from typing import Optional
from typing import Tuple

import torch
import torch.nn as nn

SUPPORTED_PEFT_TYPES = ["LORA"]  # on the native models; others only through the ``peft`` package on transformers models


def library_peft_types() -> List[str]:
    """Adapter types the installed ``peft`` package offers (empty without the package); usable on models that the
    factory builds through ``transformers``."""
    try:
        import peft
    except ImportError:
        return []
    mapping = getattr(peft, "PEFT_TYPE_TO_CONFIG_MAPPING", None) or getattr(getattr(peft, "mapping", None), "PEFT_TYPE_TO_CONFIG_MAPPING", {})
    return [str(getattr(k, "value", k)).upper() for k in mapping]


def apply_library_peft(model: nn.Module, cfg: Dict[str, Any]) -> nn.Module:
    """Wrap a ``transformers`` model with the ``peft`` package (any adapter type it knows), as the reference does
    (arctic_training/model/hf_factory.py:77-84)."""
    import peft

    conf = dict(cfg)
    conf["peft_type"] = str(conf["peft_type"]).upper()
    return peft.get_peft_model(model, peft.get_peft_config(conf))
_FUSED = {
    "q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj",
    "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj",
}
_GATE_UP_BLOCK = 64


def _rows_of(parent: nn.Module, fused_name: str, hf_name: str, out_features: int) -> Optional[torch.Tensor]:
    """Row indices of the fused projection's output that belong to the Hugging Face projection ``hf_name``
    (``None``: the whole output)."""
    if fused_name == "qkv_proj":
        hq, hkv, d = parent.hq, parent.hkv, parent.d
        lo = {"q_proj": 0, "k_proj": hq * d, "v_proj": (hq + hkv) * d}[hf_name]
        n = hq * d if hf_name == "q_proj" else hkv * d
        return torch.arange(lo, lo + n)
    if fused_name == "gate_up_proj":
        inter = out_features // 2
        j = torch.arange(inter)
        base = (j // _GATE_UP_BLOCK) * (2 * _GATE_UP_BLOCK) + j % _GATE_UP_BLOCK
        return base if hf_name == "gate_proj" else base + _GATE_UP_BLOCK
    return None


class LoRALinear(nn.Module):
    """``base(x)`` plus one low-rank update per adapted Hugging Face projection inside ``base``."""

    def __init__(self, base: nn.Module, r: int, alpha: float, dropout: float, rows: Dict[str, Optional[torch.Tensor]]) -> None:
        super().__init__()
        self.base = base
        w = base.weight
        self.lora_A = nn.ParameterDict()
        self.lora_B = nn.ParameterDict()
        self._row_names: List[str] = []
        for name, idx in rows.items():
            n_out = w.shape[0] if idx is None else idx.numel()
            a = nn.Parameter(torch.empty(r, w.shape[1], dtype=w.dtype, device=w.device))
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            self.lora_A[name] = a
            self.lora_B[name] = nn.Parameter(torch.zeros(n_out, r, dtype=w.dtype, device=w.device))
            if idx is not None:
                self.register_buffer(f"rows_{name}", idx.to(w.device), persistent=False)
                self._row_names.append(name)
        self.scaling = alpha / r
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def weight(self) -> torch.Tensor:
        return self.base.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.base(x)
        xd = self.dropout(x)
        for name, a in self.lora_A.items():
            delta = (xd @ a.t() @ self.lora_B[name].t()) * self.scaling
            if name in self._row_names:
                y = y.index_add(-1, getattr(self, f"rows_{name}"), delta.to(y.dtype))
            else:
                y = y + delta
        return y


def apply_lora(model: nn.Module, cfg: Dict[str, Any]) -> Tuple[int, int]:
    """Freeze the model, wrap the targeted projections and return (trainable, total) parameter counts."""
    targets: Iterable[str] = cfg.get("target_modules") or ["q_proj", "v_proj"]
    if isinstance(targets, str):
        targets = [targets]
    r = int(cfg.get("r", 8))
    alpha = float(cfg.get("lora_alpha", 2 * r))
    dropout = float(cfg.get("lora_dropout", 0.0))
    for p in model.parameters():
        p.requires_grad_(False)
    by_native: Dict[str, List[str]] = {}
    for t in targets:
        by_native.setdefault(_FUSED.get(t, t), []).append(t)
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            hf_names = by_native.get(child_name)
            if not hf_names or not hasattr(child, "weight") or child.weight.dim() != 2 or isinstance(child, LoRALinear):
                continue
            rows = {n: _rows_of(parent, child_name, n, child.weight.shape[0]) if child_name in ("qkv_proj", "gate_up_proj") else None
                    for n in hf_names}
            setattr(parent, child_name, LoRALinear(child, r, alpha, dropout, rows))
    model._peft_config = {"r": r, "lora_alpha": alpha, "lora_dropout": dropout, "target_modules": sorted(set(targets))}
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    total = sum(p.numel() for p in model.parameters())
    return trainable, total


# ---------------------------------------------------------------------------------------------- PEFT export
def peft_key(native_name: str) -> Optional[str]:
    """``model.layers.0.self_attn.qkv_proj.lora_A.q_proj`` -> ``base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight``
    (``None`` for names that are not adapter tensors)."""
    parts = native_name.split(".")
    if len(parts) < 3 or parts[-2] not in ("lora_A", "lora_B"):
        return None
    module_path = parts[:-3] + [parts[-1]]  # the fused native module name is replaced by the Hugging Face one
    return "base_model.model." + ".".join(module_path) + f".{parts[-2]}.weight"


def adapter_config(model: nn.Module, base_model_name_or_path: str) -> Dict[str, Any]:
    c = getattr(model, "_peft_config", {})
    return {
        "peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model_name_or_path,
        "r": c.get("r", 8), "lora_alpha": c.get("lora_alpha", 16), "lora_dropout": c.get("lora_dropout", 0.0),
        "target_modules": c.get("target_modules", []), "bias": "none", "fan_in_fan_out": False, "inference_mode": True,
        "init_lora_weights": True, "modules_to_save": None, "use_rslora": False, "use_dora": False,
    }


def save_adapter(out_dir: Path, named_tensors: Iterable[Tuple[str, torch.Tensor]], model: nn.Module, base_name: str) -> int:
    """Write ``adapter_model.safetensors`` + ``adapter_config.json`` from ``(native name, full tensor)`` pairs; tensors
    that are not adapter weights are ignored.  Returns the number of tensors written."""
    from safetensors.torch import save_file

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for name, t in named_tensors:
        key = peft_key(name)
        if key is not None:
            tensors[key] = t.detach().to("cpu").contiguous().clone()
    save_file(tensors, str(out_dir / "adapter_model.safetensors"), metadata={"format": "pt"})
    (out_dir / "adapter_config.json").write_text(json.dumps(adapter_config(model, base_name), indent=2))
    return len(tensors)


def merged_weight_delta(model: nn.Module) -> Dict[str, torch.Tensor]:
    """``{hf module path: B A * scaling}`` for every adapter of the model (what the update amounts to on the Hugging
    Face weight of that module); used to check an export against the model it came from."""
    out = {}
    for mod_name, mod in model.named_modules():
        if isinstance(mod, LoRALinear):
            prefix = mod_name.rsplit(".", 1)[0]
            for name, a in mod.lora_A.items():
                out[f"{prefix}.{name}"] = (mod.lora_B[name].float() @ a.float()) * mod.scaling
    return out
