"""Parameter-efficient fine-tuning: LoRA adapters on the native ``Linear`` modules.

The reference delegates to the ``peft`` package (arctic_training/config/model.py:62-82,
arctic_training/model/hf_factory.py:77-84); this is an own, small implementation with the same recipe
keys (``peft_type``, ``r``, ``lora_alpha``, ``lora_dropout``, ``target_modules``).  HF target names
(``q_proj``, ``gate_proj`` ...) select the fused native projection that contains them.
"""

from __future__ import annotations

import math
from typing import Any
from typing import Dict
from typing import Iterable
from typing import Tuple

import torch
import torch.nn as nn

SUPPORTED_PEFT_TYPES = ["LORA"]
_ALIASES = {
    "q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj",
    "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj",
}


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Module, r: int, alpha: float, dropout: float) -> None:
        super().__init__()
        self.base = base
        w = base.weight
        self.lora_A = nn.Parameter(torch.empty(r, w.shape[1], dtype=w.dtype, device=w.device))
        self.lora_B = nn.Parameter(torch.zeros(w.shape[0], r, dtype=w.dtype, device=w.device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = alpha / r
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def weight(self) -> torch.Tensor:
        return self.base.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.base(x)
        return y + (self.dropout(x) @ self.lora_A.t() @ self.lora_B.t()) * self.scaling


def apply_lora(model: nn.Module, cfg: Dict[str, Any]) -> Tuple[int, int]:
    """Freeze the model, wrap the targeted projections and return (trainable, total) parameter counts."""
    targets: Iterable[str] = cfg.get("target_modules") or ["q_proj", "v_proj"]
    wanted = {_ALIASES.get(t, t) for t in targets}
    r = int(cfg.get("r", 8))
    alpha = float(cfg.get("lora_alpha", 2 * r))
    dropout = float(cfg.get("lora_dropout", 0.0))
    for p in model.parameters():
        p.requires_grad_(False)
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            if child_name in wanted and hasattr(child, "weight") and child.weight.dim() == 2:
                setattr(parent, child_name, LoRALinear(child, r, alpha, dropout))
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    total = sum(p.numel() for p in model.parameters())
    return trainable, total
