# SPDX-License-Identifier: Apache-2.0
"""Learning-rate schedules as ``LambdaLR`` multipliers (own implementations of the usual families)."""

from __future__ import annotations

import math
from functools import partial
from typing import Any
from typing import Dict

from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR


def _linear(step: int, warmup: int, total: int) -> float:
    if step < warmup:
        return step / max(1, warmup)
    return max(0.0, (total - step) / max(1, total - warmup))


def _cosine(step: int, warmup: int, total: int, num_cycles: float = 0.5, min_lr_rate: float = 0.0) -> float:
    if step < warmup:
        return step / max(1, warmup)
    prog = (step - warmup) / max(1, total - warmup)
    f = max(0.0, 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * prog)))
    return f * (1 - min_lr_rate) + min_lr_rate


def _constant(step: int, warmup: int, total: int) -> float:
    return 1.0


def _constant_with_warmup(step: int, warmup: int, total: int) -> float:
    return step / max(1, warmup) if step < warmup else 1.0


def _polynomial(step: int, warmup: int, total: int, lr_end_ratio: float = 1e-7, power: float = 1.0) -> float:
    if step < warmup:
        return step / max(1, warmup)
    if step > total:
        return lr_end_ratio
    remaining = 1 - (step - warmup) / max(1, total - warmup)
    return (1 - lr_end_ratio) * remaining**power + lr_end_ratio


def _inverse_sqrt(step: int, warmup: int, total: int) -> float:
    if step < warmup:
        return step / max(1, warmup)
    shift = max(1, warmup)
    return math.sqrt(shift / (step + shift - warmup)) if warmup else 1.0 / math.sqrt(max(step, 1))


SCHEDULES = {
    "linear": _linear,
    "cosine": _cosine,
    "cosine_with_min_lr": _cosine,
    "constant": _constant,
    "constant_with_warmup": _constant_with_warmup,
    "polynomial": _polynomial,
    "inverse_sqrt": _inverse_sqrt,
}


def get_scheduler(name: str, optimizer: Optimizer, num_warmup_steps: int, num_training_steps: int,
                  scheduler_specific_kwargs: Dict[str, Any] | None = None) -> LambdaLR:
    if name not in SCHEDULES:
        raise ValueError(f"unknown scheduler {name!r}; known: {sorted(SCHEDULES)}")
    fn = partial(SCHEDULES[name], warmup=num_warmup_steps, total=num_training_steps, **(scheduler_specific_kwargs or {}))
    return LambdaLR(optimizer, fn)


def _wsd(step: int, warmup: int, stable: int, decay: int, min_lr_ratio: float, warmup_type: str = "linear",
         decay_type: str = "cosine") -> float:
    if step < warmup:
        prog = step / max(1, warmup)
        f = prog if warmup_type == "linear" else 0.5 * (1 - math.cos(math.pi * prog))
        return min_lr_ratio + (1 - min_lr_ratio) * f
    if step < warmup + stable:
        return 1.0
    if step < warmup + stable + decay:
        prog = (step - warmup - stable) / max(1, decay)
        f = 1 - prog if decay_type == "linear" else 0.5 * (1 + math.cos(math.pi * prog))
        return min_lr_ratio + (1 - min_lr_ratio) * f
    return min_lr_ratio


def get_wsd_schedule(optimizer: Optimizer, num_warmup_steps: int, num_stable_steps: int, num_decay_steps: int,
                     min_lr_ratio: float = 0.0) -> LambdaLR:
    """Warmup - stable - decay schedule."""
    return LambdaLR(optimizer, partial(_wsd, warmup=num_warmup_steps, stable=num_stable_steps, decay=num_decay_steps,
                                       min_lr_ratio=min_lr_ratio))
