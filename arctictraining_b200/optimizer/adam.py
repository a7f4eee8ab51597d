# SPDX-License-Identifier: Apache-2.0
"""AdamW optimizers and their factories.

``FusedAdamW`` runs this library's fused CUDA kernel (one launch per flat view: moment update, bias
correction, decoupled weight decay, clip factor read from device memory, bf16 parameter write) and
falls back to the PyTorch reference on CPU.  ``CPUAdamW`` keeps states in host memory (optimizer
offload).  Registered names match the reference (arctic_training/optimizer/adam_factory.py:33-160):
``fused_adam``, ``cpu_adam``, ``fused_adam_moe``, ``cpu_adam_moe``.
"""

from __future__ import annotations

from typing import Any
from typing import Dict
from typing import List
from typing import Optional

import torch

from .. import ops
from ..config.optimizer import OptimizerConfig
from .factory import OptimizerFactory


class FusedAdamW(torch.optim.Optimizer):
    writes_lp = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))

    def _state_for(self, p: torch.Tensor) -> Dict[str, Any]:
        st = self.state[p]
        if not st:
            sdt = getattr(p, "_atb_state_dtype", torch.float32)
            st["step"] = 0
            pin = p.device.type == "cpu" and p.is_pinned()
            st["exp_avg"] = torch.zeros(p.numel(), dtype=sdt, device=p.device, pin_memory=pin)
            st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=sdt, device=p.device, pin_memory=pin)
        return st

    @torch.no_grad()
    def step_one(self, p: torch.Tensor, group: Dict[str, Any], grad_scale: Optional[torch.Tensor] = None) -> None:
        """Update one flat view (gradient in ``_atb_grad``, optional low-precision copy written to ``_atb_lp``).
        The view, its states and its gradient may live on the device (fused CUDA kernel) or in host memory
        (vectorised multi-threaded C++)."""
        g = getattr(p, "_atb_grad", None)
        if g is None:
            g = p.grad
        if g is None:
            return
        b1, b2 = group["betas"]
        st = self._state_for(p)
        st["step"] += 1
        gs = grad_scale
        if gs is not None and torch.is_tensor(gs) and gs.device != p.device:
            gs = float(gs)
        ops.adamw_step(
            p.data, g, st["exp_avg"], st["exp_avg_sq"], float(group["lr"]), b1, b2, group["eps"],
            group["weight_decay"], st["step"], gs, getattr(p, "_atb_lp", None),
        )

    @torch.no_grad()
    def step_flat(self, grad_scale: Optional[torch.Tensor] = None) -> None:
        """Update every flat view handed over by the engine (gradient in ``_atb_grad``)."""
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "_atb_skip", False):
                    continue  # already updated (during the backward pass, or view by view by the engine)
                self.step_one(p, group, grad_scale)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self.step_flat(None)
        return loss


class CPUAdamW(FusedAdamW):
    """Same update rule; the recipe name ``cpu_adam`` of the reference.  Where the states live is decided by the
    engine (``zero_optimization.offload_optimizer``): views in host memory are updated by the host kernel, views on
    the device by the CUDA kernel, so a partial offload (``ratio``) runs both."""


def _make(cls, groups: List[Dict[str, Any]], cfg: OptimizerConfig):
    return cls(groups, lr=cfg.learning_rate, betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay)


def _split_expert_groups(model: torch.nn.Module, groups: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Move expert-parallel parameters into groups of their own (flag ``moe=True``) so the engine can
    reduce them over the expert-data-parallel group only."""
    expert_ids = {id(p) for n, p in model.named_parameters() if getattr(p, "is_expert_param", False)}
    out: List[Dict[str, Any]] = []
    for g in groups:
        dense = [p for p in g["params"] if id(p) not in expert_ids]
        exp = [p for p in g["params"] if id(p) in expert_ids]
        base = {k: v for k, v in g.items() if k != "params"}
        out.append({**base, "params": dense})
        if exp:
            out.append({**base, "params": exp, "moe": True, "name": "experts"})
    return out


class FusedAdamOptimizerFactory(OptimizerFactory):
    name = "fused_adam"

    def create_optimizer(self, model: Any, optimizer_config: OptimizerConfig) -> Any:
        groups = self.get_optimizer_grouped_params(model, optimizer_config.weight_decay)
        return _make(FusedAdamW, groups, optimizer_config)


class CPUAdamOptimizerFactory(OptimizerFactory):
    name = "cpu_adam"

    def create_optimizer(self, model: Any, optimizer_config: OptimizerConfig) -> Any:
        groups = self.get_optimizer_grouped_params(model, optimizer_config.weight_decay)
        return _make(CPUAdamW, groups, optimizer_config)


class FusedAdamMoEOptimizerFactory(OptimizerFactory):
    name = "fused_adam_moe"

    def create_optimizer(self, model: Any, optimizer_config: OptimizerConfig) -> Any:
        groups = _split_expert_groups(model, self.get_optimizer_grouped_params(model, optimizer_config.weight_decay))
        return _make(FusedAdamW, groups, optimizer_config)


class CPUAdamMoEOptimizerFactory(OptimizerFactory):
    name = "cpu_adam_moe"

    def create_optimizer(self, model: Any, optimizer_config: OptimizerConfig) -> Any:
        groups = _split_expert_groups(model, self.get_optimizer_grouped_params(model, optimizer_config.weight_decay))
        return _make(CPUAdamW, groups, optimizer_config)
