# SPDX-License-Identifier: Apache-2.0
"""Typed view of the engine section of a recipe (the ``deepspeed:`` dict of the reference's YAML).

Keys understood (same spelling as the recipes of the reference, arctic_training/config/trainer.py:395-440
and projects/sequence-parallelism/*.yml): ``zero_optimization.{stage, offload_optimizer.{device,ratio},
offload_param.device, reduce_bucket_size, stage3_*}``, ``bf16|bfloat16.{enabled,
bf16_master_weights_and_grads, bf16_optimizer_states}``, ``fp16.enabled``, ``torch_autocast.{enabled,
dtype}``, ``gradient_clipping``, ``prescale_gradients``, ``gradient_accumulation_steps``,
``wall_clock_breakdown``, ``communication_data_type``, ``seq_parallel_communication_data_type``.
Own extensions: ``fused_comm`` = ``auto`` | ``off`` (peer-memory kernels vs NCCL-only);
``activation_checkpoint_keep`` = ``0`` (recompute every layer, the behaviour of the reference) | ``N`` (the last
N layers keep their activations) | ``auto`` (each step keeps as many layers as the free device memory allows).
"""

from __future__ import annotations

from dataclasses import dataclass
from dataclasses import field
from typing import Any
from typing import Dict
from typing import Optional

import torch


# keys this engine acts on (top level / zero_optimization); everything else in the section is a tuning knob of the
# engine the recipes were written for (bucket sizes, overlap switches, ...) and is reported once, not silently dropped
_ACTED_TOP = {"zero_optimization", "bf16", "bfloat16", "fp16", "torch_autocast", "gradient_clipping",
              "gradient_accumulation_steps", "wall_clock_breakdown", "communication_data_type", "fused_comm",
              "activation_checkpoint_keep", "activation_keep_memory_fraction", "activation_checkpoint_cpu_offload",
              "train_micro_batch_size_per_gpu", "train_batch_size", "sequence_parallel_size"}
_ACTED_ZERO = {"stage", "offload_optimizer", "offload_param", "stage3_param_persistence_threshold"}
# defaults that the recipe loader itself writes into the section (so that the section reads like the reference's):
# not worth a message
_QUIET = {"steps_per_print", "zero_optimization.stage3_max_live_parameters",
          "zero_optimization.stage3_prefetch_bucket_size", "zero_optimization.reduce_bucket_size"}
_reported: set = set()


def keys_without_effect(d: Dict[str, Any]) -> list:
    """Dotted names of the entries of an engine section that this engine does not act on.  ``prescale_gradients`` and
    ``seq_parallel_communication_data_type`` count only when they ask for something else than what the engine does
    (no pre-scaling; exchanges in the activation dtype, bf16)."""
    out = []
    for k, v in d.items():
        if k in _ACTED_TOP:
            continue
        if k == "prescale_gradients" and not v:
            continue
        if k == "seq_parallel_communication_data_type" and str(v).replace("torch.", "") in ("None", "bf16", "bfloat16"):
            continue
        out.append(k)
    zo = d.get("zero_optimization") or {}
    out += [f"zero_optimization.{k}" for k in zo if k not in _ACTED_ZERO]
    return sorted(k for k in out if k not in _QUIET)


def _parse_keep(v: Any) -> Any:
    if isinstance(v, str):
        if v.strip().lower() == "auto":
            return "auto"
        return int(v)
    return int(v or 0)


def _parse_comm_dtype(v: Any) -> Optional[torch.dtype]:
    if v is None:
        return None
    name = str(v).replace("torch.", "").lower()
    table = {"fp32": torch.float32, "float32": torch.float32, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
             "fp16": torch.float16, "float16": torch.float16}
    if name not in table:
        raise ValueError(f"communication_data_type: unknown dtype {v!r} (fp32, bf16 or fp16)")
    return table[name]


@dataclass
class EngineConfig:
    zero_stage: int = 0
    gradient_accumulation_steps: int = 1
    gradient_clipping: float = 1.0
    micro_batch_size: int = 1
    sequence_parallel_size: int = 1
    bf16: bool = False
    fp16: bool = False
    initial_scale_power: int = 16
    loss_scale_window: int = 1000
    min_loss_scale: float = 1.0
    loss_scale: float = 0.0  # 0: dynamic
    communication_data_type: Optional[torch.dtype] = None  # dtype in which gradients cross the wire (None: as stored)
    bf16_master_weights_and_grads: bool = False
    bf16_optimizer_states: bool = False
    autocast: bool = False
    autocast_dtype: torch.dtype = torch.bfloat16
    offload_optimizer: bool = False
    offload_optimizer_ratio: float = 1.0
    offload_param: bool = False
    wall_clock_breakdown: bool = False
    fused_comm: str = "auto"
    activation_checkpoint_cpu_offload: bool = False
    activation_checkpoint_keep: Any = 0  # int, or "auto"
    activation_keep_memory_fraction: float = 0.88
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "EngineConfig":
        d = dict(d or {})
        unused = tuple(keys_without_effect(d))
        if unused and unused not in _reported:
            _reported.add(unused)
            from ..logging import logger

            logger.info("engine section: these keys tune the engine the recipe was written for and have no effect here: "
                        + ", ".join(unused))
        zo = d.get("zero_optimization", {}) or {}
        bf = d.get("bfloat16", d.get("bf16", {})) or {}
        fp = d.get("fp16", {}) or {}
        ac = d.get("torch_autocast", {}) or {}
        off_o = zo.get("offload_optimizer", {}) or {}
        off_p = zo.get("offload_param", {}) or {}
        dt = str(ac.get("dtype", "bfloat16")).replace("torch.", "")
        return cls(
            zero_stage=int(zo.get("stage", 0)),
            gradient_accumulation_steps=int(d.get("gradient_accumulation_steps", 1)),
            gradient_clipping=float(d.get("gradient_clipping", 0.0) or 0.0),
            micro_batch_size=int(d.get("train_micro_batch_size_per_gpu", 1)),
            sequence_parallel_size=int(d.get("sequence_parallel_size", 1)),
            bf16=bool(bf.get("enabled", False)),
            fp16=bool(fp.get("enabled", False)),
            initial_scale_power=int(fp.get("initial_scale_power", 16)),
            loss_scale_window=int(fp.get("loss_scale_window", 1000)),
            min_loss_scale=float(fp.get("min_loss_scale", 1.0)),
            loss_scale=float(fp.get("loss_scale", 0.0)),
            communication_data_type=_parse_comm_dtype(d.get("communication_data_type")),
            bf16_master_weights_and_grads=bool(bf.get("bf16_master_weights_and_grads", False)),
            bf16_optimizer_states=bool(bf.get("bf16_optimizer_states", False)),
            autocast=bool(ac.get("enabled", False)),
            autocast_dtype={"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
                            "fp16": torch.float16, "float32": torch.float32}.get(dt, torch.bfloat16),
            offload_optimizer=str(off_o.get("device", "none")).lower() == "cpu",
            offload_optimizer_ratio=float(off_o.get("ratio", 1.0)),
            offload_param=str(off_p.get("device", "none")).lower() == "cpu",
            wall_clock_breakdown=bool(d.get("wall_clock_breakdown", False)),
            fused_comm=str(d.get("fused_comm", "auto")),
            activation_checkpoint_cpu_offload=bool(d.get("activation_checkpoint_cpu_offload", False)),
            activation_checkpoint_keep=_parse_keep(d.get("activation_checkpoint_keep", 0)),
            activation_keep_memory_fraction=float(d.get("activation_keep_memory_fraction", 0.88)),
            raw=d,
        )
