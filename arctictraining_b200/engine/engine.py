# SPDX-License-Identifier: Apache-2.0
"""The training engine: flat-buffer ZeRO stages 0-3, mixed precision, gradient accumulation and
clipping, per-layer activation checkpointing with optional host offload, and sharded checkpoints.

It takes the place of the external engine the reference drives through ``deepspeed.initialize``
(arctic_training/trainer/trainer.py:315-322) and offers the same surface to trainers and checkpoint
engines: ``backward(loss)``, ``step()``, ``global_steps``, ``is_gradient_accumulation_boundary()``,
``save_checkpoint`` / ``load_checkpoint``, ``module``, ``lr_scheduler``, ``get_global_grad_norm()``,
``zero_optimization_stage()``, ``get_wall_clock_timers()``.

Design
------
* The model is cut into *units* (one per decoder layer, plus embedding and head).  All parameters of a
  unit live in one flat low-precision buffer; ``param.data`` are views into it.  The trainable prefix of
  each unit is covered by fp32 master / Adam state shards (1/world of the unit per rank for stage >= 1).
* Stage 3 keeps only the shard resident.  Checkpointed units are gathered into one of a few pooled
  full-size buffers right before they run (forward, and again for recompute + backward) with the next
  unit prefetched on a communication stream; small or non-checkpointed units stay gathered.
* Backward of a unit writes into a pooled flat gradient buffer which is then reduced (reduce-scatter
  for stage >= 1, all-reduce for stage 0) on the communication stream and accumulated into the fp32
  gradient shard while earlier layers are still computing.
* The optimizer only ever sees flat fp32 views (one per unit and weight-decay group), so any
  ``torch.optim.Optimizer`` works; with the framework's fused AdamW the update, the clip factor and
  the low-precision parameter write happen in one kernel per view.
"""

from __future__ import annotations

import os
import time
import weakref
from contextlib import contextmanager
from contextlib import nullcontext
from pathlib import Path
from typing import Any
from typing import Callable
from typing import Dict
from typing import Iterable
from typing import List
from typing import Optional
from typing import Sequence
from typing import Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..logging import logger
from ..exceptions import EngineConfigError
from .config import EngineConfig
from .timers import TimerGroup

ALIGN = 256  # elements; keeps every shard 16-byte aligned for fp32 and bf16 vector kernels


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


class _BufferPool:
    """A few reusable device buffers with events so that a buffer is not reused while a side stream
    still reads or writes it."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, count: int) -> None:
        self.bufs = [torch.empty(numel, dtype=dtype, device=device) for _ in range(count)]
        self.free = list(range(count))
        self.events: List[Optional[torch.cuda.Event]] = [None] * count

    def acquire(self) -> Tuple[int, torch.Tensor]:
        if not self.free:
            raise RuntimeError("engine buffer pool exhausted (more units alive than pooled buffers)")
        idx = self.free.pop(0)
        ev = self.events[idx]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self.events[idx] = None
        return idx, self.bufs[idx]

    def release(self, idx: int, event: Optional["torch.cuda.Event"] = None) -> None:
        self.events[idx] = event
        self.free.append(idx)


class ZeroUnit:
    """One sharding / checkpointing unit: a flat parameter buffer plus optimizer-state shards."""

    def __init__(self, name: str, modules: Sequence[nn.Module], checkpointed: bool, index: int) -> None:
        self.name = name
        self.modules = list(modules)
        self.checkpointed = checkpointed
        self.index = index
        self.params: List[nn.Parameter] = []
        self.param_names: List[str] = []
        self.offsets: List[int] = []
        self.numel = 0  # padded
        self.n_train = 0  # elements of the trainable prefix (unpadded)
        self.shard_size = 0
        self.flat: Optional[torch.Tensor] = None  # full low-precision buffer (None while released in stage 3)
        self.shard: Optional[torch.Tensor] = None  # this rank's slice (persistent in stage 3)
        self.persistent = True
        self.pool_slot: Optional[int] = None
        self.gather_event = None
        self.grad_flat: Optional[torch.Tensor] = None
        self.grad_slot: Optional[int] = None
        self.master: Optional[torch.Tensor] = None
        self.grad_acc: Optional[torch.Tensor] = None
        self.grad_acc_valid = False
        self.runs: List[Tuple[int, int, int]] = []  # (start, end, group) inside the local trainable shard
        self.group: Optional[dist.ProcessGroup] = None
        self.group_size = 1
        self.group_rank = 0
        self.resident = True
        self.grad_divisor = 1.0
        self.host_states = False  # master weights, moments and the gradient shard live in pinned host memory
        self.host_params = False  # the low-precision shard lives in pinned host memory (parameter offload)
        self.grad_event = None    # completion of the asynchronous device -> host copy of the gradient shard
        self.grad_sumsq = None    # sum of squares of that shard, computed on the device before it left
        self.lp_stage: Optional[torch.Tensor] = None  # pinned bf16 buffer the host optimizer writes updated weights to
        self.grad_symm = None     # symmetric gradient buffer of a unit outside the pool (embedding, head)
        self.grad_hook_left = 0   # parameters of such a unit whose gradients have not arrived yet in this backward

    @property
    def train_len(self) -> int:
        """Length of this rank's part of the trainable prefix."""
        lo = self.group_rank * self.shard_size
        return max(0, min(self.n_train - lo, self.shard_size))


_LIVE_ENGINES: "weakref.WeakSet[TrainingEngine]" = weakref.WeakSet()


def live_engines() -> List["TrainingEngine"]:
    """Engines that currently exist in this process, oldest first (look-up of the engine that owns a parameter)."""
    return sorted(_LIVE_ENGINES, key=lambda e: e._serial)


class TrainingEngine:
    _next_serial = 0

    def __init__(
        self,
        model: nn.Module,
        optimizer: Optional[torch.optim.Optimizer] = None,
        lr_scheduler: Any = None,
        config: Optional[Dict[str, Any]] = None,
        dp_group: Optional[dist.ProcessGroup] = None,
        expert_dp_group: Optional[dist.ProcessGroup] = None,
        is_expert_param: Optional[Callable[[str, nn.Parameter], bool]] = None,
        training: bool = True,
    ) -> None:
        self.module = model
        self.optimizer = optimizer
        self.lr_scheduler = lr_scheduler
        self.cfg = EngineConfig.from_dict(config)
        self._serial = TrainingEngine._next_serial
        TrainingEngine._next_serial += 1
        _LIVE_ENGINES.add(self)
        self.training_mode = training
        self.device = next(model.parameters()).device
        self.on_gpu = self.device.type == "cuda"
        self._nvtx = self.on_gpu and os.getenv("ATB200_NVTX", "0") == "1"
        self.dist_on = dist.is_initialized() and dist.get_world_size() > 1
        self.dp_group = dp_group
        self.expert_dp_group = expert_dp_group
        self._is_expert_param = is_expert_param or (lambda n, p: False)
        self.world = dist.get_world_size(dp_group) if self.dist_on else 1
        self.rank = dist.get_rank(dp_group) if self.dist_on else 0
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.stage = self.cfg.zero_stage if (training and optimizer is not None) else min(self.cfg.zero_stage, 3)
        if not training and self.stage in (1, 2):
            self.stage = 0
        self.gas = max(1, self.cfg.gradient_accumulation_steps)
        self.global_steps = 0
        self.micro_steps = 0
        self.global_samples = 0
        self.skipped_steps = 0
        self._grad_norm: Optional[torch.Tensor] = None
        self._single_pass_sumsq: Optional[torch.Tensor] = None
        # fp16: gradients are computed on a scaled loss; the scale is divided out when they are accumulated, halved
        # after a step whose gradient norm is not finite (that step is skipped) and doubled after a window of good steps
        self.loss_scale = 1.0
        self._good_steps = 0
        if self.cfg.fp16:
            self.loss_scale = self.cfg.loss_scale if self.cfg.loss_scale > 0 else float(2 ** self.cfg.initial_scale_power)
        self.timers = TimerGroup()
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.on_gpu else None
        self.sp_size = max(1, self.cfg.sequence_parallel_size)
        self._dummy = torch.zeros((), device=self.device, requires_grad=True)
        self.checkpoint_activations = bool(getattr(model, "activation_checkpointing", True)) and training
        from .activation import ActivationStore

        self.act_store = ActivationStore(self.device, offload=self.cfg.activation_checkpoint_cpu_offload)
        self.units: List[ZeroUnit] = []
        self._build_units()
        self._layout_units()
        if training and optimizer is not None:
            self._attach_optimizer()
        self._wrap_units()
        self._native_launches = 0

    # ================================================================== construction
    def _discover_units(self) -> List[Tuple[str, List[nn.Module], bool]]:
        m = self.module
        if hasattr(m, "zero_units"):
            return list(m.zero_units())
        best, best_n = None, 0
        for mod in m.modules():
            if isinstance(mod, nn.ModuleList) and len(mod) > 1:
                n = sum(p.numel() for p in mod.parameters())
                if n > best_n:
                    best, best_n = mod, n
        units: List[Tuple[str, List[nn.Module], bool]] = []
        if best is not None:
            for i, layer in enumerate(best):
                units.append((f"layer{i}", [layer], True))
        units.append(("rest", [m], False))
        return units

    def _build_units(self) -> None:
        seen: Dict[int, str] = {}
        names = {id(p): n for n, p in self.module.named_parameters(remove_duplicate=True)}
        ckpt_ok = self.checkpoint_activations or not self.training_mode
        for idx, (name, mods, ckpt) in enumerate(self._discover_units()):
            unit = ZeroUnit(name, mods, bool(ckpt and ckpt_ok), idx)
            for mod in mods:
                for p in mod.parameters():
                    if id(p) in seen:
                        continue
                    seen[id(p)] = name
                    unit.params.append(p)
            if not unit.params:
                unit.checkpointed_only = True
            expert_flags = {self._is_expert_param(names.get(id(p), ""), p) for p in unit.params}
            unit.is_expert = expert_flags == {True}
            if True in expert_flags and False in expert_flags:
                # split: expert parameters get a unit of their own so they can use their own group
                exp = ZeroUnit(name + ".experts", [], False, idx)
                exp.params = [p for p in unit.params if self._is_expert_param(names.get(id(p), ""), p)]
                exp.is_expert = True
                exp.attached_to = unit
                unit.params = [p for p in unit.params if not self._is_expert_param(names.get(id(p), ""), p)]
                unit.is_expert = False
                unit.expert_unit = exp
                self.units.append(unit)
                self.units.append(exp)
                continue
            self.units.append(unit)
        leftovers = [p for p in self.module.parameters() if id(p) not in seen]
        if leftovers:
            misc = ZeroUnit("misc", [], False, len(self.units))
            misc.params = []
            for p in leftovers:
                if id(p) not in seen:
                    seen[id(p)] = "misc"
                    misc.params.append(p)
            misc.is_expert = False
            self.units.append(misc)
        for i, u in enumerate(self.units):
            u.index = i
            u.param_names = [names.get(id(p), f"{u.name}.{j}") for j, p in enumerate(u.params)]

    def _group_index_of(self, p: nn.Parameter) -> int:
        if self.optimizer is None:
            return 0
        return self._param_group.get(id(p), -1)

    def _layout_units(self) -> None:
        self._param_group: Dict[int, int] = {}
        if self.optimizer is not None:
            for gi, g in enumerate(self.optimizer.param_groups):
                for p in g["params"]:
                    self._param_group[id(p)] = gi
        max_pool_numel = 0
        self._decide_host_placement()
        for u in self.units:
            if getattr(u, "is_expert", False) and self.expert_dp_group is not None:
                u.group = self.expert_dp_group
            else:
                u.group = self.dp_group
            u.group_size = dist.get_world_size(u.group) if self.dist_on else 1
            u.group_rank = dist.get_rank(u.group) if self.dist_on else 0
            shard_ways = u.group_size if self.stage >= 1 else 1
            if self.stage == 0:
                u.group_rank_for_shard = 0
            trainable = [p for p in u.params if p.requires_grad and self._group_index_of(p) >= 0] if self.optimizer else []
            trainable.sort(key=lambda p: self._group_index_of(p))
            frozen = [p for p in u.params if not any(p is q for q in trainable)]
            ordered = trainable + frozen
            names = dict(zip(map(id, u.params), u.param_names))
            u.params = ordered
            u.param_names = [names[id(p)] for p in ordered]
            off = 0
            u.offsets = []
            u.shapes = [tuple(p.shape) for p in ordered]
            u.numels = [p.numel() for p in ordered]
            for p in ordered:
                u.offsets.append(off)
                off += p.numel()
                off = (off + 7) // 8 * 8  # keep every parameter 16-byte aligned (TMA, vector loads)
            u.n_train = 0
            u.n_trainable_params = len(trainable)
            u.param_group_index = [self._group_index_of(p) for p in trainable]
            if trainable:
                u.n_train = u.offsets[len(trainable) - 1] + trainable[-1].numel()
            gran = ALIGN * shard_ways
            u.numel = max(gran, (off + gran - 1) // gran * gran)
            u.shard_size = u.numel // shard_ways
            if self.stage == 0:
                u.group_rank = 0  # every rank owns the whole unit
            dtype = u.params[0].dtype if u.params else torch.float32
            u.dtype = dtype
            flat = torch.zeros(u.numel, dtype=dtype, device=self.device)
            for p, o in zip(ordered, u.offsets):
                flat[o : o + p.numel()].copy_(p.data.reshape(-1))
                p.data = flat[o : o + p.numel()].view(p.shape)
                p._atb_numel = p.numel()  # the logical size: ``p.data`` is empty while a stage-3 unit is released
            u.flat = flat
            lo = u.group_rank * u.shard_size
            # a group of one rank has nothing to gather: the shard is the whole unit and stays in place
            u.host_params = bool(self.cfg.offload_param and self.stage == 3 and u.checkpointed and self.on_gpu)
            u.persistent = not (
                self.stage == 3 and u.checkpointed and (u.group_size > 1 or u.host_params)
                and u.numel >= self._persist_threshold()
            )
            u.host_params = u.host_params and not u.persistent
            if self.stage == 3 and not u.persistent:
                if u.host_params:
                    # parameter offload: the shard waits in pinned host memory and is copied in right before use
                    u.shard = torch.empty(u.shard_size, dtype=dtype, device="cpu", pin_memory=True)
                    u.shard.copy_(flat[lo : lo + u.shard_size])
                else:
                    u.shard = flat[lo : lo + u.shard_size].clone()
                max_pool_numel = max(max_pool_numel, u.numel)
            else:
                u.shard = flat[lo : lo + u.shard_size]
            # runs of the local trainable shard by optimizer group
            u.runs = self._runs_of_rank(u, u.group_rank)
            dp_replicas = max(1, (dist.get_world_size() if self.dist_on else 1) // self.sp_size)
            u.grad_divisor = float(dp_replicas)
        self._setup_fused_comm(max_pool_numel)
        self._param_pool: Optional[_BufferPool] = None
        if max_pool_numel:
            dtype = next(u.dtype for u in self.units if not u.persistent)
            # the running unit plus the units being prefetched (``ATB200_PREFETCH_DEPTH``, default 1: a deeper prefetch
            # measured no faster on two GPUs) plus one in release
            self._prefetch_depth = max(1, int(os.getenv("ATB200_PREFETCH_DEPTH", "1")))
            self._param_pool = _BufferPool(max_pool_numel, dtype, self.device, 2 + self._prefetch_depth)
            for u in self.units:
                if not u.persistent:
                    self._release_params(u)
        self._grad_pool: Optional[_BufferPool] = None
        if self.training_mode and self.optimizer is not None:
            train_units = [u for u in self.units if u.n_train > 0 and u.checkpointed]
            if train_units:
                n = max(u.numel for u in train_units)
                self._grad_pool = _BufferPool(n, train_units[0].dtype, self.device, 3 if self.on_gpu else 1)
                if self.symm is not None and train_units[0].dtype == torch.bfloat16:
                    # gradient buffers that peers read directly: same three slots on every rank
                    self._grad_symm = [self.symm.alloc(f"grad{i}", n, torch.bfloat16) for i in range(3)]
                    self._grad_pool.bufs = [b.tensor for b in self._grad_symm]
            if self.symm is not None:
                # the large units outside the pool (embedding, head) get symmetric gradient buffers of their own, so
                # that they are reduced by the same peer-memory kernel, as soon as their gradients are complete
                for u in self.units:
                    if (not u.checkpointed and u.n_train > 0 and u.group_size > 1 and u.dtype == torch.bfloat16
                            and not getattr(u, "is_expert", False) and u.numel >= (1 << 16)):
                        u.grad_symm = self.symm.alloc(f"grad_{u.name}", u.numel, torch.bfloat16)
                self._install_grad_ready_hooks()

    @staticmethod
    def _runs_of_rank(u: ZeroUnit, group_rank: int) -> List[Tuple[int, int, int]]:
        """``(start, end, optimizer group)`` runs of the trainable prefix inside the shard of ``group_rank``.  The layout
        is the same on every rank, so any rank can compute the runs of any other (decisions that must agree across
        the group are taken over all ranks' runs)."""
        lo = group_rank * u.shard_size
        runs: List[Tuple[int, int, int]] = []
        for o, n, gi in zip(u.offsets[: u.n_trainable_params], u.numels, u.param_group_index):
            s, e = max(o, lo) - lo, min(o + n, lo + u.shard_size) - lo
            if e <= s:
                continue
            if runs and runs[-1][2] == gi:
                runs[-1] = (runs[-1][0], e, gi)
            else:
                runs.append((s, e, gi))
        return runs

    def _decide_host_placement(self) -> None:
        """``zero_optimization.offload_optimizer``: which units keep master weights, moments and gradient shards in
        host memory.  ``ratio`` is the fraction of the trainable elements that is offloaded (units are taken in
        model order until the fraction is reached); the rest is updated on the device.  The decision uses sizes
        that are the same on every rank (the unit's trainable length, not the local slice of it).  The reference
        passes these keys to its engine (projects/sequence-parallelism/run-h100-sp1-llama-8b.yml:8-14,
        news/qwen3-32b-dgx-station/run-qwen3-32b.yml:7-12)."""
        for u in self.units:
            u.host_states = False
        if not (self.cfg.offload_optimizer and self.training_mode and self.optimizer is not None):
            return
        pg = {id(p) for g in self.optimizer.param_groups for p in g["params"]}
        sizes = [sum(p.numel() for p in u.params if p.requires_grad and id(p) in pg) for u in self.units]
        total = float(sum(sizes)) or 1.0
        ratio = min(1.0, max(0.0, self.cfg.offload_optimizer_ratio))
        done = 0
        for u, n in zip(self.units, sizes):
            u.host_states = n > 0 and done < ratio * total - 0.5
            done += n

    def _setup_fused_comm(self, max_pool_numel: int) -> None:
        """Peer-memory data plane: on when the whole data-parallel group sits on one NVLink node."""
        from ..comm.symm import SymmetricContext
        from ..comm.symm import symmetric_memory_available

        self.symm = None
        # ZeRO-3 parameter gathers run as peer copies on the copy engines (measured 3 % faster per step on 4 GPUs than the
        # pull kernel, which shares the SMs with the GEMMs of the compute stream); ATB200_GATHER=kernel: pull kernel
        self._gather_on_copy_engines = os.getenv("ATB200_GATHER", "ce") != "kernel"
        self._grad_symm = None
        self._shard_symm = None
        want = self.cfg.fused_comm != "off" and self.stage >= 1 and self.expert_dp_group is None
        if not (want and self.on_gpu and self.dist_on and symmetric_memory_available(self.dp_group)):
            return
        try:
            self.symm = SymmetricContext(self.dp_group)
        except Exception as exc:  # noqa: BLE001
            logger.warning(f"peer-memory communication unavailable ({exc}); using NCCL")
            self.symm = None
            return
        if self.stage >= 1:
            # bf16 shards live in one symmetric slab so that peers can pull them: the released units of stage 3
            # (gathered right before use) and the units that stay assembled (every unit below stage 3; embedding and
            # head at stage 3), whose full buffers are re-assembled from the peers' shards after each update
            units = [u for u in self.units
                     if u.dtype == torch.bfloat16 and not u.host_params and u.group_size > 1 and not getattr(u, "is_expert", False)
                     and (not u.persistent or (u.n_train > 0 and self.training_mode and self.optimizer is not None))]
            total = sum(u.shard_size for u in units)
            if total:
                self._shard_symm = self.symm.alloc("shards", total, torch.bfloat16)
                off = 0
                for u in units:
                    view = self._shard_symm.tensor[off : off + u.shard_size]
                    view.copy_(u.shard)
                    u.shard = view
                    u.symm_shard_offset = off
                    off += u.shard_size
                torch.cuda.synchronize()
                dist.barrier(group=self.dp_group, device_ids=[self.device.index])

    def _install_grad_ready_hooks(self) -> None:
        """Units that are not wrapped (embedding, final norm + head) are reduced as soon as every one of their
        parameters has received its gradient in the running backward pass: the head's weight gradient exists right at
        the start of backward, and reducing it then leaves the whole pass to hide the transfer.  A parameter that
        gets no gradient in some pass simply leaves the unit to the sweep at the end of ``backward``."""
        for u in self.units:
            if u.grad_symm is None:
                continue
            trainable = [p for p in u.params[: u.n_trainable_params]]
            u.grad_hook_params = len(trainable)

            def hook(_p, __unit=u):
                if __unit.grad_flat is None:
                    return
                __unit.grad_hook_left -= 1
                if __unit.grad_hook_left == 0:
                    self._reduce_unit(__unit)

            for p in trainable:
                p.register_post_accumulate_grad_hook(hook)

    def _persist_threshold(self) -> int:
        zo = self.cfg.raw.get("zero_optimization", {}) or {}
        return int(zo.get("stage3_param_persistence_threshold", 0) or 0)

    def _attach_optimizer(self) -> None:
        """Replace the optimizer's parameters by flat fp32 views over the local shards."""
        opt = self.optimizer
        state_dtype = torch.bfloat16 if self.cfg.bf16_optimizer_states else torch.float32
        master_dtype = torch.bfloat16 if self.cfg.bf16_master_weights_and_grads else torch.float32
        new_groups: List[List[torch.Tensor]] = [[] for _ in opt.param_groups]
        self._views: List[Tuple[ZeroUnit, int, int, int, torch.Tensor]] = []
        for u in self.units:
            tl = u.train_len
            if tl <= 0:
                continue
            opt_dev = torch.device("cpu") if u.host_states else self.device
            pad = (tl + 7) // 8 * 8
            u.view_list = []
            u.master = torch.zeros(pad, dtype=master_dtype, device=opt_dev, pin_memory=(opt_dev.type == "cpu" and self.on_gpu))
            u.master[:tl].copy_(u.shard[:tl].to(master_dtype))
            # Without accumulation steps and without peers to reduce with, the bf16 gradients that autograd writes
            # are final: the unit's gradient buffer lives for the whole step and the optimizer reads it directly
            # (no fp32 copy: 4 bytes per parameter less memory and one pass less over the gradients).
            u.direct_grad = bool(
                self.gas == 1 and u.group_size == 1 and self.on_gpu and opt_dev == self.device and u.persistent
                and u.dtype == torch.bfloat16 and master_dtype == torch.float32 and hasattr(opt, "step_flat")
                and os.getenv("ATB200_DIRECT_GRADS", "1") != "0"
            )
            if u.direct_grad:
                u.grad_acc = torch.zeros(pad, dtype=torch.bfloat16, device=self.device)
            else:
                u.grad_acc = torch.zeros(pad, dtype=torch.float32 if master_dtype == torch.float32 else master_dtype,
                                         device=opt_dev, pin_memory=(opt_dev.type == "cpu" and self.on_gpu))
            lp_ok = master_dtype == torch.float32 and u.dtype == torch.bfloat16
            lp_target = None  # where the optimizer kernel writes the rounded weights in the same pass
            if lp_ok and opt_dev == self.device and not u.host_params:
                lp_target = u.shard
            elif lp_ok and opt_dev.type == "cpu" and self.on_gpu:
                if u.host_params:
                    lp_target = u.shard  # host optimizer -> host shard: the update never touches the device
                else:
                    u.lp_stage = torch.empty(pad, dtype=torch.bfloat16, device="cpu", pin_memory=True)
                    lp_target = u.lp_stage
            u.lp_in_step = lp_target is not None
            for s, e, gi in u.runs:
                view = u.master[s:e]
                view._atb_unit = u  # type: ignore[attr-defined]
                view._atb_range = (s, e)  # type: ignore[attr-defined]
                view._atb_lp = lp_target[s:e] if lp_target is not None else None  # type: ignore[attr-defined]
                view._atb_state_dtype = state_dtype  # type: ignore[attr-defined]
                new_groups[gi].append(view)
                self._views.append((u, s, e, gi, view))
                u.view_list.append((s, e, gi, view))
        opt.state.clear()
        for g, params in zip(opt.param_groups, new_groups):
            g["params"] = params

    # ================================================================== parameter residency (stage 3)
    def _assign_param_views(self, u: ZeroUnit, flat: torch.Tensor) -> None:
        for p, o, n, shp in zip(u.params, u.offsets, u.numels, u.shapes):
            p.data = flat[o : o + n].view(shp)

    def _release_params(self, u: ZeroUnit) -> None:
        if u.persistent or not u.resident and u.flat is None:
            return
        if u.pool_slot is not None:
            ev = None
            if self.on_gpu:
                ev = torch.cuda.Event()
                ev.record()
            self._param_pool.release(u.pool_slot, ev)
            u.pool_slot = None
        u.flat = None
        u.resident = False
        empty = torch.empty(0, dtype=u.dtype, device=self.device)
        for p in u.params:
            p.data = empty

    def _launch_gather(self, u: ZeroUnit) -> None:
        """Start the all-gather of a released unit into a pooled buffer (on the communication stream)."""
        if u.persistent or u.flat is not None:
            return
        slot, buf = self._param_pool.acquire()
        flat = buf[: u.numel]
        u.pool_slot = slot
        if u.host_params:
            # parameter offload: pinned host shard -> own slice of the pooled buffer (then the usual all-gather, in
            # place), all on the communication stream so that the copy of the next unit runs under this one's compute
            lo = u.group_rank * u.shard_size
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream), self._timed("gather"):
                flat[lo : lo + u.shard_size].copy_(u.shard, non_blocking=True)
                if self.dist_on and u.group_size > 1:
                    self._all_gather(flat, flat[lo : lo + u.shard_size], u.group)
                u.gather_event = torch.cuda.Event()
                u.gather_event.record()
        elif self.dist_on and u.group_size > 1:
            if self.on_gpu:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream), self._timed("gather"):
                    if self._shard_symm is not None and hasattr(u, "symm_shard_offset"):
                        # shards only change in the optimizer step, which ends with a barrier: pull directly
                        if self._gather_on_copy_engines:
                            self.symm.all_gather_copy_engine(self._shard_symm, u.symm_shard_offset, u.shard_size, flat)
                        else:
                            self.symm.all_gather(self._shard_symm, u.symm_shard_offset, u.shard_size, flat)
                    else:
                        self._all_gather(flat, u.shard, u.group)
                    u.gather_event = torch.cuda.Event()
                    u.gather_event.record()
            else:
                self._all_gather(flat, u.shard, u.group)
        else:
            flat.copy_(u.shard)
        u.flat = flat

    def _ensure_resident(self, u: ZeroUnit, prefetch: Optional[ZeroUnit] = None) -> None:
        if not u.persistent:
            if u.flat is None:
                self._launch_gather(u)
            if u.gather_event is not None:
                torch.cuda.current_stream().wait_event(u.gather_event)
                u.gather_event = None
            if not u.resident:
                self._assign_param_views(u, u.flat)
                u.resident = True
        # gathers of the following units run on the communication stream under this unit's compute
        step = 0 if prefetch is None else (1 if prefetch.index > u.index else -1)
        depth = getattr(self, "_prefetch_depth", 1)
        while prefetch is not None and depth > 0:
            if not prefetch.persistent and prefetch.flat is None:
                if len(self._param_pool.free) <= 1:
                    break  # keep one buffer for the unit that has to run next
                self._launch_gather(prefetch)
            prefetch = self._neighbour(prefetch, step)
            depth -= 1

    def _neighbour(self, u: ZeroUnit, step: int) -> Optional[ZeroUnit]:
        i = u.index + step
        while 0 <= i < len(self.units):
            cand = self.units[i]
            if not cand.persistent:
                return cand
            i += step
        return None

    # ================================================================== collectives (NCCL / Gloo baseline)
    def _all_gather(self, out: torch.Tensor, shard: torch.Tensor, group) -> None:
        try:
            dist.all_gather_into_tensor(out, shard, group=group)
        except (RuntimeError, NotImplementedError):
            n = dist.get_world_size(group)
            parts = [out[i * shard.numel() : (i + 1) * shard.numel()] for i in range(n)]
            dist.all_gather(parts, shard.contiguous(), group=group)

    def _reduce_scatter(self, out: torch.Tensor, full: torch.Tensor, group) -> None:
        if not self.on_gpu:
            dist.all_reduce(full, group=group)
            r = dist.get_rank(group)
            out.copy_(full[r * out.numel() : (r + 1) * out.numel()])
            return
        dist.reduce_scatter_tensor(out, full, group=group)

    # ================================================================== unit execution
    def _wrap_units(self) -> None:
        self._wrapped_units: List[ZeroUnit] = []
        self._keep_state: Dict[str, Any] = {"phase": 0, "bytes_per_token": 0.0, "reserve": 0, "limit": 0}
        for u in self.units:
            if not u.checkpointed or not u.modules:
                continue
            u.wrapped_index = len(self._wrapped_units)
            self._wrapped_units.append(u)
            assert len(u.modules) == 1, "a checkpointed unit wraps exactly one module"
            mod = u.modules[0]
            orig = mod.forward
            engine = self

            def wrapped(x, *args, __orig=orig, __unit=u, **kwargs):
                if not torch.is_grad_enabled() or not engine.training_mode or not engine.module.training:
                    engine._ensure_resident(__unit, engine._neighbour(__unit, +1))
                    if getattr(__unit, "expert_unit", None) is not None:
                        engine._ensure_resident(__unit.expert_unit)
                    try:
                        return __orig(x, *args, **kwargs)
                    finally:
                        engine._release_params(__unit)
                # positional tensor arguments that carry gradients (e.g. shared K/V) are routed through autograd
                t_idx = [i for i, a in enumerate(args) if torch.is_tensor(a) and a.requires_grad]
                extras = [args[i] for i in t_idx]
                if not extras and engine._keeps_activations(__unit, x):
                    return engine._run_kept(__unit, __orig, x, args, kwargs)

                def fn(inp, *ext, __args=args, __idx=tuple(t_idx)):
                    call_args = list(__args)
                    for i, e in zip(__idx, ext):
                        call_args[i] = e
                    return __orig(inp, *call_args, **kwargs)

                return _CheckpointedUnit.apply(engine, __unit, fn, engine._dummy, x, *extras)

            mod.forward = wrapped  # type: ignore[method-assign]

    # ---------------------------------------------------------------- layers that keep their activations
    def _keeps_activations(self, u: ZeroUnit, x: torch.Tensor) -> bool:
        """Whether this unit runs without recomputation in this pass.  A fixed count keeps the last layers (their
        backward runs first and frees memory early); ``auto`` decides layer by layer from the memory that is
        free right now, the measured activation bytes per token and the measured head-room that the rest of a
        step needs on top of what is allocated when the first layer starts."""
        mode = self.cfg.activation_checkpoint_keep
        if not mode or not getattr(u, "keep_ok", True):
            return False
        wrapped = self._wrapped_units
        if mode != "auto":
            return u.wrapped_index >= len(wrapped) - int(mode)
        if not self.on_gpu:
            return False
        st = self._keep_state
        if u.wrapped_index == 0:
            st["alloc0"] = torch.cuda.memory_allocated(self.device)
            st["kept_bytes"] = 0
            st["kept_layers"] = 0
            if st["phase"] < 2:
                torch.cuda.reset_peak_memory_stats(self.device)
        if st["phase"] < 2:
            # two measurement passes (one layer kept, the rest recomputed): the first also sees the buffers that
            # are allocated lazily during the very first step, so the head-room is taken from the second
            return u.wrapped_index == 0
        need = int(st["bytes_per_token"] * (x.numel() // x.shape[-1]))
        ok = torch.cuda.memory_allocated(self.device) + need + st["reserve"] <= st["limit"]
        if ok:
            st["kept_bytes"] += need
            st["kept_layers"] += 1
        return ok

    def _run_kept(self, u: ZeroUnit, orig, x: torch.Tensor, args, kwargs):
        st = self._keep_state
        measure = self.cfg.activation_checkpoint_keep == "auto" and st["phase"] < 2 and self.on_gpu
        before = torch.cuda.memory_allocated(self.device) if measure else 0
        y = orig(_UnitEnter.apply(self, u, self._dummy, x), *args, **kwargs)
        if not torch.is_tensor(y):
            raise EngineConfigError(
                f"unit {u.name} returns {type(y).__name__}; only units with a single tensor output can keep activations"
            )
        y = _UnitExit.apply(self, u, y)
        if measure:
            tokens = max(1, x.numel() // x.shape[-1])
            st["bytes_per_token"] = max(1.0, (torch.cuda.memory_allocated(self.device) - before) / tokens)
        return y

    def _update_keep_state(self) -> None:
        """End of an optimizer step: turn the step's measured peak into the head-room for the next one."""
        if self.cfg.activation_checkpoint_keep != "auto" or not self.on_gpu:
            return
        st = self._keep_state
        if "alloc0" not in st:
            return
        peak = torch.cuda.max_memory_allocated(self.device)
        free, total = torch.cuda.mem_get_info(self.device)
        foreign = max(0, (total - free) - torch.cuda.memory_reserved(self.device))
        st["limit"] = int(self.cfg.activation_keep_memory_fraction * total) - foreign
        # everything that was live on top of the start-of-forward level and is not a kept layer
        reserve = peak - st["alloc0"] - st.get("kept_bytes", 0)
        if st["phase"] < 2:
            # includes the one measured layer: errs on the safe side
            st["reserve"] = int(peak - st["alloc0"]) if st["phase"] == 1 else 0
            st["phase"] += 1
        else:
            st["reserve"] = max(st["reserve"], int(reserve))
        torch.cuda.reset_peak_memory_stats(self.device)

    def _begin_unit_backward(self, u: ZeroUnit) -> None:
        self._ensure_resident(u, self._neighbour(u, -1))
        self._prepare_grad_buffer(u)
        exp = getattr(u, "expert_unit", None)
        if exp is not None:
            self._ensure_resident(exp)
            self._prepare_grad_buffer(exp)

    def _prepare_grad_buffer(self, u: ZeroUnit) -> None:
        if u.n_train <= 0 or u.grad_flat is not None:
            return
        if getattr(u, "direct_grad", False):
            g = u.grad_acc
            store_first = self._store_first_params(u) if not u.grad_acc_valid else frozenset()
            if not u.grad_acc_valid:
                if store_first:
                    # weights of plain linear layers get their first gradient by a storing GEMM epilogue: only the
                    # other (small) slices need zeroing
                    for p, o, n in zip(u.params, u.offsets, u.numels):
                        if p.requires_grad and id(p) not in store_first:
                            g[o : o + n].zero_()
                else:
                    g.zero_()
            u.grad_flat, u.grad_slot = g, None
            for p, o, n, shp in zip(u.params, u.offsets, u.numels, u.shapes):
                if p.requires_grad:
                    view = g[o : o + n].view(shp)
                    p._atb_main_grad = view
                    if id(p) in store_first:
                        # autograd must not add into the uninitialised slice: a gradient that does not come from the
                        # GEMM epilogue arrives as a tensor of its own and is folded in by _finish_store_first
                        p.grad = None
                        p._atb_grad_fresh = True
                    else:
                        p.grad = view
            u.store_first = store_first
            return
        if u.checkpointed:
            slot, buf = self._grad_pool.acquire()
            g = buf[: u.numel]
            g.zero_()
        elif u.grad_symm is not None:
            slot, g = None, u.grad_symm.tensor[: u.numel]
            g.zero_()
            u.grad_hook_left = u.grad_hook_params
        else:
            slot, g = None, torch.zeros(u.numel, dtype=u.dtype, device=self.device)
        u.grad_flat, u.grad_slot = g, slot
        for p, o, n, shp in zip(u.params, u.offsets, u.numels, u.shapes):
            if p.requires_grad:
                p.grad = g[o : o + n].view(shp)
                p._atb_main_grad = p.grad

    def _store_first_params(self, u: ZeroUnit) -> frozenset:
        """Parameters of ``u`` whose gradient buffer slice is not zeroed before the backward pass: trainable 2-D bf16
        weights of this package's plain ``Linear`` modules, whose weight gradient is written by a GEMM epilogue (store
        on the first write of a step, accumulate afterwards).  ``ATB200_STORE_FIRST_WGRAD=0`` switches it off."""
        cached = getattr(u, "_store_first_cache", None)
        if cached is not None:
            return cached
        found = set()
        if os.getenv("ATB200_STORE_FIRST_WGRAD", "1") != "0" and self.on_gpu:
            from ..models.modules import Linear

            for mod in u.modules:
                for m in mod.modules():
                    if type(m) is Linear and m.weight.requires_grad and m.weight.dim() == 2 and m.weight.dtype == torch.bfloat16:
                        found.add(id(m.weight))
            found &= {id(p) for p in u.params}
        u._store_first_cache = frozenset(found)
        return u._store_first_cache

    def _finish_store_first(self, u: ZeroUnit) -> None:
        """After the unit's backward pass: a store-first parameter that the GEMM epilogue never wrote gets its
        autograd gradient copied in (or zeros when it received none); one that was written and also received an
        autograd gradient (a weight used by two code paths) gets that added."""
        for p in u.params:
            if id(p) not in u.store_first:
                continue
            main = p._atb_main_grad
            extra = p.grad
            if getattr(p, "_atb_grad_fresh", False):
                if extra is not None:
                    main.copy_(extra)
                else:
                    main.zero_()
                p._atb_grad_fresh = False
            elif extra is not None:
                main.add_(extra)
        u.store_first = None

    def _end_unit_backward(self, u: ZeroUnit) -> None:
        self._reduce_unit(u)
        exp = getattr(u, "expert_unit", None)
        if exp is not None:
            self._reduce_unit(exp)
        self._release_params(u)

    def _reduce_unit(self, u: ZeroUnit) -> None:
        """Reduce the unit's flat gradient across its group and accumulate into the fp32 shard."""
        if u.grad_flat is None:
            return
        g = u.grad_flat
        if getattr(u, "store_first", None):
            self._finish_store_first(u)
        for p in u.params:
            p.grad = None
            p._atb_main_grad = None
        if getattr(u, "direct_grad", False):
            u.grad_flat = None
            u.grad_acc_valid = True
            return
        tl = u.train_len
        scale = 1.0 / (u.grad_divisor * self.gas * self.loss_scale)
        lo = u.group_rank * u.shard_size

        # Both decisions use values that are equal on every rank of the group: a rank whose shard holds no trainable
        # element (a partly frozen unit: LoRA, SwiftKV) still joins the barriers and skips the arithmetic.
        fused = self._fused_reduce_ok(u)
        single_pass = fused and self._single_pass_update_ok(u)

        symm_buf = u.grad_symm if u.grad_symm is not None else (
            self._grad_symm[u.grad_slot] if (self._grad_symm is not None and u.grad_slot is not None) else None)

        def work() -> None:
            if single_pass:
                # no clipping, no accumulation steps: the reduction feeds AdamW directly (one pass over the gradients:
                # peer loads -> fp32 sum -> moments, master weights and the bf16 shard), the fp32 gradient shard is
                # never written
                self.symm.barrier(slot=1)
                opt = self.optimizer
                for s, e, gi, view in (getattr(u, "view_list", None) or []):
                    group = opt.param_groups[gi]
                    st = opt._state_for(view)
                    st["step"] += 1
                    b1, b2 = group["betas"]
                    ss = torch.ops.atb200.p2p_reduce_scatter_adamw(
                        symm_buf.ptrs, lo + s, e - s, scale, view, st["exp_avg"], st["exp_avg_sq"],
                        view._atb_lp, float(group["lr"]), b1, b2, group["eps"], group["weight_decay"], st["step"],
                    )
                    self._single_pass_sumsq = ss if self._single_pass_sumsq is None else self._single_pass_sumsq + ss
                    ops.functional._count(comm="p2p_reduce_scatter_adamw")
                u.stepped_in_backward = True
                self.symm.barrier(slot=2)
                return
            if fused:
                # every rank has finished writing this unit's gradients -> read my slice from all peers, reduce
                # in fp32, accumulate; second barrier: nobody still reads a buffer that is about to be reused
                self.symm.barrier(slot=1)
                if tl > 0:
                    n8 = (tl + 7) // 8 * 8
                    self.symm.reduce_scatter_accumulate(
                        symm_buf, lo, min(n8, u.grad_acc.numel() // 8 * 8), u.grad_acc, scale,
                        overwrite=not u.grad_acc_valid,
                    )
                    u.grad_acc_valid = True
                self.symm.barrier(slot=2)
                return
            if self.dist_on and u.group_size > 1:
                # ``communication_data_type``: the dtype in which the library collective sums (the peer-memory kernel
                # always sums in fp32)
                cdt = self.cfg.communication_data_type
                src = g if cdt is None or cdt == g.dtype else g.to(cdt)
                if self.stage >= 1:
                    piece = torch.empty(u.shard_size, dtype=src.dtype, device=src.device)
                    self._reduce_scatter(piece, src, u.group)
                else:
                    dist.all_reduce(src, group=u.group)
                    piece = src[lo : lo + u.shard_size]
            else:
                piece = g[lo : lo + u.shard_size]
            if tl > 0:
                self._accumulate(u, piece[:tl], scale)

        if self.on_gpu:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                with self._timed("reduce"):
                    work()
                ev = torch.cuda.Event()
                ev.record()
            if u.grad_slot is not None:
                self._grad_pool.release(u.grad_slot, ev)
            elif u.grad_symm is None:
                g.record_stream(self.comm_stream)
        else:
            with self._timed("reduce"):
                work()
            if u.grad_slot is not None:
                self._grad_pool.release(u.grad_slot, None)
        u.grad_flat, u.grad_slot = None, None

    def _states_on_device_fp32(self, u: ZeroUnit) -> bool:
        """fp32 master weights and gradient shards that live on the device (the same answer on every rank)."""
        return not u.host_states and not self.cfg.bf16_master_weights_and_grads

    def _fused_reduce_ok(self, u: ZeroUnit) -> bool:
        """Whether this unit's gradients are reduced by the peer-memory kernel (between two device barriers) instead
        of NCCL.  Every input is the same on all ranks of the unit's group: taking the decision from rank-local
        values (for instance the length of the local trainable slice, which is zero on the ranks behind a frozen
        tail) would send some ranks into the barriers and the others into a collective nobody else joins."""
        pooled = self._grad_symm is not None and u.checkpointed
        return bool(
            self.symm is not None and (pooled or u.grad_symm is not None) and u.n_train > 0
            and self._states_on_device_fp32(u) and u.group_size > 1 and u.dtype == torch.bfloat16
            and u.shard_size % 8 == 0
        )

    def _single_pass_update_ok(self, u: ZeroUnit) -> bool:
        """Reduce-scatter and AdamW in one kernel: only without clipping (the clip factor needs the global norm of all
        gradients first) and without accumulation steps, for fp32 states on the device and 8-aligned parameter runs
        on every rank of the group (group-uniform, like :meth:`_fused_reduce_ok`)."""
        opt = self.optimizer
        if (self.cfg.gradient_clipping and self.cfg.gradient_clipping > 0) or self.gas != 1 or not hasattr(opt, "step_flat"):
            return False
        if os.getenv("ATB200_SINGLE_PASS_UPDATE", "1") == "0" or u.n_train <= 0:
            return False
        if getattr(u, "is_expert", False) or not self._states_on_device_fp32(u) or u.dtype != torch.bfloat16 or u.host_params:
            return False
        if self.cfg.bf16_optimizer_states:
            return False
        return all(
            s % 8 == 0 and (e - s) % 8 == 0 for r in range(u.group_size) for s, e, gi in self._runs_of_rank(u, r)
        )

    def _accumulate(self, u: ZeroUnit, piece: torch.Tensor, scale: float) -> None:
        acc = u.grad_acc[: piece.numel()]
        if acc.device != piece.device:
            # offloaded optimizer states: the reduced shard leaves for pinned host memory on the current (communication)
            # stream while backward goes on; its squared norm is taken on the device first
            tmp = piece.float() * scale if (piece.dtype != torch.float32 or scale != 1.0) else piece
            if u.grad_acc_valid:
                if u.grad_event is not None:
                    u.grad_event.synchronize()
                host = torch.empty(tmp.shape, dtype=tmp.dtype, device="cpu", pin_memory=self.on_gpu)
                host.copy_(tmp)  # accumulation steps: add on the host (synchronous)
                acc.add_(host.to(acc.dtype))
                u.grad_sumsq = None
            else:
                u.grad_sumsq = ops.sumsq(tmp) if acc.dtype == torch.float32 else None
                acc.copy_(tmp.to(acc.dtype), non_blocking=True)
                if self.on_gpu:
                    u.grad_event = torch.cuda.Event()
                    u.grad_event.record()
        elif acc.dtype == torch.float32 and piece.dtype == torch.bfloat16:
            ops.accumulate_lp_grad(piece, acc, scale, overwrite=not u.grad_acc_valid)
        else:
            if u.grad_acc_valid:
                acc.add_(piece.to(acc.dtype), alpha=scale)
            else:
                acc.copy_(piece.to(acc.dtype) * scale)
        u.grad_acc_valid = True

    # ================================================================== public training surface
    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    @contextmanager
    def _timed(self, name: str):
        """``wall_clock_breakdown``: device-timed sections ``forward`` / ``backward`` / ``step`` on the compute stream and
        ``gather`` / ``reduce`` on the communication stream (milliseconds, merged into the trainer's JSONL metrics as
        the reference merges its engine's wall-clock timers, arctic_training/trainer/trainer.py:603-605)."""
        nvtx = self._nvtx
        if nvtx:
            torch.cuda.nvtx.range_push(f"atb200/{name}")  # ATB200_NVTX=1: phases show up as ranges in a system trace
        try:
            if not self.cfg.wall_clock_breakdown:
                yield
                return
            t = self.timers(name)
            t.start()
            try:
                yield
            finally:
                t.stop()
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()

    def forward(self, *args, **kwargs):
        with self._timed("forward"), self.autocast():
            return self.module(*args, **kwargs)

    def autocast(self):
        if self.cfg.autocast:
            return torch.autocast(device_type=self.device.type, dtype=self.cfg.autocast_dtype)
        return nullcontext()

    def train(self, mode: bool = True):
        self.module.train(mode)
        return self

    def eval(self):
        self.module.eval()
        return self

    def parameters(self):
        return self.module.parameters()

    def named_parameters(self, *a, **k):
        return self.module.named_parameters(*a, **k)

    def zero_optimization_stage(self) -> int:
        return self.stage

    def is_gradient_accumulation_boundary(self) -> bool:
        return (self.micro_steps + 1) % self.gas == 0

    def get_global_grad_norm(self) -> Optional[float]:
        return None if self._grad_norm is None else float(self._grad_norm)

    def get_wall_clock_timers(self) -> TimerGroup:
        return self.timers

    def wall_clock_breakdown(self) -> bool:
        return self.cfg.wall_clock_breakdown

    def get_lr(self) -> List[float]:
        return [g["lr"] for g in self.optimizer.param_groups] if self.optimizer else []

    def backward(self, loss: torch.Tensor) -> None:
        """Back-propagate one micro-batch; gradients end up reduced in the fp32 shards."""
        with self._timed("backward"):
            for u in self.units:
                if not u.checkpointed and u.n_train > 0:
                    self._ensure_resident(u)
                    self._prepare_grad_buffer(u)
            (loss * self.loss_scale if self.cfg.fp16 else loss).backward()
            for u in self.units:
                if u.grad_flat is not None:
                    self._reduce_unit(u)

    def step(self) -> None:
        boundary = self.is_gradient_accumulation_boundary()
        self.micro_steps += 1
        self.global_samples += self.cfg.micro_batch_size * max(1, (dist.get_world_size() if self.dist_on else 1) // self.sp_size)
        if not boundary:
            return
        if self.on_gpu:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self.check_device_errors()
        with self._timed("step"):
            self._optimizer_step()
        self.global_steps += 1
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()

    def _read_error_words(self) -> Tuple[int, int]:
        from ..comm.errors import read_error_words

        return read_error_words(self._dummy)

    def check_device_errors(self) -> None:
        """Raise if a kernel of this device gave up a bounded wait since the last check (a barrier a peer never
        reached, a staging or tensor-core wait, an expert-parallel buffer overflow).  Runs before every optimizer
        step and before every checkpoint: gradients reduced from stale peer buffers or a partial GEMM output must
        not reach the weights or the disk.  Costs one device synchronisation (nothing on a CPU engine)."""
        from ..comm.errors import raise_for_error_words

        kernel_code, comm_code = self._read_error_words()
        raise_for_error_words(kernel_code, comm_code, self.global_rank)

    # ---------------------------------------------------------------- optimizer step
    def _compute_grad_norm(self) -> torch.Tensor:
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        expert_total = torch.zeros((), dtype=torch.float32, device=self.device)
        if self._single_pass_sumsq is not None:
            total += self._single_pass_sumsq.to(self.device)
            self._single_pass_sumsq = None
        for u in self.units:
            if u.grad_acc is None or not u.grad_acc_valid:
                continue
            if u.grad_sumsq is not None:
                sq = u.grad_sumsq  # taken on the device before the shard was copied to the host
            else:
                if u.grad_event is not None:
                    u.grad_event.synchronize()
                sq = ops.sumsq(u.grad_acc)  # fp32 or bf16 on the kernel; other cases fall back inside
            sq = sq.to(self.device)
            if getattr(u, "is_expert", False) and self.expert_dp_group is not None:
                expert_total += sq
            else:
                total += sq
        if self.dist_on:
            if self.stage >= 1:
                total = self._sum_over_ranks(total)
            if self.expert_dp_group is not None:
                if self.stage >= 1:
                    dist.all_reduce(expert_total, group=self.expert_dp_group)
                # experts differ across expert-parallel ranks: sum their norms over the whole world's EP axis
                ep_world = (dist.get_world_size() // dist.get_world_size(self.expert_dp_group))
                if ep_world > 1:
                    dist.all_reduce(expert_total, group=self._ep_group_for_norm())
        return (total + expert_total).sqrt()

    def _sum_over_ranks(self, value: torch.Tensor) -> torch.Tensor:
        """Sum of a scalar over the data-parallel group.  With the peer-memory path every rank writes its part into a
        symmetric slot, a device barrier follows, and each rank reads and adds all parts in rank order (the same
        bits everywhere); otherwise a library all-reduce."""
        if self.symm is None:
            dist.all_reduce(value, group=self.dp_group)
            return value
        if getattr(self, "_scalar_symm", None) is None:
            self._scalar_symm = self.symm.alloc("scalars", 2 * 4, torch.float32)  # two turns of one 16-byte slot
            self._scalar_turn = 0
            self._scalar_gathered = torch.zeros(self.world * 4, dtype=torch.float32, device=self.device)
        turn = self._scalar_turn
        self._scalar_turn ^= 1
        slot = self._scalar_symm.tensor[turn * 4 : turn * 4 + 4]
        slot.zero_()
        slot[0:1].copy_(value.reshape(1))
        self.symm.barrier(slot=3)
        self.symm.all_gather(self._scalar_symm, turn * 4, 4, self._scalar_gathered)
        return self._scalar_gathered.view(self.world, 4)[:, 0].sum()

    def _ep_group_for_norm(self):
        return getattr(self, "ep_group", None)

    def _optimizer_step(self) -> None:
        opt = self.optimizer
        if opt is None:
            return
        norm = self._compute_grad_norm()
        self._grad_norm = norm
        if self.cfg.fp16 and self._fp16_overflow(norm):
            return
        clip = self.cfg.gradient_clipping
        coef: Optional[torch.Tensor] = None
        if clip and clip > 0:
            coef = torch.clamp(clip / (norm + 1e-6), max=1.0).reshape(1).float()
        fused = hasattr(opt, "step_flat")
        for u, s, e, gi, view in self._views:
            if getattr(u, "stepped_in_backward", False):
                view._atb_grad = None  # type: ignore[attr-defined]
                view.grad = None
                view._atb_skip = True  # type: ignore[attr-defined]
                continue
            view._atb_skip = False  # type: ignore[attr-defined]
            gslice = u.grad_acc[s:e]
            if not u.grad_acc_valid:
                gslice.zero_()
            if fused:
                view._atb_grad = gslice  # type: ignore[attr-defined]
            else:
                view.grad = gslice if coef is None else gslice * coef.to(gslice.device)
                if view.grad.dtype != view.dtype:
                    view.grad = view.grad.to(view.dtype)
        if fused:
            self._step_host_units(opt, coef)
            opt.step_flat(coef)
            opt._opt_called = True  # keeps torch's scheduler-order check quiet
        else:
            opt.step()
            for u, s, e, gi, view in self._views:
                view.grad = None
        # low-precision copies + re-gather
        for u in self.units:
            if u.master is None:
                continue
            tl = u.train_len
            if not (fused and getattr(u, "lp_in_step", False)):
                # the optimizer did not write the rounded weights itself: round the master copy
                u.shard[:tl].copy_(u.master[:tl].to(u.dtype))
            u.grad_acc_valid = False
            u.grad_sumsq = None
            u.grad_event = None
            u.stepped_in_backward = False
        self._sync_full_params()
        self._update_keep_state()

    def _fp16_overflow(self, norm: torch.Tensor) -> bool:
        """Dynamic loss scaling: a gradient norm that is not finite means the scaled loss overflowed somewhere.  The
        step is skipped (gradients dropped, ``skipped_steps`` counted) and the scale halved; after
        ``loss_scale_window`` good steps in a row the scale doubles.  One host read of the norm per step."""
        finite = bool(torch.isfinite(norm))
        dynamic = self.cfg.loss_scale <= 0
        if finite:
            self._good_steps += 1
            if dynamic and self._good_steps % self.cfg.loss_scale_window == 0:
                self.loss_scale *= 2.0
            return False
        self.skipped_steps += 1
        self._good_steps = 0
        if dynamic:
            self.loss_scale = max(self.cfg.min_loss_scale, self.loss_scale / 2.0)
        for u in self.units:
            u.grad_acc_valid = False
            u.grad_sumsq = None
            u.grad_event = None
        logger.warning(f"fp16: gradient overflow, step skipped, loss scale now {self.loss_scale:g}")
        return True

    def _step_host_units(self, opt, coef: Optional[torch.Tensor]) -> None:
        """Units whose optimizer states live in host memory, one after the other: wait for the unit's gradient shard
        to have arrived, run the host AdamW over its views (which also writes the rounded bf16 weights into a pinned
        buffer), and queue the copy of those weights back to the device on the communication stream, so that the
        copy of one unit runs under the host arithmetic of the next."""
        host_units = [u for u in self.units if u.host_states and u.master is not None and getattr(u, "view_list", None)]
        if not host_units:
            return
        scale = None if coef is None else float(coef)  # one synchronisation: the clip factor is needed on the host
        for u in host_units:
            if u.grad_event is not None:
                u.grad_event.synchronize()
            for s, e, gi, view in u.view_list:
                if view._atb_skip:
                    continue
                opt.step_one(view, opt.param_groups[gi], scale)
                view._atb_skip = True  # type: ignore[attr-defined]
            if u.lp_stage is not None and self.on_gpu:
                tl = u.train_len
                with torch.cuda.stream(self.comm_stream):
                    u.shard[:tl].copy_(u.lp_stage[:tl], non_blocking=True)
        if self.on_gpu:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def _sync_full_params(self) -> None:
        """After an update every unit that stays assembled rebuilds its full buffer from the shards: pulled from the
        peers' symmetric shard slabs where the peer-memory path is up (after a device barrier: shards are final on
        every rank before anyone reads them), through the library all-gather otherwise."""
        if self.stage == 0 or not self.dist_on:
            return
        if self.symm is not None:
            self.symm.barrier(slot=0)
        for u in self.units:
            if u.group_size <= 1 or u.master is None and u.n_train == 0:
                continue
            if u.persistent:
                if self._shard_symm is not None and hasattr(u, "symm_shard_offset"):
                    self.symm.all_gather(self._shard_symm, u.symm_shard_offset, u.shard_size, u.flat)
                else:
                    # shard is a view of flat: in-place all-gather
                    self._all_gather(u.flat, u.shard.clone() if self.on_gpu is False else u.shard, u.group)

    # ================================================================== gathered access (checkpoint export etc.)
    @contextmanager
    def gathered_unit(self, u: ZeroUnit):
        was_released = not u.persistent and u.flat is None
        self._ensure_resident(u)
        if self.on_gpu:
            torch.cuda.current_stream().synchronize()
        try:
            yield u
        finally:
            if was_released:
                self._release_params(u)

    def refresh_unit_from_full(self, u: ZeroUnit) -> None:
        """After the gathered parameters of a unit were overwritten in place (weights read from files): copy this
        rank's slice back into the resident shard and into the master weights."""
        if u.flat is None:
            return
        lo = u.group_rank * u.shard_size
        if u.shard.data_ptr() != u.flat[lo : lo + 1].data_ptr():
            u.shard.copy_(u.flat[lo : lo + u.shard_size])
        if u.master is not None:
            tl = u.train_len
            u.master[:tl].copy_(u.shard[:tl].to(u.master.dtype))

    def iter_full_named_parameters(self) -> Iterable[Tuple[str, torch.Tensor]]:
        """Yield ``(name, full tensor)`` for every parameter, gathering stage-3 units one at a time.
        Every rank must iterate (the gathers are collectives)."""
        for u in self.units:
            with self.gathered_unit(u):
                for n, p in zip(u.param_names, u.params):
                    yield n, p.data

    # ================================================================== checkpoints (sharded, resumable)
    def _ckpt_rank_file(self, d: Path) -> Path:
        return d / f"zero_pp_rank_{self.global_rank}_mp_rank_00_optim_states.pt"

    @staticmethod
    def _save_atomically(obj: Any, path: Path) -> None:
        """Write to a temporary name and rename: a job killed in the middle of a save leaves no half-written file under
        the final name (and ``latest`` is only moved once every rank has finished)."""
        tmp = path.with_name(path.name + ".tmp")
        torch.save(obj, tmp)
        os.replace(tmp, path)

    @staticmethod
    def _load_checked(path: Path) -> Any:
        from ..exceptions import CheckpointError

        if not path.exists():
            raise CheckpointError(f"checkpoint file {path} is missing")
        try:
            return torch.load(path, map_location="cpu", weights_only=False)
        except Exception as e:  # noqa: BLE001 - whatever the unpickler raises on a damaged file
            raise CheckpointError(f"checkpoint file {path} cannot be read ({type(e).__name__}: {e}); it may be truncated") from e

    def save_checkpoint(self, save_dir: Any, tag: Optional[str] = None, client_state: Optional[Dict[str, Any]] = None) -> None:
        save_dir = Path(save_dir)
        tag = tag or f"global_step{self.global_steps}"
        d = save_dir / tag
        d.mkdir(parents=True, exist_ok=True)
        if self.on_gpu:
            torch.cuda.synchronize()
        self.check_device_errors()
        units_state = {}
        for u in self.units:
            tl = u.train_len
            st: Dict[str, Any] = {
                "numel": u.numel, "shard_size": u.shard_size, "n_train": u.n_train,
                "param_names": u.param_names, "offsets": u.offsets,
                "shard": u.shard.detach().cpu().clone(),
            }
            if u.master is not None:
                st["master"] = u.master[:tl].detach().cpu().clone()
            units_state[u.name] = st
        opt_state = None
        if self.optimizer is not None:
            opt_state = self._optimizer_state_for_save()
        self._save_atomically(
            {
                "units": units_state, "optimizer": opt_state, "stage": self.stage, "world": self.world,
                "group_rank": self.rank,
            },
            self._ckpt_rank_file(d),
        )
        if self.global_rank == 0:
            self._save_atomically(
                {
                    "lr_scheduler": self.lr_scheduler.state_dict() if self.lr_scheduler is not None else None,
                    "global_steps": self.global_steps, "micro_steps": self.micro_steps,
                    "global_samples": self.global_samples, "skipped_steps": self.skipped_steps,
                    "dp_world_size": self.world, "mp_world_size": 1, "zero_stage": self.stage,
                    "client_state": client_state or {},
                    "param_shapes": {n: shp for u in self.units for n, shp in zip(u.param_names, u.shapes)},
                },
                d / "mp_rank_00_model_states.pt",
            )
        from ..moe.convert import save_moe_states

        save_moe_states(self, d)  # ep_rank_<r>_moe_layer_<l>_model_states.pt (nothing for dense models)
        if self.dist_on:
            dist.barrier()
        if self.global_rank == 0:
            (save_dir / "latest").write_text(tag)
        if self.dist_on:
            dist.barrier()

    def _optimizer_state_for_save(self) -> Dict[str, Any]:
        opt = self.optimizer
        per_view = []
        for u, s, e, gi, view in self._views:
            st = opt.state.get(view, {})
            per_view.append({
                "unit": u.name, "range": (s, e), "group": gi,
                "state": {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v) for k, v in st.items()},
            })
        groups = [{k: v for k, v in g.items() if k != "params"} for g in opt.param_groups]
        return {"views": per_view, "param_groups": groups}

    def load_checkpoint(self, load_dir: Any, tag: Optional[str] = None, load_optimizer_states: bool = True):
        load_dir = Path(load_dir)
        if tag is None:
            latest = load_dir / "latest"
            if not latest.exists():
                return None, {}
            tag = latest.read_text().strip()
        from ..exceptions import CheckpointError

        d = load_dir / tag
        if not d.is_dir():
            raise CheckpointError(f"{load_dir / 'latest'} names the checkpoint {tag!r}, but {d} does not exist")
        meta = self._load_checked(d / "mp_rank_00_model_states.pt")
        rank_file = self._ckpt_rank_file(d)
        if not rank_file.exists():
            raise CheckpointError(
                f"{rank_file} is missing: the checkpoint was written with a different world size "
                f"({meta.get('dp_world_size')}) than this run ({self.world})"
            )
        mine = self._load_checked(rank_file)
        if mine["stage"] != self.stage or mine["world"] != self.world:
            raise CheckpointError("checkpoint was written with another ZeRO stage or world size")
        for u in self.units:
            st = mine["units"].get(u.name)
            if st is None or st["numel"] != u.numel or st["param_names"] != u.param_names:
                raise CheckpointError(f"layout of unit {u.name} differs between the checkpoint and this model")
            u.shard.copy_(st["shard"].to(u.shard.dtype))
            if u.master is not None and "master" in st:
                u.master[: u.train_len].copy_(st["master"].to(u.master.dtype))
        if self.stage >= 1 and self.dist_on:
            self._sync_full_params()
        if load_optimizer_states and self.optimizer is not None and mine.get("optimizer"):
            saved = mine["optimizer"]
            for (u, s, e, gi, view), sv in zip(self._views, saved["views"]):
                assert sv["unit"] == u.name and tuple(sv["range"]) == (s, e)
                self.optimizer.state[view] = {
                    k: (v.to(view.device) if torch.is_tensor(v) and v.dim() > 0 else v) for k, v in sv["state"].items()
                }
            for g, sg in zip(self.optimizer.param_groups, saved["param_groups"]):
                for k, v in sg.items():
                    g[k] = v
        if self.lr_scheduler is not None and meta.get("lr_scheduler") is not None:
            self.lr_scheduler.load_state_dict(meta["lr_scheduler"])
        self.global_steps = meta["global_steps"]
        self.micro_steps = meta["micro_steps"]
        self.global_samples = meta.get("global_samples", 0)
        self.skipped_steps = meta.get("skipped_steps", 0)
        return str(d), meta.get("client_state", {})

    def save_pretrained(self, *args, **kwargs):
        return self.module.save_pretrained(*args, **kwargs)


class _CheckpointedUnit(torch.autograd.Function):
    """Runs one unit without keeping its activations; the backward pass gathers the unit's parameters
    again, recomputes the forward from the saved (possibly host-resident) input, back-propagates and hands
    the unit's gradients to the engine for reduction.  ``x`` is the hidden state (saved, possibly on the
    host); further tensor inputs (``extras``) are kept on the device."""

    @staticmethod
    def forward(ctx, engine: TrainingEngine, unit: ZeroUnit, fn, dummy, x, *extras):
        ctx.engine, ctx.unit, ctx.fn = engine, unit, fn
        engine._ensure_resident(unit, engine._neighbour(unit, +1))
        exp = getattr(unit, "expert_unit", None)
        if exp is not None:
            engine._ensure_resident(exp)
        with torch.no_grad():
            y = fn(x, *extras)
        engine._release_params(unit)
        ctx.handle = engine.act_store.save(x)
        ctx.x_requires_grad = x.requires_grad
        ctx.extras = [e.detach() for e in extras]
        ctx.extras_require_grad = [e.requires_grad for e in extras]
        return y

    @staticmethod
    def backward(ctx, *grads):
        engine, unit, fn = ctx.engine, ctx.unit, ctx.fn
        engine._begin_unit_backward(unit)
        x = ctx.handle.restore().detach()
        x.requires_grad_(True)
        extras = [e.requires_grad_(r) for e, r in zip(ctx.extras, ctx.extras_require_grad)]
        with torch.enable_grad():
            y = fn(x, *extras)
        outs = y if isinstance(y, (tuple, list)) else (y,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        engine._end_unit_backward(unit)
        gx = x.grad if ctx.x_requires_grad else None
        gextras = tuple(e.grad if r else None for e, r in zip(extras, ctx.extras_require_grad))
        ctx.handle = None
        ctx.extras = None
        return (None, None, None, None, gx) + gextras


class _UnitEnter(torch.autograd.Function):
    """Entry of a unit that keeps its activations: gathers the parameters on the way in; in the backward pass this
    node runs after all of the unit's own backward operations (and after the accumulation of its parameter
    gradients, which autograd schedules first), so it reduces the unit's gradients and releases the parameters."""

    @staticmethod
    def forward(ctx, engine: "TrainingEngine", unit: ZeroUnit, dummy, x):
        ctx.engine, ctx.unit = engine, unit
        engine._ensure_resident(unit, engine._neighbour(unit, +1))
        if getattr(unit, "expert_unit", None) is not None:
            engine._ensure_resident(unit.expert_unit)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._end_unit_backward(ctx.unit)
        return None, None, None, g


class _UnitExit(torch.autograd.Function):
    """Exit of a unit that keeps its activations: releases the parameters on the way out; in the backward pass it
    runs before the unit's operations and gathers the parameters again.  Operations inside the unit must have saved
    the parameter objects themselves (their storage is re-pointed at the freshly gathered buffer), not views."""

    @staticmethod
    def forward(ctx, engine: "TrainingEngine", unit: ZeroUnit, y):
        ctx.engine, ctx.unit = engine, unit
        engine._release_params(unit)
        return y.view_as(y)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._begin_unit_backward(ctx.unit)
        return None, None, g


def initialize(
    model: nn.Module,
    optimizer: Optional[torch.optim.Optimizer] = None,
    lr_scheduler: Any = None,
    config: Optional[Dict[str, Any]] = None,
    **kwargs: Any,
) -> Tuple[TrainingEngine, Optional[torch.optim.Optimizer], None, Any]:
    """Convenience constructor with the return shape of the reference's engine initialiser."""
    engine = TrainingEngine(model, optimizer, lr_scheduler, config, **kwargs)
    return engine, engine.optimizer, None, engine.lr_scheduler
