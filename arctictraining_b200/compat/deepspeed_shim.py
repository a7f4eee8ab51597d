# SPDX-License-Identifier: Apache-2.0
"""Stand-in ``deepspeed`` modules for user code written against the reference.

The reference trains through an external engine package and its user-facing code (custom trainers, model factories,
checkpoint engines) imports a handful of that package's names: ``deepspeed.comm``, ``get_accelerator``,
``GatheredParameters``, ``FusedAdam`` / ``DeepSpeedCPUAdam``, ``SynchronizedWallClockTimer``, ``TiledMLP`` /
``TiledFusedLogitsLoss``, ``UlyssesSPDataLoaderAdapter``, ``deepspeed.initialize`` (inventory of the call sites:
arctic_training/trainer/trainer.py:195-354, arctic_training/checkpoint/hf_engine.py:47-64,
arctic_training/optimizer/adam_factory.py:77-127, arctic_training/metrics.py:86-101,
projects/swiftkv/train.py:113-148,197-224).  :func:`install` registers modules of those names that map every one of
them onto this package's engine, so such a file imports and runs unchanged.  Nothing is registered when the real
package is installed (unless ``force=True``), and nothing happens unless :func:`install` is called - or the
environment variable ``ATB200_DEEPSPEED_SHIM=1`` is set when ``arctic_training`` is imported.
"""

from __future__ import annotations

import contextlib
import enum
import importlib.util
import os
import sys
import time
import types
from typing import Any
from typing import Dict
from typing import Iterable
from typing import List
from typing import Optional

import torch
import torch.distributed as torch_dist

__all__ = ["install", "uninstall", "GatheredParameters", "ZeroParamStatus", "SynchronizedWallClockTimer", "Accelerator"]

_installed: List[str] = []


# ------------------------------------------------------------------------------------------------- gathered parameters
class ZeroParamStatus(enum.Enum):
    AVAILABLE = 1
    NOT_AVAILABLE = 2
    INFLIGHT = 3


def _units_of(params: Iterable[torch.nn.Parameter]):
    """(engine, unit) pairs that own the given parameters, each once, in engine order."""
    from ..engine.engine import live_engines

    wanted = {id(p) for p in params}
    found = []
    for engine in live_engines():
        for unit in engine.units:
            if any(id(p) in wanted for p in unit.params):
                found.append((engine, unit))
    return found


class GatheredParameters(contextlib.AbstractContextManager):
    """``with GatheredParameters(params, modifier_rank=None):`` - inside the block the given parameters hold their
    full values on every rank, also under ZeRO-3.  With ``modifier_rank`` set, what that rank wrote into them inside
    the block becomes the value on all ranks (shards and master weights are refreshed on exit).  Parameters that no
    engine of this package manages are left alone (they are whole already).  Every rank must enter the block."""

    def __init__(self, params, modifier_rank: Optional[int] = None, fwd_module=None, enabled: bool = True) -> None:
        if isinstance(params, torch.nn.Module):
            params = list(params.parameters())
        elif isinstance(params, torch.Tensor):
            params = [params]
        self.params = [p for p in params if p is not None]
        self.modifier_rank = modifier_rank
        self.enabled = enabled
        self._stack: Optional[contextlib.ExitStack] = None
        self._owned = []

    def __enter__(self):
        if not self.enabled:
            return self
        self._stack = contextlib.ExitStack()
        self._owned = _units_of(self.params)
        for engine, unit in self._owned:
            self._stack.enter_context(engine.gathered_unit(unit))
        return self

    def __exit__(self, *exc):
        if self._stack is None:
            return False
        try:
            if self.modifier_rank is not None and exc[0] is None:
                for engine, unit in self._owned:
                    if unit.flat is None:
                        continue
                    group = getattr(unit, "group", None)
                    if torch_dist.is_initialized() and torch_dist.get_world_size(group) > 1:
                        src = self.modifier_rank if group is None else torch_dist.get_global_rank(group, self.modifier_rank)
                        torch_dist.broadcast(unit.flat, src=src, group=group)
                    engine.refresh_unit_from_full(unit)
        finally:
            self._stack.close()
            self._stack = None
        return False


# ------------------------------------------------------------------------------------------------------------- timers
class _WallClockTimer:
    def __init__(self, name: str) -> None:
        self.name = name
        self.started_ = False
        self._t0 = 0.0
        self._elapsed = 0.0
        self._records: List[float] = []

    @staticmethod
    def _sync() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def start(self) -> None:
        self._sync()
        self._t0 = time.perf_counter()
        self.started_ = True

    def stop(self, reset: bool = False, record: bool = False) -> None:
        if not self.started_:
            return
        self._sync()
        dt = (time.perf_counter() - self._t0) * 1e3
        self._elapsed = dt if reset else self._elapsed + dt
        if record:
            self._records.append(dt)
        self.started_ = False

    def elapsed(self, reset: bool = True) -> float:
        """Milliseconds accumulated so far; a running timer keeps running."""
        running = self.started_
        if running:
            self.stop()
        out = self._elapsed
        if reset:
            self.reset()
        if running:
            self.start()
        return out

    def reset(self) -> None:
        self._elapsed = 0.0
        self.started_ = False

    def mean(self) -> float:
        return sum(self._records) / len(self._records) if self._records else 0.0


class SynchronizedWallClockTimer:
    """Named start/stop timers that synchronise the device on both ends; ``timers("name").start()`` ...
    ``.stop()`` ... ``.elapsed()`` in milliseconds."""

    Timer = _WallClockTimer

    def __init__(self) -> None:
        self.timers: Dict[str, _WallClockTimer] = {}

    def get_timers(self) -> Dict[str, _WallClockTimer]:
        return self.timers

    def __call__(self, name: str) -> _WallClockTimer:
        if name not in self.timers:
            self.timers[name] = _WallClockTimer(name)
        return self.timers[name]

    def has(self, name: str) -> bool:
        return name in self.timers

    def log(self, names: Iterable[str], normalizer: float = 1.0, reset: bool = True, ranks: Optional[List[int]] = None) -> None:
        from ..logging import logger

        parts = [f"{n}: {self.timers[n].elapsed(reset=reset) / normalizer:.2f}" for n in names if n in self.timers]
        rank = torch_dist.get_rank() if torch_dist.is_initialized() else 0
        if parts and (ranks is None or rank in ranks):
            logger.info("time (ms) | " + " | ".join(parts))

    def get_mean(self, names: Iterable[str], normalizer: float = 1.0, reset: bool = True) -> Dict[str, float]:
        return {n: self.timers[n].mean() / normalizer for n in names if n in self.timers}


# -------------------------------------------------------------------------------------------------------- accelerator
class Accelerator:
    """The device-abstraction object of the upstream package, for the one device family of this package (CUDA; CPU
    when no GPU is present, which is what the CPU tests run on)."""

    def __init__(self) -> None:
        self._cuda = torch.cuda.is_available()
        self._name = "cuda" if self._cuda else "cpu"

    def device_name(self, device_index: Optional[int] = None) -> str:
        return self._name if device_index is None or not self._cuda else f"cuda:{device_index}"

    def current_device(self) -> int:
        return torch.cuda.current_device() if self._cuda else 0

    def current_device_name(self) -> str:
        return f"cuda:{torch.cuda.current_device()}" if self._cuda else "cpu"

    def device_count(self) -> int:
        return torch.cuda.device_count() if self._cuda else 0

    def is_available(self) -> bool:
        return self._cuda

    def set_device(self, index: int) -> None:
        if self._cuda:
            torch.cuda.set_device(index)

    def synchronize(self, device_index: Optional[int] = None) -> None:
        if self._cuda:
            torch.cuda.synchronize(device_index)

    def communication_backend_name(self) -> str:
        return "nccl" if self._cuda else "gloo"

    def is_bf16_supported(self) -> bool:
        return True

    def is_fp16_supported(self) -> bool:
        return self._cuda

    def manual_seed(self, seed: int) -> None:
        torch.manual_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        torch.manual_seed(seed)
        if self._cuda:
            torch.cuda.manual_seed_all(seed)

    def get_rng_state(self, device_index: Optional[int] = None):
        return torch.cuda.get_rng_state(device_index or self.current_device()) if self._cuda else torch.get_rng_state()

    def set_rng_state(self, state, device_index: Optional[int] = None) -> None:
        if self._cuda:
            torch.cuda.set_rng_state(state, device_index or self.current_device())
        else:
            torch.set_rng_state(state)

    def empty_cache(self) -> None:
        if self._cuda:
            torch.cuda.empty_cache()

    def _mem(self, fn: str, device_index: Optional[int] = None) -> int:
        return int(getattr(torch.cuda, fn)(device_index)) if self._cuda else 0

    def memory_allocated(self, device_index: Optional[int] = None) -> int:
        return self._mem("memory_allocated", device_index)

    def max_memory_allocated(self, device_index: Optional[int] = None) -> int:
        return self._mem("max_memory_allocated", device_index)

    def memory_reserved(self, device_index: Optional[int] = None) -> int:
        return self._mem("memory_reserved", device_index)

    def max_memory_reserved(self, device_index: Optional[int] = None) -> int:
        return self._mem("max_memory_reserved", device_index)

    def reset_peak_memory_stats(self, device_index: Optional[int] = None) -> None:
        if self._cuda:
            torch.cuda.reset_peak_memory_stats(device_index)

    def total_memory(self, device_index: Optional[int] = None) -> int:
        return torch.cuda.get_device_properties(device_index or self.current_device()).total_memory if self._cuda else 0

    def available_memory(self, device_index: Optional[int] = None) -> int:
        return torch.cuda.mem_get_info(device_index)[0] if self._cuda else 0

    def Stream(self, *a: Any, **k: Any):  # noqa: N802
        return torch.cuda.Stream(*a, **k) if self._cuda else None

    def stream(self, s):
        return torch.cuda.stream(s) if self._cuda and s is not None else contextlib.nullcontext()

    def current_stream(self, device_index: Optional[int] = None):
        return torch.cuda.current_stream(device_index) if self._cuda else None

    def Event(self, **k: Any):  # noqa: N802
        return torch.cuda.Event(**k) if self._cuda else None

    def pin_memory(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor.pin_memory() if self._cuda else tensor


_accelerator: Optional[Accelerator] = None


def get_accelerator() -> Accelerator:
    global _accelerator
    if _accelerator is None:
        _accelerator = Accelerator()
    return _accelerator


# ---------------------------------------------------------------------------------------------------- module assembly
def _init_distributed(dist_backend: Optional[str] = None, auto_mpi_discovery: bool = False, timeout=None, **_: Any) -> None:
    from ..comm import dist as cdist

    cdist.init_distributed()


def _get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", 0))


def _initialize(args=None, model=None, optimizer=None, model_parameters=None, training_data=None, lr_scheduler=None,
                mpu=None, config=None, config_params=None, **kwargs: Any):
    """``deepspeed.initialize(...)`` -> ``(engine, optimizer, dataloader, lr_scheduler)`` on this package's engine."""
    from ..engine.engine import initialize

    cfg = config if config is not None else config_params
    if isinstance(cfg, (str, os.PathLike)):
        import json

        with open(cfg) as f:
            cfg = json.load(f)
    return initialize(model, optimizer=optimizer, lr_scheduler=lr_scheduler, config=dict(cfg or {}))


def _fused_adam(params, lr: float = 1e-3, bias_correction: bool = True, betas=(0.9, 0.999), eps: float = 1e-8,
                adam_w_mode: bool = True, weight_decay: float = 0.0, amsgrad: bool = False, **_: Any):
    from ..optimizer.adam import FusedAdamW

    if amsgrad or not adam_w_mode or not bias_correction:
        raise ValueError("only bias-corrected AdamW (decoupled weight decay, no amsgrad) is implemented")
    return FusedAdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)


def _cpu_adam(model_params, lr: float = 1e-3, bias_correction: bool = True, betas=(0.9, 0.999), eps: float = 1e-8,
              weight_decay: float = 0.0, amsgrad: bool = False, adamw_mode: bool = True, **_: Any):
    from ..optimizer.adam import CPUAdamW

    if amsgrad or not adamw_mode or not bias_correction:
        raise ValueError("only bias-corrected AdamW (decoupled weight decay, no amsgrad) is implemented")
    return CPUAdamW(model_params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)


class _CommModule(types.ModuleType):
    """``deepspeed.comm``: ``torch.distributed`` plus the few names that differ."""

    def __getattr__(self, name: str) -> Any:
        return getattr(torch_dist, name)


def _module(name: str, **attrs: Any) -> types.ModuleType:
    mod = _CommModule(name) if name == "deepspeed.comm" else types.ModuleType(name)
    mod.__dict__.update(attrs)
    mod.__atb200_shim__ = True
    return mod


def _build_modules() -> Dict[str, types.ModuleType]:
    from ..engine.engine import TrainingEngine
    from ..logging import logger
    from ..ops.tiled import TiledFusedLogitsLoss
    from ..ops.tiled import TiledMLP
    from ..parallel.ulysses import UlyssesDataLoaderAdapter
    from ..parallel.ulysses_hf import UlyssesSPAttentionHF

    comm = _module("deepspeed.comm", init_distributed=_init_distributed, get_local_rank=_get_local_rank)
    zero = _module("deepspeed.runtime.zero", GatheredParameters=GatheredParameters, ZeroParamStatus=ZeroParamStatus)
    partition = _module("deepspeed.runtime.zero.partition_parameters", GatheredParameters=GatheredParameters,
                        ZeroParamStatus=ZeroParamStatus)
    zero.partition_parameters = partition
    engine = _module("deepspeed.runtime.engine", DeepSpeedEngine=TrainingEngine)
    ulysses = _module("deepspeed.runtime.sequence_parallel.ulysses_sp", TiledMLP=TiledMLP,
                      TiledFusedLogitsLoss=TiledFusedLogitsLoss, UlyssesSPDataLoaderAdapter=UlyssesDataLoaderAdapter,
                      UlyssesSPAttentionHF=UlyssesSPAttentionHF)
    seqpar = _module("deepspeed.runtime.sequence_parallel", ulysses_sp=ulysses)
    runtime = _module("deepspeed.runtime", zero=zero, engine=engine, sequence_parallel=seqpar)
    adam = _module("deepspeed.ops.adam", FusedAdam=_fused_adam, DeepSpeedCPUAdam=_cpu_adam)
    ops = _module("deepspeed.ops", adam=adam)
    accelerator = _module("deepspeed.accelerator", get_accelerator=get_accelerator)
    timer = _module("deepspeed.utils.timer", SynchronizedWallClockTimer=SynchronizedWallClockTimer)
    utils = _module("deepspeed.utils", timer=timer, logger=logger)
    top = _module("deepspeed", comm=comm, zero=zero, runtime=runtime, ops=ops, accelerator=accelerator, utils=utils,
                  initialize=_initialize, init_distributed=_init_distributed, DeepSpeedEngine=TrainingEngine,
                  __version__="0.0.0+arctictraining_b200", __path__=[])
    for pkg in (runtime, zero, seqpar, ops, utils):
        pkg.__path__ = []
    return {m.__name__: m for m in (top, comm, zero, partition, engine, ulysses, seqpar, runtime, adam, ops, accelerator,
                                    timer, utils)}


def install(force: bool = False) -> bool:
    """Register the stand-in modules in ``sys.modules``.  Returns False (and registers nothing) when the real package
    is importable and ``force`` is not set, or when the stand-ins are already in place."""
    if _installed:
        return False
    existing = sys.modules.get("deepspeed")
    real_present = (existing is not None and not getattr(existing, "__atb200_shim__", False)) or (
        existing is None and importlib.util.find_spec("deepspeed") is not None)
    if real_present and not force:
        return False
    for name, mod in _build_modules().items():
        sys.modules[name] = mod
        _installed.append(name)
    return True


def uninstall() -> None:
    for name in _installed:
        if getattr(sys.modules.get(name), "__atb200_shim__", False):
            del sys.modules[name]
    _installed.clear()
