# SPDX-License-Identifier: Apache-2.0
"""Top-level recipe config (one YAML file == one ``TrainerConfig``) and ``get_config``.

Behaviour parity: arctic_training/config/trainer.py:67-548 — same field names and defaults, sub-config
classes resolved from the trainer class' type hints (first hint is the default, ``type:`` selects
another, ``skip_validation`` lifts the compatibility check), human-readable numbers inside the engine
dict, derived batch sizes, single ``auto_resume`` engine, and loading of the user's ``train.py`` so
that custom classes register themselves before the config is validated.

The engine section keeps the YAML key ``deepspeed`` (recipes written for the reference keep working);
it configures this framework's own ZeRO engine (``arctictraining_b200.engine``).
"""

from __future__ import annotations

import importlib.util
import os
import sys
import tempfile
import uuid
from functools import partial
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Callable
from typing import Dict
from typing import List
from typing import Literal
from typing import Union

import yaml
from pydantic import Field
from pydantic import ValidationInfo
from pydantic import field_validator
from pydantic import model_validator
from typing_extensions import Self

from ..registry import _get_class_attr_type_hints
from ..registry import get_registered_checkpoint_engine
from ..registry import get_registered_data_factory
from ..registry import get_registered_model_factory
from ..registry import get_registered_optimizer_factory
from ..registry import get_registered_scheduler_factory
from ..registry import get_registered_tokenizer_factory
from ..registry import get_registered_trainer
from .base import BaseConfig
from .checkpoint import CheckpointConfig
from .data import DataConfig
from .enums import DType
from .logger import LoggerConfig
from .model import ModelConfig
from .optimizer import OptimizerConfig
from .scheduler import SchedulerConfig
from .tokenizer import TokenizerConfig
from .utils import HumanInt
from .utils import UniqueKeyLoader
from .utils import parse_human_val
from .wandb import WandBConfig

if TYPE_CHECKING:
    from ..checkpoint.engine import CheckpointEngine

TRAINER_DEFAULT = "sft"
CUSTOM_CODE_DEFAULT = Path("train.py")
_RANK_FIELDS = {"local_rank", "global_rank", "world_size"}


def _coerce_human(tree: Dict[str, Any]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for key, value in tree.items():
        if isinstance(value, dict):
            out[key] = _coerce_human(value)
        elif isinstance(value, str):
            try:
                out[key] = parse_human_val(value)
            except Exception:
                out[key] = value
        else:
            out[key] = value
    return out


class TrainerConfig(BaseConfig):
    """Base trainer configuration."""

    type: str = TRAINER_DEFAULT
    """ Trainer type. """

    code: Path = CUSTOM_CODE_DEFAULT
    """ Python file with custom trainer / factory classes (imported before validation). """

    skip_validation: bool = False
    """ Skip the check that sub-config types are compatible with the trainer. """

    model: ModelConfig
    """ Model configuration. """

    tokenizer: TokenizerConfig = Field(default_factory=TokenizerConfig)
    """ Tokenizer configuration. """

    data: DataConfig
    """ Train and eval data configuration. """

    logger: LoggerConfig = Field(default_factory=LoggerConfig)
    """ Logger configuration. """

    wandb: WandBConfig = Field(default_factory=WandBConfig)
    """ Weights and Biases configuration. """

    scheduler: SchedulerConfig = Field(default_factory=SchedulerConfig)
    """ Scheduler configuration. """

    optimizer: OptimizerConfig = Field(default_factory=OptimizerConfig)
    """ Optimizer configuration. """

    deepspeed: Dict[str, Any] = Field(default_factory=dict, alias="engine")
    """ Engine config dict (ZeRO stage, offload, precision, clipping ...); missing keys are filled in. """

    epochs: int = Field(default=1, ge=0)
    """ Number of epochs to train. """

    loss_log_interval: HumanInt = Field(default=1, ge=0)
    """ Number of steps between logging loss. """

    train_log_iter_interval: Literal[0, 1] = 1
    """ Iterations between training metric log lines (0: off). """

    train_log_metrics_path: Path = Path("train-log-metrics.jsonl")
    """ JSONL file receiving one metrics record per logged iteration. """

    gradient_accumulation_steps: int = Field(default=1, ge=1)
    """ Number of gradient accumulation steps. """

    micro_batch_size: int = Field(default=1, ge=1)
    """ Micro batch size per GPU. """

    sequence_parallel_size: int = Field(default=1, ge=1)
    """ Ulysses sequence-parallel degree (1: off). """

    expert_parallel_size: int = Field(default=1, ge=1)
    """ Expert-parallel degree (1: off). """

    arctic_moe: Union[bool, Literal["auto"]] = False
    """ Replace the model's MoE blocks by ArcticMoE (``auto``: when the architecture has experts). """

    enable_arctic_moe_custom_optimization: bool = False
    """ Use the fused CUDA routing / dispatch / combine kernels inside ArcticMoE. """

    enable_routing_replay: bool = False
    """ Re-use recorded routing decisions in MoE layers. """

    activation_checkpoint_cpu_offload: bool = False
    """ Keep per-layer activation checkpoints in pinned host memory (long sequences). """

    tiled_mlp_compute: bool = False
    """ Run MLP blocks over sequence tiles to bound activation memory. """

    seed: int = Field(default=42, ge=0)
    """ Seed for python, numpy and torch. """

    checkpoint: List[CheckpointConfig] = []
    """ Checkpoint engines; several may be used together. """

    train_iters: HumanInt = Field(default=0, ge=0)
    """ Maximum number of training iterations (0: defined by epochs). """

    eval_interval: HumanInt = Field(default=0, ge=0)
    """ Iterations between evaluations (0: never). """

    eval_log_iter_interval: HumanInt = Field(default=1, ge=0)
    """ Iterations between eval metric log lines (0: off). """

    exit_iteration: int = Field(default=0, ge=0)
    """ Stop for good after this many iterations (debugging, tests). """

    exit_iteration_this_run: int = Field(default=0, ge=0)
    """ Stop this run after this many iterations; a resumed run continues. """

    min_iterations: HumanInt = Field(default=0, ge=0)
    """ Replicate the training set until it yields this many iterations. """

    overfit_first_batch: bool = False
    """ Train on repetitions of the first batch only. """

    mem_profiler: Literal[None, "step", "e2e"] = None
    """ Record the CUDA allocator history for one step or the whole run. """

    mem_profiler_dir: Path = Field(default_factory=lambda data: data["logger"].output_dir / "mem-prof")
    """ Where memory snapshots are written. """

    mem_profiler_max_entries: HumanInt = Field(default=100_000, ge=1)
    """ Allocator events kept by the memory profiler. """

    kill_switch_path: Path = Path("/tmp/at_kill_switch")
    """ Creating this file makes training stop gracefully at the next iteration. """

    # ------------------------------------------------------------------ sub-config resolution
    @staticmethod
    def _subconfig(v: Any, info: ValidationInfo, lookup: Callable[[str], type], attr: str) -> BaseConfig:
        trainer_cls = get_registered_trainer(info.data["type"])
        hints = _get_class_attr_type_hints(trainer_cls, attr)
        fields = dict(v) if isinstance(v, dict) else v.model_dump(exclude=_RANK_FIELDS)
        chosen = lookup(fields["type"]) if fields.get("type") else hints[0]
        if not info.data.get("skip_validation") and chosen not in hints:
            raise ValueError(
                f"{chosen.__name__} is not supported for {attr} in {trainer_cls.__name__}. "
                f"Supported types are {[h.__name__ for h in hints]}."
            )
        fields["type"] = chosen.name
        config_cls = _get_class_attr_type_hints(chosen, "config")[0]
        return config_cls(**fields)

    @field_validator("checkpoint", mode="before")
    @classmethod
    def _init_checkpoint(cls, v: Any, info: ValidationInfo) -> List[CheckpointConfig]:
        items = v if isinstance(v, list) else [v]
        return [cls._subconfig(i, info, get_registered_checkpoint_engine, "checkpoint_engine") for i in items]

    @field_validator("data", mode="before")
    @classmethod
    def _init_data(cls, v: Any, info: ValidationInfo) -> DataConfig:
        return cls._subconfig(v, info, get_registered_data_factory, "data_factory")

    @field_validator("model", mode="before")
    @classmethod
    def _init_model(cls, v: Any, info: ValidationInfo) -> ModelConfig:
        return cls._subconfig(v, info, get_registered_model_factory, "model_factory")

    @field_validator("optimizer", mode="before")
    @classmethod
    def _init_optimizer(cls, v: Any, info: ValidationInfo) -> OptimizerConfig:
        return cls._subconfig(v, info, get_registered_optimizer_factory, "optimizer_factory")

    @field_validator("scheduler", mode="before")
    @classmethod
    def _init_scheduler(cls, v: Any, info: ValidationInfo) -> SchedulerConfig:
        return cls._subconfig(v, info, get_registered_scheduler_factory, "scheduler_factory")

    @field_validator("tokenizer", mode="before")
    @classmethod
    def _init_tokenizer(cls, v: Any, info: ValidationInfo) -> TokenizerConfig:
        return cls._subconfig(v, info, get_registered_tokenizer_factory, "tokenizer_factory")

    @field_validator("logger", mode="after")
    @classmethod
    def _init_logger(cls, v: LoggerConfig) -> LoggerConfig:
        from ..logging import setup_logger

        setup_logger(v)
        return v

    @field_validator("deepspeed", mode="before")
    @classmethod
    def _human_numbers_in_engine_dict(cls, v: Dict[str, Any]) -> Dict[str, Any]:
        return _coerce_human(v or {})

    # ------------------------------------------------------------------ whole-model validation
    @model_validator(mode="after")
    def _set_max_length(self) -> Self:
        if "max_length" not in self.data.model_fields_set:
            from ..models.arch import load_arch_config

            arch = load_arch_config(self.model.name_or_path, self.model.hf_config_kwargs)
            if arch.get("max_position_embeddings") is None:
                raise ValueError(
                    f"Model config for {self.model.name_or_path} has no `max_position_embeddings`. "
                    "Set `data.max_length` in your config."
                )
            self.data.max_length = int(arch["max_position_embeddings"])
        return self

    @model_validator(mode="after")
    def _init_dist(self) -> Self:
        from ..comm.dist import init_distributed

        init_distributed(local_rank=self.local_rank)
        return self

    @model_validator(mode="after")
    def _check_eval_interval(self) -> Self:
        has_eval = (bool(self.data.eval_sources) or self.data.train_eval_split[1] > 0.0
                    or bool(getattr(self.data, "eval_root_directories", None)))  # pre-batched evaluation directories
        if has_eval:
            assert self.eval_interval > 0, "`eval_interval` must be set if eval dataset is provided."
        if self.eval_interval > 0:
            assert has_eval, "`eval_interval` must be set only if eval dataset is provided."
        return self

    @model_validator(mode="after")
    def _default_tokenizer_path(self) -> Self:
        if not self.tokenizer.name_or_path:
            self.tokenizer.name_or_path = self.model.name_or_path
        return self

    @model_validator(mode="after")
    def _build_engine_config(self) -> Self:
        from ..models.arch import load_arch_config

        cfg = self.deepspeed
        cfg["train_micro_batch_size_per_gpu"] = self.micro_batch_size
        cfg["train_batch_size"] = (
            self.micro_batch_size * self.gradient_accumulation_steps * self.world_size / self.sequence_parallel_size
        )
        cfg["gradient_accumulation_steps"] = self.gradient_accumulation_steps
        cfg["sequence_parallel_size"] = self.sequence_parallel_size
        cfg.setdefault("steps_per_print", 10)
        if "zero_optimization" in cfg:
            hidden = 0  # only the defaults below depend on the model's width
        else:
            arch = load_arch_config(self.model.name_or_path, self.model.hf_config_kwargs)
            hidden = arch.get("hidden_size") or max(arch.get("hidden_sizes") or [0])
            if not hidden:
                raise ValueError(f"Cannot find `hidden_size` in the config of {self.model.name_or_path}")
        cfg.setdefault(
            "zero_optimization",
            {
                "stage": 2,
                "stage3_param_persistence_threshold": 10 * hidden,
                "stage3_max_live_parameters": 2 * hidden * hidden,
                "stage3_prefetch_bucket_size": int(0.9 * hidden * hidden),
                "reduce_bucket_size": hidden * hidden,
            },
        )
        if "bf16" in cfg and "bfloat16" not in cfg:
            cfg["bfloat16"] = cfg["bf16"]
        if "bfloat16" not in cfg and self.model.dtype == DType.BF16.value:
            cfg["bfloat16"] = {"enabled": True}
        if "fp16" not in cfg and self.model.dtype == DType.FP16.value:
            cfg["fp16"] = {"enabled": True}
        cfg.setdefault("gradient_clipping", 1.0)
        cfg.setdefault("prescale_gradients", False)
        cfg.setdefault("wall_clock_breakdown", False)
        return self

    @model_validator(mode="after")
    def _one_resume_engine(self) -> Self:
        assert sum(c.auto_resume for c in self.checkpoint) <= 1, "Only one checkpoint can auto resume."
        return self

    @model_validator(mode="after")
    def _prepare_paths(self) -> Self:
        if self.local_rank == 0:
            self.train_log_metrics_path.parent.mkdir(parents=True, exist_ok=True)
            self.train_log_metrics_path.open(mode="a").close()
        if self.mem_profiler is not None:
            self.mem_profiler_dir.mkdir(parents=True, exist_ok=True)
        return self

    @model_validator(mode="after")
    def _packing_needs_mbs_one(self) -> Self:
        if getattr(self.data, "pack_samples", False):
            assert self.micro_batch_size == 1, "`micro_batch_size` must be 1 if `pack_samples` is enabled."
        return self

    # ------------------------------------------------------------------ conveniences
    @property
    def checkpoint_engines(self) -> List[Callable[..., "CheckpointEngine"]]:
        return [partial(get_registered_checkpoint_engine(c.type), config=c) for c in self.checkpoint]

    @property
    def zero_stage(self) -> int:
        return int(self.deepspeed.get("zero_optimization", {}).get("stage", 0))

    @property
    def zero_3_enabled(self) -> bool:
        return self.zero_stage == 3


def load_user_module_from_path(script_path: Path) -> None:
    """Import a user's ``train.py`` so the classes it declares register themselves.

    The script's directory is linked under a private temp directory with a stable unique name and that
    link is put on ``sys.path``: sibling imports inside the script keep working and two recipes whose
    scripts share a file name do not clash.
    """
    script_path = Path(script_path).resolve()
    if not script_path.exists():
        raise FileNotFoundError(f"Cannot import custom code from {script_path}: no such file.")
    link_root = Path(tempfile.gettempdir()) / "atb200_user_modules"
    link_root.mkdir(parents=True, exist_ok=True)
    link_name = "m" + uuid.uuid5(uuid.NAMESPACE_URL, str(script_path.parent)).hex
    link = link_root / link_name
    if not link.exists():
        try:
            link.symlink_to(script_path.parent, target_is_directory=True)
        except FileExistsError:
            pass
    for p in (str(link), str(script_path.parent)):
        if p not in sys.path:
            sys.path.insert(0, p)
    mod_name = f"{link_name}.{script_path.stem}"
    if mod_name in sys.modules:
        return
    # the same file may already be loaded under another name (one project's script importing a sibling project's):
    # executing it again would declare, and try to register, its classes a second time
    for loaded in list(sys.modules.values()):
        f = getattr(loaded, "__file__", None)
        if f and Path(f).resolve() == script_path:
            sys.modules[mod_name] = loaded
            return
    spec = importlib.util.spec_from_file_location(mod_name, link / script_path.name)
    assert spec is not None and spec.loader is not None
    module = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = module
    spec.loader.exec_module(module)


def get_config(config_file_or_dict: Union[Path, str, Dict[str, Any]]) -> TrainerConfig:
    """Build the validated config of a recipe given as a YAML path or as a dict."""
    if isinstance(config_file_or_dict, dict):
        raw = dict(config_file_or_dict)
        config_dir = Path.cwd()
    else:
        path = Path(config_file_or_dict)
        with open(path) as fh:
            raw = yaml.load(fh, Loader=UniqueKeyLoader) or {}
        config_dir = path.parent
    code = Path(raw.get("code", CUSTOM_CODE_DEFAULT))
    if not code.is_absolute():
        code = config_dir / code
    code = code.resolve()
    if code.exists():
        raw["code"] = code
        load_user_module_from_path(code)
    elif raw.get("code") is not None:
        raise FileNotFoundError(f"Cannot find custom code file {code}")
    raw["type"] = raw.get("type", TRAINER_DEFAULT)
    trainer_cls = get_registered_trainer(raw["type"])
    config_cls = _get_class_attr_type_hints(trainer_cls, "config")[0]
    return config_cls(**raw)
