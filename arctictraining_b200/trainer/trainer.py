# SPDX-License-Identifier: Apache-2.0
"""Base trainer: owns the whole lifecycle of a run.

Behaviour parity: arctic_training/trainer/trainer.py:68-771.  Construction order: seeds -> tokenizer ->
data -> checkpoint engines (resume detection) -> parallel groups / sequence parallelism -> model ->
(ArcticMoE) -> optimizer -> scheduler -> engine -> sequence-parallel dataloader adapter -> auto resume ->
metrics -> wandb.  Loop: ``train()`` -> ``epoch()`` -> ``step()`` -> ``loss()`` / ``backward()`` /
``engine.step()`` / ``checkpoint()``; all of these are callback-wrapped.  Early exit on ``exit_iteration``,
``exit_iteration_this_run``, the kill-switch file or the training horizon; a resumed run skips the batches it
already consumed in the current epoch.
"""

from __future__ import annotations

import math
import random
from abc import ABC
from abc import abstractmethod
from collections import defaultdict
from functools import cached_property
from typing import Any
from typing import Callable
from typing import Dict
from typing import List
from typing import Optional
from typing import Tuple

import numpy as np
import torch
from tqdm import tqdm

from ..callback.logging import post_loss_log_cb
from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..checkpoint.engine import CheckpointEngine
from ..config.trainer import TrainerConfig
from ..data.factory import DataFactory
from ..data.utils import OverfitOneBatchDataLoader
from ..debug.utils import see_memory_usage
from ..engine import TrainingEngine
from ..logging import logger
from ..metrics import Metrics
from ..models.factory import ModelFactory
from ..optimizer.factory import OptimizerFactory
from ..parallel.mesh import ParallelGroups
from ..parallel.ulysses import UlyssesContext
from ..parallel.ulysses import UlyssesDataLoaderAdapter
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from ..scheduler.factory import SchedulerFactory
from ..tokenizer.factory import TokenizerFactory
from ..utils.misc import append_json_file


class Trainer(ABC, CallbackMixin, metaclass=RegistryMeta):
    supports_sequence_parallel = False
    """ Whether ``loss`` works on a rank's slice of the sequence (``shift_labels``, group-wide loss aggregation). """

    name: str
    """ Name under which the trainer is selected in a recipe (``type``). """

    config: TrainerConfig
    """ Config class of the trainer (a ``TrainerConfig`` subclass may add fields). """

    data_factory: DataFactory
    """ Compatible data factory types; the first is the default. """

    model_factory: ModelFactory
    """ Compatible model factory types; the first is the default. """

    checkpoint_engine: CheckpointEngine
    """ Compatible checkpoint engine types; the first is the default. """

    optimizer_factory: OptimizerFactory
    """ Compatible optimizer factory types; the first is the default. """

    scheduler_factory: SchedulerFactory
    """ Compatible scheduler factory types; the first is the default. """

    tokenizer_factory: TokenizerFactory
    """ Compatible tokenizer factory types; the first is the default. """

    callbacks: List[Tuple[str, Callable]] = [post_loss_log_cb]
    """ ``(event, fn)`` callbacks; events are ``pre-``/``post-`` + init, train, epoch, step, loss, backward,
    evaluate, checkpoint. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", TrainerConfig)
        _validate_class_attribute_type(cls, "data_factory", DataFactory)
        _validate_class_attribute_type(cls, "model_factory", ModelFactory)
        _validate_class_attribute_type(cls, "checkpoint_engine", CheckpointEngine)
        _validate_class_attribute_type(cls, "optimizer_factory", OptimizerFactory)
        _validate_class_attribute_type(cls, "scheduler_factory", SchedulerFactory)
        _validate_class_attribute_type(cls, "tokenizer_factory", TokenizerFactory)
        _validate_class_method(cls, "loss", ["self", "batch"])
        _validate_class_method(cls, "step", ["self", "batch"])
        _validate_class_method(cls, "epoch", ["self"])
        _validate_class_method(cls, "train", ["self"])
        _validate_class_method(cls, "checkpoint", ["self"])

    # ================================================================== construction
    def __init__(self, config: TrainerConfig, mode: str = "train") -> None:
        self.config = config
        self.epoch_idx = 0
        self.train_batch_idx = 0
        self.global_step = 0
        self.global_step_this_run = 0
        self.global_step_at_start_this_run = 0
        self.early_stop = False
        self.early_stop_reason = ""
        self.world_size = config.world_size
        self.global_rank = config.global_rank
        self.epoch_finished = False
        self.training_finished = False
        self.wandb_experiment = None
        self.is_resume = False
        self.wandb_run_id: Optional[str] = None
        self.gas_boundary = True
        self.sp_context: Optional[UlyssesContext] = None

        self._set_seeds(config.seed)
        if config.mem_profiler == "e2e" and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=config.mem_profiler_max_entries)

        self.tokenizer = config.tokenizer.factory(self)()
        self.train_dataloader, self.eval_dataloader = config.data.factory(self)()
        if mode == "process-data":
            return
        if config.overfit_first_batch:
            self.train_dataloader = OverfitOneBatchDataLoader(self.train_dataloader)

        self.checkpoint_engines = [make(self) for make in config.checkpoint_engines]
        for eng in self.checkpoint_engines:
            if eng.name == "deepspeed" and eng.config.auto_resume and eng.latest_checkpoint_exists:
                self.is_resume = True

        if config.sequence_parallel_size > 1 and not self.supports_sequence_parallel:
            raise ValueError(
                f"trainer '{self.name}' computes its loss over whole sequences and does not support "
                f"sequence_parallel_size={config.sequence_parallel_size}; sequence parallelism is available for the "
                "sft / causal trainers and those derived from them that handle `shift_labels` (swiftkv, moba)"
            )
        self.groups = ParallelGroups(config.sequence_parallel_size, config.expert_parallel_size)
        if config.sequence_parallel_size > 1:
            self.sp_group = self.groups.sp_group
            self.sp_world_size = self.groups.sp_size
            self.sp_rank = self.groups.sp_rank
            self.sp_context = UlyssesContext(self.sp_group, self.sp_world_size, self.sp_rank)

        self.model = config.model.factory(self)()
        self._configure_model(self.model)
        self.original_model_params = self._count_params(self.model)

        self.use_arctic_moe = self._resolve_arctic_moe()
        if config.expert_parallel_size > 1 and not self.use_arctic_moe:
            raise ValueError(
                f"expert_parallel_size={config.expert_parallel_size} needs a mixture-of-experts model run as ArcticMoE "
                "(`arctic_moe: true` or `auto`); this model has no experts to distribute"
            )
        if self.use_arctic_moe:
            from ..moe.convert import convert_hf_blocks_to_arctic_moe
            from ..moe.convert import convert_to_arctic_moe

            # a model of the ``transformers`` fallback (e.g. Qwen3-Next) still carries the library's sparse blocks
            replaced = convert_hf_blocks_to_arctic_moe(self.model, self.groups)
            if replaced:
                logger.info(f"replaced {replaced} transformers sparse MoE blocks by ArcticMoE")
            convert_to_arctic_moe(
                self.model, self.groups, is_resume=self.is_resume,
                use_fused_kernels=config.enable_arctic_moe_custom_optimization,
                routing_replay=config.enable_routing_replay,
            )
        see_memory_usage("after model creation", force=False)

        self.optimizer = config.optimizer.factory(self)()
        self.scheduler = config.scheduler.factory(self)()
        self.model = self._create_engine(self.model, self.optimizer, self.scheduler)
        self.ds_wall_clock_available = hasattr(self.model, "get_wall_clock_timers")
        if self.use_arctic_moe and self.ds_wall_clock_available and self.model.wall_clock_breakdown():
            from ..moe.timers import enable_moe_timers

            enable_moe_timers(self.model_unwrapped)

        if config.sequence_parallel_size > 1:
            self.train_dataloader = UlyssesDataLoaderAdapter(
                self.train_dataloader, self.sp_rank, self.sp_group, self.sp_world_size, self.device
            )
            if self.eval_dataloader is not None:
                self.eval_dataloader = UlyssesDataLoaderAdapter(
                    self.eval_dataloader, self.sp_rank, self.sp_group, self.sp_world_size, self.device
                )

        for eng in self.checkpoint_engines:
            if eng.config.auto_resume:
                eng.load(self.model)

        self.metrics = Metrics(self)
        self._init_wandb()

    def _configure_model(self, model: torch.nn.Module) -> None:
        """Hand run-time switches of the recipe to a native model."""
        if hasattr(model, "sp_context"):
            model.sp_context = self.sp_context
        elif self.config.sequence_parallel_size > 1:
            # a model of the transformers library: its attention calls go through a registered function that does the
            # sequence <-> head exchange around the core attention
            from ..parallel.ulysses_hf import enable_ulysses_for_hf_model

            self.hf_ulysses = enable_ulysses_for_hf_model(model, self.sp_context, self.config.model.attn_implementation)
        if hasattr(model, "tiled_mlp"):
            model.tiled_mlp = self.config.tiled_mlp_compute
        elif self.config.tiled_mlp_compute:
            from ..ops.tiled import enable_tiled_mlp_compute

            enable_tiled_mlp_compute(model)

    def _create_engine(self, model, optimizer, scheduler, training: bool = True) -> TrainingEngine:
        cfg = dict(self.config.deepspeed)
        cfg["activation_checkpoint_cpu_offload"] = self.config.activation_checkpoint_cpu_offload
        expert_dp = self.groups.expert_dp_group if self.groups.ep_size > 1 else None
        engine = TrainingEngine(
            model, optimizer, scheduler, cfg,
            expert_dp_group=expert_dp,
            is_expert_param=lambda n, p: bool(getattr(p, "is_expert_param", False)) and self.groups.ep_size > 1,
            training=training,
        )
        engine.ep_group = self.groups.ep_group
        return engine

    def _resolve_arctic_moe(self) -> bool:
        flag = self.config.arctic_moe
        if flag == "auto":
            cfg = getattr(self.model, "config", {})
            get = cfg.get if isinstance(cfg, dict) else (lambda k, d=None: getattr(cfg, k, d))
            return bool(get("num_experts") or get("num_local_experts") or get("n_routed_experts"))
        return bool(flag)

    def _config_for_logging(self) -> dict:
        """The recipe as plain JSON types (enum members with non-JSON values, e.g. ``torch.dtype``, become strings)."""
        try:
            return self.config.model_dump(mode="json", fallback=str)
        except TypeError:  # pydantic without the ``fallback`` argument
            import json

            return json.loads(json.dumps(self.config.model_dump(), default=str))

    def _init_wandb(self) -> None:
        if self.global_rank != 0 or not self.config.wandb.enable:
            return
        import wandb

        if self.wandb_run_id is None:
            self.wandb_run_id = wandb.util.generate_id()
        self.wandb_experiment = wandb.init(
            id=self.wandb_run_id, entity=self.config.wandb.entity, project=self.config.wandb.project,
            name=self.config.wandb.name, config=self._config_for_logging(),
            dir=f"{self.config.logger.output_dir}/wandb", resume="allow",
        )

    def _set_seeds(self, seed: int) -> None:
        torch.manual_seed(seed)
        np.random.seed(seed)
        random.seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    @staticmethod
    def _count_params(model: torch.nn.Module) -> Dict[str, int]:
        sizes: Dict[str, int] = defaultdict(int)
        seen = set()
        for p in model.parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            n = getattr(p, "_atb_numel", p.numel())  # released ZeRO-3 parameters are empty views: use the logical size
            sizes["total"] += n
            if p.requires_grad:
                sizes["trainable"] += n
        return dict(sizes)

    # ================================================================== accessors
    @property
    def model_unwrapped(self) -> torch.nn.Module:
        return self.model.module if hasattr(self.model, "module") else self.model

    @cached_property
    def device(self) -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", self.config.local_rank % torch.cuda.device_count())
        return torch.device("cpu")

    @property
    def _quiet_bars(self) -> bool:
        return self.global_rank != 0 or self.config.train_log_iter_interval != 0

    @property
    def epochs(self):
        total = self.config.epochs
        if self.config.train_iters:
            total = math.ceil(self.config.train_iters * self.config.gradient_accumulation_steps / len(self.train_dataloader))
        return tqdm(range(self.epoch_idx, total), desc="Epochs", unit="epoch", disable=self._quiet_bars)

    @property
    def train_batches(self):
        return tqdm(self.train_dataloader, desc="Train Batches", unit="batch", disable=self._quiet_bars)

    @property
    def eval_batches(self):
        return tqdm(self.eval_dataloader, desc="Eval Batches", unit="batch",
                    disable=self.global_rank != 0 or not self.is_eval_log_iter())

    def is_eval_log_iter(self) -> bool:
        every = self.config.eval_log_iter_interval
        return bool(every) and self.global_step // self.config.eval_interval % every == 0

    @property
    def training_horizon(self) -> int:
        if self.train_dataloader is None:
            raise ValueError("Train dataloader not initialized.")
        if self.config.train_iters:
            return self.config.train_iters
        return self.config.epochs * len(self.train_dataloader)

    # ================================================================== the loop
    @callback_wrapper("loss")
    @abstractmethod
    def loss(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError("Loss method must be implemented by the trainer.")

    @callback_wrapper("backward")
    def backward(self, loss: torch.Tensor) -> None:
        self.model.backward(loss)

    def need_early_exit(self) -> bool:
        c = self.config
        if c.exit_iteration_this_run > 0 and c.exit_iteration_this_run == self.global_step_this_run:
            self.early_stop_reason = f"reached exit_iteration_this_run of {self.global_step_this_run}"
        elif c.exit_iteration > 0 and c.exit_iteration == self.global_step:
            self.early_stop_reason = f"reached exit_iteration of {self.global_step}"
        elif c.kill_switch_path.exists():
            self.early_stop_reason = f"detected kill switch {c.kill_switch_path}"
        elif self.global_step >= self.training_horizon:
            self.early_stop_reason = f"reached training_horizon of {self.global_step}"
        else:
            return False
        return True

    @callback_wrapper("step")
    def step(self, batch: Dict[str, torch.Tensor]) -> None:
        self.model.train()
        with self.model.autocast():
            loss = self.loss(batch)
        self.backward(loss)
        self.metrics.record("loss", loss.item() if torch.is_tensor(loss) else loss)
        self.model.step()  # reads the kernels' error words (bounded waits, expert-buffer overflow) before the update
        self.checkpoint()
        self.global_step = self.model.global_steps
        self.global_step_this_run = self.global_step - self.global_step_at_start_this_run

    def _sample_seqlens(self, batch: Dict[str, Any]) -> List[List[int]]:
        if "packed_sample_seqlens" in batch:
            seqlens = batch.pop("packed_sample_seqlens")
            if self.config.model.attn_implementation != "eager" and self.config.sequence_parallel_size == 1:
                return [list(s) for s in seqlens]
            if self.config.sequence_parallel_size > 1:
                return [list(s) for s in seqlens]
        n = self.config.sequence_parallel_size
        return [[len(row) * n] for row in batch["input_ids"]]

    @callback_wrapper("epoch")
    def epoch(self) -> None:
        self.epoch_finished = False
        self.metrics.start_timer("iter")
        if self.config.mem_profiler == "step" and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=self.config.mem_profiler_max_entries)

        it = iter(self.train_batches)
        if self.is_resume:
            skip = self.global_step % len(self.train_dataloader)
            logger.info(f"Resumed from checkpoint at global step {self.global_step}; advancing {skip} batches.")
            for _ in range(skip):
                next(it)
            self.train_batch_idx += skip
            self.is_resume = False

        for batch in it:
            self.train_batch_idx += 1
            if self.need_early_exit():
                self.early_stop = True
                break
            self.gas_boundary = self.train_batch_idx % self.config.gradient_accumulation_steps == 0
            self.metrics.seqlens = self._sample_seqlens(batch)

            self.metrics.start_timer("step")
            self.step(batch)
            self.metrics.stop_timer("step")
            self.metrics.restart_timer("iter")

            if self.config.train_log_iter_interval != 0:
                self.metrics.print_summary()
            if not self.gas_boundary:
                continue
            if (self.global_rank == 0 and self.config.train_log_iter_interval != 0
                    and self.global_step % self.config.train_log_iter_interval == 0):
                record = dict(self.metrics.summary_dict)
                if self.ds_wall_clock_available and self.model.wall_clock_breakdown():
                    record.update(self.model.get_wall_clock_timers().snapshot())
                    if self.use_arctic_moe:
                        from ..moe.timers import format_breakdown
                        from ..moe.timers import forward_breakdown

                        moe_times = forward_breakdown(self.model_unwrapped)
                        if moe_times:
                            logger.info(format_breakdown(moe_times))
                            record.update({f"amoe/{k}": v for k, v in moe_times.items()})
                append_json_file(self.config.train_log_metrics_path, record)
                if self.wandb_experiment is not None and self.global_step > 1:
                    self.wandb_experiment.log({k: v for k, v in record.items() if k != "iter"}, step=self.global_step)
            if self.config.eval_interval != 0 and self.global_step % self.config.eval_interval == 0:
                self.evaluate()
                if self.is_eval_log_iter():
                    self.metrics.print_summary(prefix="eval")
                    if self.wandb_experiment is not None:
                        self.wandb_experiment.log({"loss/eval": self.metrics.summary_dict["loss/eval"]}, step=self.global_step)

        self.metrics.stop_timer("iter")
        self.epoch_finished = True

    @callback_wrapper("train")
    def train(self) -> None:
        self.print_model_parameters_header()
        try:
            self.global_step_at_start_this_run = self.global_step
            for epoch_idx in self.epochs:
                self.epoch_idx = epoch_idx
                self.epoch()
                if self.early_stop:
                    break
                self.checkpoint()
            self.training_finished = True
            if self.global_rank == 0:
                if self.early_stop:
                    print(f"*** Exiting training early because training {self.early_stop_reason}", flush=True)
                else:
                    print("*** Training finished normally.", flush=True)
            self.checkpoint()
        except Exception as exc:
            logger.error(f"Training failed with error: {exc}")
            raise
        finally:
            if self.config.mem_profiler is not None and torch.cuda.is_available():
                torch.cuda.memory._dump_snapshot(str(self.config.mem_profiler_dir / f"{self.global_rank}.pickle"))
            if self.wandb_experiment is not None:
                self.wandb_experiment.finish()

    @callback_wrapper("evaluate")
    def evaluate(self) -> None:
        self.model.eval()
        with torch.no_grad():
            losses = []
            for batch in self.eval_batches:
                batch.pop("packed_sample_seqlens", None)
                losses.append(float(self.loss(batch)))
        self.metrics.record("loss/eval", sum(losses) / max(1, len(losses)))
        self.model.train()

    @callback_wrapper("checkpoint")
    def checkpoint(self) -> None:
        if self.global_step_this_run == 0:
            return
        for eng in self.checkpoint_engines:
            if not eng.do_checkpoint:
                continue
            if eng.name == "huggingface" and self.use_arctic_moe and not self.training_finished:
                raise ValueError(
                    "Hugging Face export of ArcticMoE models is only supported at the end of training; use the "
                    "`deepspeed` checkpoint type for intermediate checkpoints."
                )
            logger.info(f"Saving checkpoint at global step {self.global_step}.")
            eng.save(self.model)

    # ================================================================== reporting
    def count_model_parameters(self) -> Dict[str, int]:
        return self._count_params(self.model_unwrapped)

    def print_model_parameters_header(self) -> None:
        if self.global_rank != 0:
            return
        sizes = self.count_model_parameters()
        total, trainable = sizes.get("total", 0), sizes.get("trainable", 0)
        print(
            f"Model parameters: total {total / 1e9:.3f}B, trainable {trainable / 1e9:.3f}B "
            f"({100.0 * trainable / max(total, 1):.2f}%) | world {self.world_size} | "
            f"ZeRO stage {self.model.zero_optimization_stage()} | SP {self.config.sequence_parallel_size} | "
            f"EP {self.config.expert_parallel_size}",
            flush=True,
        )
