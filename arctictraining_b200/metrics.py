# SPDX-License-Identifier: Apache-2.0
"""Per-iteration metrics: loss, iteration / step time, tflops, sequence length, learning rate.

Behaviour parity: arctic_training/metrics.py:35-201 — one value per key per iteration (writing a key
twice raises), the console line format, the summary dict written to the JSONL log, loss averaging over
gradient-accumulation steps, tflos divided by the sequence-parallel degree.  The cross-rank reduction is
a single all-reduce of a small stats vector instead of several pickled object gathers per iteration, and
the timers are device timers.
"""

from __future__ import annotations

from collections import defaultdict
from typing import TYPE_CHECKING
from typing import Dict
from typing import List
from typing import Optional
from typing import Union

import torch
import torch.distributed as dist

from .debug.utils import get_mem_metrics
from .engine.timers import DeviceTimer
from .flops import estimate_decoder_transformer_tflos
from .utils.misc import human_format_base10_number
from .utils.misc import human_format_secs

if TYPE_CHECKING:
    from .trainer.trainer import Trainer

_KEYS = ("loss", "loss/eval", "iter_time", "step_time", "seqlen_total", "tflos")


def gather_object(value, world_size: int) -> List[Union[float, int]]:
    if world_size == 1 or not dist.is_initialized():
        out = [value]
    else:
        out = [None] * world_size
        dist.all_gather_object(out, value)
    return [v for item in out for v in (item if isinstance(item, list) else [item])]


class Metrics:
    def __init__(self, trainer: "Trainer") -> None:
        self.enabled = trainer.config.train_log_iter_interval > 0
        if not self.enabled:
            return
        self.trainer = trainer
        self.summary_dict: Dict[str, Union[int, float]] = {}
        self.timers: Dict[str, DeviceTimer] = {}
        self.values: Dict[str, Union[int, float]] = defaultdict(float)
        self.seqlens: Optional[List[List[int]]] = None
        self.losses: List[float] = []
        module = trainer.model_unwrapped
        self.model_size = module.num_parameters() if hasattr(module, "num_parameters") else sum(
            getattr(p, "_atb_numel", p.numel()) for p in module.parameters()
        )
        self.model_config = getattr(module, "config", {})
        horizon = trainer.training_horizon
        exit_it = trainer.config.exit_iteration
        self.max_iter = min(exit_it, horizon) if exit_it > 0 else horizon
        self.max_iter_pad = len(str(self.max_iter))

    # ------------------------------------------------------------------ recording
    def record(self, key: str, value: Union[int, float]) -> None:
        if not self.enabled:
            return
        if key in self.values:
            raise KeyError(
                f"Key {key} already exists: a value was written twice before being reported "
                "(one value per key and training iteration)."
            )
        self.values[key] = value

    def start_timer(self, key: str) -> None:
        if not self.enabled:
            return
        self.timers.setdefault(key, DeviceTimer(key)).start()

    def stop_timer(self, key: str) -> None:
        if not self.enabled:
            return
        if key not in self.timers:
            raise KeyError(f"Timer {key} not started")
        self.timers[key].stop()
        self.values[f"{key}_time"] = self.timers[key].elapsed() / 1000.0

    def restart_timer(self, key: str) -> None:
        self.stop_timer(key)
        self.start_timer(key)

    def get_value(self, key: str) -> Union[int, float]:
        return self.values[key]

    # ------------------------------------------------------------------ reporting
    def _reduce(self) -> Dict[str, float]:
        """Sum every known stat over all ranks with one all-reduce; returns {key: (sum, count)}."""
        tr = self.trainer
        vec = torch.zeros(2 * len(_KEYS), dtype=torch.float64)
        for i, k in enumerate(_KEYS):
            if k in self.values:
                vec[2 * i] = float(self.values[k])
                vec[2 * i + 1] = 1.0
        if tr.world_size > 1 and dist.is_initialized():
            dev = tr.device if dist.get_backend() == "nccl" else torch.device("cpu")
            vec = vec.to(dev)
            dist.all_reduce(vec)
            vec = vec.cpu()
        return {k: (float(vec[2 * i]), float(vec[2 * i + 1])) for i, k in enumerate(_KEYS) if vec[2 * i + 1] > 0}

    def print_summary(self, prefix: str = "train") -> None:
        if not self.enabled:
            return
        tr = self.trainer
        s = self.summary_dict
        s.clear()
        s["epoch"] = tr.epoch_idx
        s["iter"] = tr.global_step
        sched = getattr(tr.model, "lr_scheduler", None)
        s["lr"] = sched.get_last_lr()[0] if sched is not None else tr.model.get_lr()[0]

        if self.seqlens is not None:
            tflos, seqlen = estimate_decoder_transformer_tflos(
                self.model_config, self.model_size, self.seqlens,
                enable_gradient_checkpointing=not tr.config.model.disable_activation_checkpoint,
            )
            self.values["tflos"] = tflos
            self.values["seqlen_total"] = seqlen
        red = self._reduce()
        world = tr.world_size
        tflos_total = red.get("tflos", (0.0, 0))[0] / tr.config.sequence_parallel_size

        if "loss" in red:
            loss = red["loss"][0] / red["loss"][1]
            s["loss"] = loss
            gas = tr.config.gradient_accumulation_steps
            if gas > 1:
                self.losses.append(loss)
                if len(self.losses) == gas:
                    s["loss"] = sum(self.losses) / gas
                    self.losses = []
        if "loss/eval" in red:
            s["loss/eval"] = red["loss/eval"][0] / red["loss/eval"][1]
        if "iter_time" in red:
            total = red["iter_time"][0]
            s["iter_time"] = total / world
            if tflos_total > 0 and total > 0:
                s["iter_tflops"] = tflos_total / total
        if "seqlen_total" in red:
            s["seqlen"] = red["seqlen_total"][0] / world
        if "step_time" in red:
            total = red["step_time"][0]
            s["step_time"] = total / world
            if tflos_total > 0 and total > 0:
                s["step_tflops"] = tflos_total / total
        self.values.clear()

        line = (
            f"{prefix.title():>{len('train')}} iter: {s['iter']:>{self.max_iter_pad}}/{self.max_iter}"
            f" {100 * s['iter'] // max(self.max_iter, 1):>3}%"
        )
        if "loss" in s:
            line += f" | loss: {s['loss']:.4f}"
        if "loss/eval" in s:
            # an evaluation loss that was recorded but not yet reported (eval_log_iter_interval > eval_interval) rides
            # along on the next training line: name it
            line += f" | {'eval loss' if 'loss' in s else 'loss'}: {s['loss/eval']:.4f}"
        if "iter_time" in s:
            line += f" | iter time: {human_format_secs(s['iter_time'])}"
        if "iter_tflops" in s:
            line += f" | iter tflops: {s['iter_tflops']:.1f}"
        line += f" | lr: {s['lr']:.3E}"
        if "seqlen" in s:
            line += f" | seqlen: {human_format_base10_number(s['seqlen'])}"
        if "step_time" in s:
            line += f" | step time: {human_format_secs(s['step_time'])}"
        if "step_tflops" in s:
            line += f" | step tflops: {s['step_tflops']:.1f}"
        line += f" | epoch: {s['epoch']}"
        if tr.global_rank == 0:
            print(line + f" | {get_mem_metrics()}", flush=True)
