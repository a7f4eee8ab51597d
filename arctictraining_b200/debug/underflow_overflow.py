# SPDX-License-Identifier: Apache-2.0
"""Numeric tracers: find where activations or gradients first become inf / nan, or drift towards the limits of the
training dtype.  Behaviour parity: arctic_training/debug/underflow_overflow.py:48-540 (forward-hook tracer that keeps
the last frames with absolute min / max of inputs, outputs and weights and aborts on inf/nan; backward-hook tracer
for gradients; optional tracing of selected batch numbers).
"""

from __future__ import annotations

import collections
from typing import Any
from typing import Deque
from typing import List
from typing import Optional

import torch
import torch.nn as nn


def get_abs_min_max(var: torch.Tensor, ctx: str) -> str:
    a = var.detach().abs().float()
    return f"{a.min().item():8.2e} {a.max().item():8.2e} {ctx}"


def detect_overflow(var: torch.Tensor, ctx: str) -> bool:
    """True (and a printed note) when ``var`` holds nan or inf."""
    bad = False
    if torch.isnan(var).any().item():
        bad = True
        print(f"{ctx} has nans")
    if torch.isinf(var).any().item():
        bad = True
        print(f"{ctx} has infs")
    return bad


class DebugUnderflowOverflow:
    """Registers forward hooks on every sub-module of ``model``.

    Mode 1 (default): keep the reports of the last ``max_frames_to_save`` module calls and, when an inf/nan shows up,
    print them and raise ``ValueError``.  Mode 2 (``trace_batch_nums``): print every frame of the listed batches.
    ``abort_after_batch_num`` stops the run after that batch.
    """

    def __init__(self, model: nn.Module, max_frames_to_save: int = 21, trace_batch_nums: Optional[List[int]] = None,
                 abort_after_batch_num: Optional[int] = None) -> None:
        self.model = model
        self.trace_batch_nums = trace_batch_nums or []
        self.abort_after_batch_num = abort_after_batch_num
        self.frames: Deque[str] = collections.deque([], max_frames_to_save)
        self.frame: List[str] = []
        self.batch_number = 0
        self.total_calls = 0
        self.detected_overflow = False
        self.prefix = "                 "
        self.module_names = {m: n for n, m in model.named_modules()}
        self.handles = [m.register_forward_hook(self._forward_hook) for m in model.modules()]

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []

    def _expand(self, line: str) -> None:
        self.frame.append(line)

    def _analyse(self, var: Any, ctx: str) -> None:
        if torch.is_tensor(var) and var.numel() > 0 and var.is_floating_point():
            self._expand(get_abs_min_max(var, ctx))
            if detect_overflow(var, ctx):
                self.detected_overflow = True
        elif isinstance(var, (tuple, list)):
            for i, x in enumerate(var):
                self._analyse(x, f"{ctx}[{i}]")
        elif var is None:
            self._expand(f"{'None':>17} {ctx}")

    def _forward_hook(self, module: nn.Module, inputs: Any, output: Any) -> None:
        is_root = module is self.model
        last_frame_of_batch = is_root
        trace = self.batch_number in self.trace_batch_nums
        self.frame = [f"{self.prefix} {self.module_names.get(module, '?')} {module.__class__.__name__}"]
        for name, p in module.named_parameters(recurse=False):
            self._analyse(p, name)
        self._analyse(inputs, "input")
        self._analyse(output, "output")
        self.frames.append("\n".join(self.frame))
        self.total_calls += 1
        if trace:
            print("\n".join(self.frame))
        if self.detected_overflow and not trace:
            report = "\n\n".join(self.frames)
            self.frames.clear()
            raise ValueError(
                "DebugUnderflowOverflow: inf/nan detected, aborting after "
                f"batch {self.batch_number}. Last {len(report.split(chr(10) * 2))} frames "
                f"(abs min, abs max, name):\n{report}"
            )
        if last_frame_of_batch:
            self.batch_number += 1
            if self.abort_after_batch_num is not None and self.batch_number > self.abort_after_batch_num:
                raise ValueError(f"DebugUnderflowOverflow: aborting after batch {self.batch_number - 1} as requested")


class DebugGradients:
    """Backward-hook counterpart: records abs min / max of the gradients flowing out of every module."""

    def __init__(self, model: nn.Module, max_frames_to_save: int = 21, trace_batch_nums: Optional[List[int]] = None) -> None:
        self.model = model
        self.frames: Deque[str] = collections.deque([], max_frames_to_save)
        self.trace_batch_nums = trace_batch_nums or []
        self.batch_number = 0
        self.detected_overflow = False
        self.module_names = {m: n for n, m in model.named_modules()}
        self.handles = [m.register_full_backward_hook(self._hook) for m in model.modules() if any(True for _ in m.parameters(recurse=False))]

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []

    def _hook(self, module: nn.Module, grad_input: Any, grad_output: Any) -> None:
        lines = [f"{self.module_names.get(module, '?')} {module.__class__.__name__}"]
        for tag, grads in (("grad_input", grad_input), ("grad_output", grad_output)):
            for i, g in enumerate(grads or ()):
                if torch.is_tensor(g) and g.numel() and g.is_floating_point():
                    lines.append(get_abs_min_max(g, f"{tag}[{i}]"))
                    if detect_overflow(g, f"{tag}[{i}]"):
                        self.detected_overflow = True
        frame = "\n".join(lines)
        self.frames.append(frame)
        if self.batch_number in self.trace_batch_nums:
            print(frame)
        if self.detected_overflow:
            report = "\n\n".join(self.frames)
            raise ValueError(f"DebugGradients: inf/nan gradient detected in batch {self.batch_number}:\n{report}")
        if module is self.model:
            self.batch_number += 1
