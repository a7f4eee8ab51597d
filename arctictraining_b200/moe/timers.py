# SPDX-License-Identifier: Apache-2.0
"""Per-stage timers of the MoE block (router, dispatch, experts, combine, shared expert, whole block) and token-count
statistics, for the ``wall_clock_breakdown`` report.

Parity: arctic_training/model/moe/timers.py:24-79 and the report of arctic_training/model/moe/moe.py:465-509.  The
reference wraps DeepSpeed's synchronising wall-clock timer (one device synchronisation per start and stop); here a stage
is bracketed by two CUDA events on the launching stream and the elapsed times are read when the report is made, so
switching the timers on adds no synchronisation to the step.  On the CPU the stages are timed with the host clock.
"""

from __future__ import annotations

import time
from collections import defaultdict
from typing import Dict
from typing import List
from typing import Tuple

import torch

STAGES = ("amoe e2e", "router", "dispatch", "experts", "combine", "shared-expert")


class StageTimers:
    def __init__(self, enabled: bool = False) -> None:
        self.wall_clock_breakdown = enabled
        self.times: Dict[str, float] = defaultdict(float)       # milliseconds, summed over the calls since the last report
        self.calls: Dict[str, int] = defaultdict(int)
        self.token_counts: Dict[str, int] = {}
        self._open: Dict[str, object] = {}
        self._pending: List[Tuple[str, object, object]] = []

    def _now(self, on_gpu: bool):
        if on_gpu:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def start(self, name: str, on_gpu: bool = False) -> None:
        if self.wall_clock_breakdown:
            self._open[name] = self._now(on_gpu)

    def stop(self, name: str, on_gpu: bool = False) -> None:
        if self.wall_clock_breakdown and name in self._open:
            self._pending.append((name, self._open.pop(name), self._now(on_gpu)))

    def collect(self) -> Dict[str, float]:
        """Resolve the recorded intervals (synchronises the device once when events are pending)."""
        if any(not isinstance(a, float) for _, a, _ in self._pending):
            torch.cuda.synchronize()
        for name, a, b in self._pending:
            self.times[name] += (b - a) * 1e3 if isinstance(a, float) else a.elapsed_time(b)
            self.calls[name] += 1
        self._pending.clear()
        return dict(self.times)

    def reset(self) -> None:
        self.times.clear()
        self.calls.clear()
        self._pending.clear()
        self._open.clear()

    def record_token_counts(self, received_per_rank, sent_per_rank) -> None:
        """Load-balance statistics of one exchange (host integers; call only with values that are on the host)."""
        if not self.wall_clock_breakdown:
            return
        self.token_counts.update(
            max_rcv_count_per_rank=int(max(received_per_rank)), min_rcv_count_per_rank=int(min(received_per_rank)),
            max_snd_count_per_rank=int(max(sent_per_rank)), min_snd_count_per_rank=int(min(sent_per_rank)),
        )


def moe_blocks(model: torch.nn.Module):
    from .layer import ArcticMoE

    return [m for m in model.modules() if isinstance(m, ArcticMoE)]


def enable_moe_timers(model: torch.nn.Module, enabled: bool = True) -> int:
    blocks = moe_blocks(model)
    for m in blocks:
        m.timers.wall_clock_breakdown = enabled
        if not enabled:
            m.timers.reset()
    return len(blocks)


def forward_breakdown(model: torch.nn.Module, reset: bool = True) -> Dict[str, float]:
    """Milliseconds per stage summed over all MoE blocks since the last report, plus the token-count statistics of the
    last block that recorded some (keys ``tokens/<name>``)."""
    total: Dict[str, float] = defaultdict(float)
    for m in moe_blocks(model):
        for k, v in m.timers.collect().items():
            total[k] += v
        for k, v in m.timers.token_counts.items():
            total[f"tokens/{k}"] = v
        if reset:
            m.timers.reset()
    return dict(total)


def format_breakdown(breakdown: Dict[str, float]) -> str:
    stages = [f"{k}: {breakdown[k]:.2f}" for k in STAGES if k in breakdown]
    counts = [f"{k[7:]}: {int(v)}" for k, v in breakdown.items() if k.startswith("tokens/")]
    return "AMoE time (ms) | " + " | ".join(stages) + ((" | " + " | ".join(counts)) if counts else "")
