# SPDX-License-Identifier: Apache-2.0
"""Named timers that measure on the device (CUDA events) when a GPU is present, else wall clock.

Parity: the reference relies on a synchronising wall-clock timer from its engine dependency
(arctic_training/metrics.py:86-101, arctic_training/model/moe/timers.py:21-72).
"""

from __future__ import annotations

import time
from typing import Dict
from typing import List

import torch


class DeviceTimer:
    def __init__(self, name: str) -> None:
        self.name = name
        self._cuda = torch.cuda.is_available()
        self._start = None
        self._pairs: List = []
        self._elapsed_ms = 0.0
        self.count = 0

    def start(self) -> None:
        if self._cuda:
            self._start = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._start = time.perf_counter()

    def stop(self) -> None:
        if self._start is None:
            return
        if self._cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pairs.append((self._start, end))
        else:
            self._elapsed_ms += (time.perf_counter() - self._start) * 1e3
        self._start = None
        self.count += 1

    def elapsed(self, reset: bool = True) -> float:
        """Milliseconds accumulated since the last reset (synchronises the pending events)."""
        if self._cuda and self._pairs:
            self._pairs[-1][1].synchronize()
            self._elapsed_ms += sum(s.elapsed_time(e) for s, e in self._pairs)
            self._pairs = []
        out = self._elapsed_ms
        if reset:
            self._elapsed_ms = 0.0
            self.count = 0
        return out


class TimerGroup:
    def __init__(self) -> None:
        self.timers: Dict[str, DeviceTimer] = {}

    def __call__(self, name: str) -> DeviceTimer:
        if name not in self.timers:
            self.timers[name] = DeviceTimer(name)
        return self.timers[name]

    def get_timers(self) -> Dict[str, DeviceTimer]:
        return self.timers

    def snapshot(self, reset: bool = True) -> Dict[str, float]:
        return {k: t.elapsed(reset) for k, t in self.timers.items()}
