# SPDX-License-Identifier: Apache-2.0
"""Batch processors for synthetic-data generation: a task is a named list of chat requests that is executed as one
batch and whose responses can be turned back into plain messages.

Behaviour parity: arctic_training/synth/base_caller.py:20-40 and callers.py:41-60.
"""

from __future__ import annotations

import json
import os
from abc import ABC
from abc import abstractmethod
from typing import Any
from typing import Dict
from typing import List
from typing import Optional


class BatchProcessor(ABC):
    @abstractmethod
    def add_chat_to_batch_task(self, task_name: str, **kwargs: Any) -> None:
        """Queue one chat-completion request under ``task_name``."""

    @abstractmethod
    def execute_batch_task(self, task_name: str) -> List[Any]:
        """Run all queued requests of the task and return the raw responses (blocking)."""

    @staticmethod
    @abstractmethod
    def extract_messages_from_responses(responses: List[Any]) -> List[Dict[str, Any]]:
        """Turn raw responses into ``{"custom_id": ..., "choices": [{"content": ...}]}`` records."""


class InMemoryBatchProcessor(BatchProcessor):
    """Keeps the queued requests in memory; optionally mirrors them to ``<work_dir>/<task>/requests.jsonl``."""

    def __init__(self, work_dir: Optional[str] = None) -> None:
        self.work_dir = work_dir
        self.requests: Dict[str, List[Dict[str, Any]]] = {}

    def _queue(self, task_name: str, request: Dict[str, Any]) -> str:
        items = self.requests.setdefault(task_name, [])
        request.setdefault("custom_id", f"{task_name}_{len(items)}")
        items.append(request)
        return request["custom_id"]

    def save_batch_task(self, task_name: str) -> Optional[str]:
        if self.work_dir is None:
            return None
        d = os.path.join(self.work_dir, task_name)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, "requests.jsonl")
        with open(path, "w") as fh:
            for r in self.requests.get(task_name, []):
                fh.write(json.dumps(r) + "\n")
        return path

    def save_results(self, task_name: str, results: List[Dict[str, Any]]) -> Optional[str]:
        if self.work_dir is None:
            return None
        d = os.path.join(self.work_dir, task_name)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, "results.jsonl")
        with open(path, "w") as fh:
            for r in results:
                fh.write(json.dumps(r) + "\n")
        return path
