# SPDX-License-Identifier: Apache-2.0
"""OpenAI / Azure OpenAI batch-API clients.  Behaviour parity: arctic_training/synth/openai_callers.py:43-428 — the
save -> upload -> submit -> poll -> download life cycle of a batch task, kept in a work directory so that an
interrupted run can be picked up again; credentials from a YAML file or the environment.  The ``openai`` package is
imported when a client is created.
"""

from __future__ import annotations

import json
import os
import time
from typing import Any
from typing import Dict
from typing import List
from typing import Optional

import yaml

from .base import BatchProcessor

MAX_REQUESTS_PER_FILE = 50_000
MAX_BYTES_PER_FILE = 190 * 1024 * 1024


class OpenAIBatchProcessor(BatchProcessor):
    def __init__(self, client: Any, work_dir: str = "./batch_work_dir", batch_size: int = MAX_REQUESTS_PER_FILE,
                 polling_interval: float = 30.0, endpoint: str = "/v1/chat/completions") -> None:
        self.client = client
        self.work_dir = work_dir
        self.batch_size = min(batch_size, MAX_REQUESTS_PER_FILE)
        self.polling_interval = polling_interval
        self.endpoint = endpoint
        self.requests: Dict[str, List[Dict[str, Any]]] = {}
        os.makedirs(work_dir, exist_ok=True)

    def _task_dir(self, task_name: str) -> str:
        d = os.path.join(self.work_dir, task_name)
        os.makedirs(d, exist_ok=True)
        return d

    def _state(self, task_name: str) -> Dict[str, Any]:
        p = os.path.join(self._task_dir(task_name), "state.json")
        return json.load(open(p)) if os.path.exists(p) else {"files": [], "file_ids": [], "batch_ids": []}

    def _save_state(self, task_name: str, state: Dict[str, Any]) -> None:
        with open(os.path.join(self._task_dir(task_name), "state.json"), "w") as fh:
            json.dump(state, fh)

    def add_chat_to_batch_task(self, task_name: str, **kwargs: Any) -> str:
        items = self.requests.setdefault(task_name, [])
        custom_id = kwargs.pop("custom_id", f"{task_name}_{len(items)}")
        items.append({"custom_id": custom_id, "method": "POST", "url": self.endpoint, "body": kwargs})
        return custom_id

    def save_batch_task(self, task_name: str) -> List[str]:
        """Write the queued requests as JSONL files that respect the service's per-file limits."""
        d, files, cur, cur_bytes = self._task_dir(task_name), [], [], 0

        def flush() -> None:
            nonlocal cur, cur_bytes
            if cur:
                path = os.path.join(d, f"requests_{len(files):04d}.jsonl")
                with open(path, "w") as fh:
                    fh.write("\n".join(cur) + "\n")
                files.append(path)
                cur, cur_bytes = [], 0

        for r in self.requests.get(task_name, []):
            line = json.dumps(r)
            if len(cur) >= self.batch_size or cur_bytes + len(line) > MAX_BYTES_PER_FILE:
                flush()
            cur.append(line)
            cur_bytes += len(line) + 1
        flush()
        state = self._state(task_name)
        state["files"] = files
        self._save_state(task_name, state)
        return files

    def upload_batch_task(self, task_name: str) -> List[str]:
        state = self._state(task_name)
        state["file_ids"] = [self.client.files.create(file=open(f, "rb"), purpose="batch").id for f in state["files"]]
        self._save_state(task_name, state)
        return state["file_ids"]

    def submit_batch_task(self, task_name: str, file_ids: Optional[List[str]] = None) -> List[str]:
        state = self._state(task_name)
        ids = file_ids or state["file_ids"]
        state["batch_ids"] = [
            self.client.batches.create(input_file_id=i, endpoint=self.endpoint, completion_window="24h").id for i in ids
        ]
        self._save_state(task_name, state)
        return state["batch_ids"]

    def retrieve_batch_task(self, task_name: Optional[str] = None, batch_ids: Optional[List[str]] = None,
                            print_status: bool = True) -> List[Any]:
        ids = batch_ids or self._state(task_name)["batch_ids"]
        batches = [self.client.batches.retrieve(i) for i in ids]
        if print_status:
            for b in batches:
                print(f"batch {b.id}: {b.status}")
        return batches

    def cancel_batch_task(self, task_name: str) -> None:
        for i in self._state(task_name)["batch_ids"]:
            self.client.batches.cancel(i)

    def download_batch_task(self, task_name: str) -> List[Dict[str, Any]]:
        results: List[Dict[str, Any]] = []
        for b in self.retrieve_batch_task(task_name, print_status=False):
            if getattr(b, "output_file_id", None):
                text = self.client.files.content(b.output_file_id).text
                results += [json.loads(line) for line in text.splitlines() if line.strip()]
        with open(os.path.join(self._task_dir(task_name), "results.jsonl"), "w") as fh:
            for r in results:
                fh.write(json.dumps(r) + "\n")
        return results

    def execute_batch_task(self, task_name: str, print_status: bool = False) -> List[Dict[str, Any]]:
        self.save_batch_task(task_name)
        self.upload_batch_task(task_name)
        self.submit_batch_task(task_name)
        done = {"completed", "failed", "expired", "cancelled"}
        while True:
            if all(b.status in done for b in self.retrieve_batch_task(task_name, print_status=print_status)):
                break
            time.sleep(self.polling_interval)
        return self.download_batch_task(task_name)

    @staticmethod
    def extract_messages_from_responses(responses: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        out = []
        for r in responses:
            body = (r.get("response") or {}).get("body") or {}
            out.append({"custom_id": r.get("custom_id"),
                        "choices": [{"content": c["message"]["content"]} for c in body.get("choices", [])]})
        return out


def load_credentials(path: Optional[str], section: str) -> Dict[str, Any]:
    """``<section>:`` block of a credential YAML file, or an empty dict (the SDK then reads the environment)."""
    if path and os.path.exists(path):
        return (yaml.safe_load(open(path)) or {}).get(section, {}) or {}
    return {}


def OpenAISynth(work_dir: str = "./batch_work_dir", credential_path: Optional[str] = None, **kw: Any) -> OpenAIBatchProcessor:
    from openai import OpenAI

    creds = load_credentials(credential_path, "openai")
    return OpenAIBatchProcessor(OpenAI(**{**creds, **kw.pop("client_kwargs", {})}), work_dir=work_dir, **kw)


def AzureOpenAISynth(work_dir: str = "./batch_work_dir", credential_path: Optional[str] = None, **kw: Any) -> OpenAIBatchProcessor:
    from openai import AzureOpenAI

    creds = load_credentials(credential_path, "azure_openai")
    return OpenAIBatchProcessor(AzureOpenAI(**{**creds, **kw.pop("client_kwargs", {})}), work_dir=work_dir,
                                endpoint="/chat/completions", **kw)
