# SPDX-License-Identifier: Apache-2.0
"""Snowflake Cortex and vLLM synthesizers.  Behaviour parity: arctic_training/synth/callers.py:62-133,
vllm_callers.py:40-207, vllm_utils.py:26-152.  Heavy dependencies (snowflake connector, vllm, aiohttp) are imported
when a client is created or used.
"""

from __future__ import annotations

import asyncio
import json
import os
import subprocess
import sys
import time
from typing import Any
from typing import Dict
from typing import List
from typing import Optional

from .base import InMemoryBatchProcessor


class CortexSynth(InMemoryBatchProcessor):
    """Calls ``SNOWFLAKE.CORTEX.COMPLETE`` once per queued request over one SQL connection."""

    def __init__(self, connection_params: Optional[Dict[str, Any]] = None, work_dir: Optional[str] = None,
                 connection: Any = None) -> None:
        super().__init__(work_dir)
        if connection is None:
            import snowflake.connector

            connection = snowflake.connector.connect(**(connection_params or {}))
        self.conn = connection

    def add_chat_to_batch_task(self, task_name: str, model: str, messages: List[Dict[str, str]],
                               options: Optional[Dict[str, Any]] = None) -> str:
        return self._queue(task_name, {"model": model, "messages": messages,
                                       "options": options or {"temperature": 1, "top_p": 1}})

    def execute_batch_task(self, task_name: str) -> List[Dict[str, Any]]:
        out = []
        cur = self.conn.cursor()
        for r in self.requests.get(task_name, []):
            cur.execute("SELECT SNOWFLAKE.CORTEX.COMPLETE(%s, PARSE_JSON(%s), PARSE_JSON(%s))",
                        (r["model"], json.dumps(r["messages"]), json.dumps(r["options"])))
            row = cur.fetchone()
            out.append({"custom_id": r["custom_id"], "response": json.loads(row[0]) if row and row[0] else None})
        self.save_results(task_name, out)
        return out

    @staticmethod
    def extract_messages_from_responses(responses: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        res = []
        for r in responses:
            choices = (r.get("response") or {}).get("choices", [])
            res.append({"custom_id": r["custom_id"],
                        "choices": [{"content": c.get("messages", c.get("message", ""))} for c in choices]})
        return res


class VllmSynth(InMemoryBatchProcessor):
    """In-process vLLM engine (``LLM.chat``) for fast local batch generation on one node."""

    def __init__(self, model_params: Dict[str, Any], sampling_params: Any = None, work_dir: Optional[str] = None,
                 llm: Any = None) -> None:
        super().__init__(work_dir)
        if llm is None:
            from vllm import LLM

            llm = LLM(**model_params)
        self.llm = llm
        self.sampling_params = sampling_params

    def add_chat_to_batch_task(self, task_name: str, messages: List[Dict[str, str]]) -> str:
        return self._queue(task_name, {"messages": messages})

    def execute_batch_task(self, task_name: str) -> List[Dict[str, Any]]:
        reqs = self.requests.get(task_name, [])
        outputs = self.llm.chat([r["messages"] for r in reqs], sampling_params=self.sampling_params, use_tqdm=True)
        out = [{"custom_id": r["custom_id"], "response": {"choices": [{"content": c.text} for c in o.outputs]}}
               for r, o in zip(reqs, outputs)]
        self.save_results(task_name, out)
        return out

    @staticmethod
    def extract_messages_from_responses(responses: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        return [{"custom_id": r["custom_id"], "choices": r["response"]["choices"]} for r in responses]


def launch_vllm_servers(model: str, n_replicas: int, tensor_parallel: int = 1, base_port: int = 8100,
                        gpu_ids: Optional[List[int]] = None, extra_args: Optional[List[str]] = None,
                        log_dir: Optional[str] = None) -> List[Dict[str, Any]]:
    """Start ``vllm serve`` once per GPU group; returns ``[{"proc", "url", "gpus"}]``."""
    gpu_ids = gpu_ids if gpu_ids is not None else list(range(n_replicas * tensor_parallel))
    servers = []
    for i in range(n_replicas):
        gpus = gpu_ids[i * tensor_parallel : (i + 1) * tensor_parallel]
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(map(str, gpus)))
        cmd = [sys.executable, "-m", "vllm.entrypoints.openai.api_server", "--model", model, "--port", str(base_port + i),
               "--tensor-parallel-size", str(tensor_parallel), *(extra_args or [])]
        log = open(os.path.join(log_dir, f"vllm_{i}.log"), "w") if log_dir else subprocess.DEVNULL
        servers.append({"proc": subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT),
                        "url": f"http://127.0.0.1:{base_port + i}", "gpus": gpus})
    return servers


def wait_until_healthy(servers: List[Dict[str, Any]], timeout_s: float = 1800.0, poll_s: float = 5.0) -> None:
    import requests

    deadline = time.time() + timeout_s
    pending = list(servers)
    while pending and time.time() < deadline:
        for s in list(pending):
            if s["proc"].poll() is not None:
                raise RuntimeError(f"vllm server for GPUs {s['gpus']} exited with code {s['proc'].returncode}")
            try:
                if requests.get(s["url"] + "/health", timeout=2).status_code == 200:
                    pending.remove(s)
            except requests.RequestException:
                pass
        if pending:
            time.sleep(poll_s)
    if pending:
        raise TimeoutError(f"{len(pending)} vllm server(s) did not become healthy within {timeout_s}s")


def check_vllm_servers_health(base_port: int, num_services: int, timeout_s: float = 1800.0, poll_s: float = 30.0,
                              host: str = "127.0.0.1") -> None:
    """Block until ``num_services`` servers on consecutive ports from ``base_port`` answer ``/health``."""
    alive = type("_Alive", (), {"poll": staticmethod(lambda: None), "returncode": None})
    servers = [{"url": f"http://{host}:{base_port + i}", "gpus": [i], "proc": alive} for i in range(num_services)]
    wait_until_healthy(servers, timeout_s=timeout_s, poll_s=poll_s)


def kill_processes(process_ids: List[int]) -> None:
    """SIGTERM to each given process id; ids that no longer exist or cannot be signalled are logged and skipped."""
    import signal

    from ..logging import logger

    for pid in process_ids:
        try:
            os.kill(pid, signal.SIGTERM)
            logger.info(f"Process {pid} terminated.")
        except ProcessLookupError:
            logger.info(f"Process {pid} does not exist.")
        except PermissionError:
            logger.info(f"Permission denied to terminate process {pid}.")


class MultiReplicaVllmSynth(InMemoryBatchProcessor):
    """Fans chat requests out over several ``vllm serve`` replicas (one per GPU group) with bounded concurrency."""

    def __init__(self, model: str, n_replicas: int, tensor_parallel: int = 1, sampling: Optional[Dict[str, Any]] = None,
                 work_dir: Optional[str] = None, max_concurrency_per_replica: int = 64, servers: Optional[List[Dict[str, Any]]] = None,
                 max_attempts: int = 3, **server_kwargs: Any) -> None:
        super().__init__(work_dir)
        self.model, self.sampling, self.concurrency = model, sampling or {}, max_concurrency_per_replica
        self.max_attempts = max(1, max_attempts)
        self.owns_servers = servers is None
        self.servers = servers if servers is not None else launch_vllm_servers(model, n_replicas, tensor_parallel, **server_kwargs)
        if self.owns_servers:
            wait_until_healthy(self.servers)

    def add_chat_to_batch_task(self, task_name: str, messages: List[Dict[str, str]]) -> str:
        return self._queue(task_name, {"messages": messages})

    async def _run(self, reqs: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        import aiohttp

        sem = asyncio.Semaphore(self.concurrency * len(self.servers))
        results: List[Optional[Dict[str, Any]]] = [None] * len(reqs)

        async def one(i: int, r: Dict[str, Any], session: Any) -> None:
            # a failed request moves on to the next replica; after ``max_attempts`` the error is the result, so that one
            # bad replica or prompt cannot lose the answers of all the others
            error = "no attempt"
            async with sem:
                for attempt in range(self.max_attempts):
                    url = self.servers[(i + attempt) % len(self.servers)]["url"] + "/v1/chat/completions"
                    try:
                        async with session.post(url, json={"model": self.model, "messages": r["messages"], **self.sampling}) as resp:
                            if resp.status == 200:
                                results[i] = {"custom_id": r["custom_id"], "response": await resp.json(content_type=None)}
                                return
                            error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                    except (aiohttp.ClientError, asyncio.TimeoutError) as e:
                        error = f"{type(e).__name__}: {e}"
            results[i] = {"custom_id": r["custom_id"], "response": None, "error": error}

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
            await asyncio.gather(*(one(i, r, session) for i, r in enumerate(reqs)))
        return [r for r in results if r is not None]

    def process_conversations_across_replicas(self, conversations: List[List[Dict[str, str]]]) -> List[Dict[str, Any]]:
        reqs = [{"custom_id": f"conv_{i}", "messages": m} for i, m in enumerate(conversations)]
        return asyncio.run(self._run(reqs))

    def execute_batch_task(self, task_name: str) -> List[Dict[str, Any]]:
        out = asyncio.run(self._run(self.requests.get(task_name, [])))
        self.save_results(task_name, out)
        return out

    @staticmethod
    def extract_messages_from_responses(responses: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        return [{"custom_id": r["custom_id"],
                 "choices": [{"content": c["message"]["content"]} for c in (r["response"] or {}).get("choices", [])]}
                for r in responses]

    def teardown(self) -> None:
        if not self.owns_servers:
            return
        for s in self.servers:
            if s["proc"].poll() is None:
                s["proc"].terminate()
        for s in self.servers:
            try:
                s["proc"].wait(timeout=30)
            except subprocess.TimeoutExpired:
                s["proc"].kill()
