# SPDX-License-Identifier: Apache-2.0
import json
from types import SimpleNamespace

from arctictraining_b200.synth import CortexSynth
from arctictraining_b200.synth import OpenAIBatchProcessor
from arctictraining_b200.synth import VllmSynth


class FakeOpenAI:
    """Stands in for the SDK client: files / batches namespaces with in-memory state."""

    def __init__(self):
        self.uploaded, self.polls = {}, 0
        self.files = SimpleNamespace(create=self._file_create, content=self._file_content)
        self.batches = SimpleNamespace(create=self._batch_create, retrieve=self._batch_retrieve, cancel=lambda i: None)

    def _file_create(self, file, purpose):
        fid = f"file-{len(self.uploaded)}"
        self.uploaded[fid] = file.read().decode()
        return SimpleNamespace(id=fid)

    def _batch_create(self, input_file_id, endpoint, completion_window):
        return SimpleNamespace(id="batch-" + input_file_id)

    def _batch_retrieve(self, bid):
        self.polls += 1
        done = self.polls > 2
        return SimpleNamespace(id=bid, status="completed" if done else "in_progress", output_file_id=bid.replace("batch-", "") if done else None)

    def _file_content(self, fid):
        lines = []
        for line in self.uploaded[fid].splitlines():
            req = json.loads(line)
            text = req["body"]["messages"][-1]["content"].upper()
            lines.append(json.dumps({"custom_id": req["custom_id"],
                                     "response": {"body": {"choices": [{"message": {"content": text}}]}}}))
        return SimpleNamespace(text="\n".join(lines))


def test_openai_batch_life_cycle(tmp_path):
    proc = OpenAIBatchProcessor(FakeOpenAI(), work_dir=str(tmp_path), batch_size=2, polling_interval=0.0)
    for w in ("a", "b", "c"):
        proc.add_chat_to_batch_task("t", model="m", messages=[{"role": "user", "content": w}])
    res = proc.execute_batch_task("t")
    msgs = OpenAIBatchProcessor.extract_messages_from_responses(res)
    assert sorted(m["choices"][0]["content"] for m in msgs) == ["A", "B", "C"]
    assert len(list((tmp_path / "t").glob("requests_*.jsonl"))) == 2  # batch_size 2 -> two files
    assert (tmp_path / "t" / "results.jsonl").exists()


def test_vllm_synth_with_injected_engine(tmp_path):
    class FakeLLM:
        def chat(self, convs, sampling_params=None, use_tqdm=False):
            return [SimpleNamespace(outputs=[SimpleNamespace(text=c[-1]["content"][::-1])]) for c in convs]

    s = VllmSynth({}, llm=FakeLLM(), work_dir=str(tmp_path))
    s.add_chat_to_batch_task("t", [{"role": "user", "content": "abc"}])
    out = VllmSynth.extract_messages_from_responses(s.execute_batch_task("t"))
    assert out[0]["choices"][0]["content"] == "cba"


def test_cortex_synth_with_fake_connection():
    class Cur:
        def execute(self, sql, params):
            self.last = params

        def fetchone(self):
            return (json.dumps({"choices": [{"messages": "ok:" + json.loads(self.last[1])[0]["content"]}]}),)

    s = CortexSynth(connection=SimpleNamespace(cursor=lambda: Cur()))
    s.add_chat_to_batch_task("t", "model", [{"role": "user", "content": "hi"}])
    out = CortexSynth.extract_messages_from_responses(s.execute_batch_task("t"))
    assert out[0]["choices"][0]["content"] == "ok:hi"


def _start_replica(fail_first: int):
    """A local HTTP server that answers like an OpenAI-compatible replica; its first `fail_first` requests get a 500."""
    import threading
    from http.server import BaseHTTPRequestHandler
    from http.server import ThreadingHTTPServer

    state = {"seen": 0, "lock": threading.Lock()}

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            self.send_response(200 if self.path == "/health" else 404)
            self.end_headers()

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            with state["lock"]:
                state["seen"] += 1
                fail = state["seen"] <= fail_first
            payload = b"boom" if fail else json.dumps(
                {"choices": [{"message": {"content": body["messages"][-1]["content"][::-1]}}]}).encode()
            self.send_response(500 if fail else 200)
            self.send_header("Content-Length", str(len(payload)))
            self.end_headers()
            self.wfile.write(payload)

    server = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    threading.Thread(target=server.serve_forever, daemon=True).start()
    return server, state


def test_multi_replica_fan_out_retries_on_another_replica_and_reports_lost_requests(tmp_path):
    import pytest

    from arctictraining_b200.synth.callers import MultiReplicaVllmSynth
    from arctictraining_b200.synth.callers import wait_until_healthy

    good, good_state = _start_replica(0)
    flaky, flaky_state = _start_replica(2)
    try:
        servers = [{"url": f"http://127.0.0.1:{s.server_address[1]}", "gpus": [i], "proc": SimpleNamespace(poll=lambda: None)}
                   for i, s in enumerate((good, flaky))]
        wait_until_healthy(servers, timeout_s=10, poll_s=0.1)
        synth = MultiReplicaVllmSynth("m", 2, servers=servers, work_dir=str(tmp_path), sampling={"temperature": 0})
        for i in range(6):
            synth.add_chat_to_batch_task("t", [{"role": "user", "content": f"abc{i}"}])
        out = synth.extract_messages_from_responses(synth.execute_batch_task("t"))
        assert [o["choices"][0]["content"] for o in out] == [f"{i}cba" for i in range(6)]
        assert flaky_state["seen"] >= 3 and good_state["seen"] >= 5  # the two refused requests went to the other replica
        synth.teardown()  # servers it did not start are left alone

        # a replica that always fails: its requests end as error records, the rest still answer
        dead, _ = _start_replica(10**6)
        only_dead = [{"url": f"http://127.0.0.1:{dead.server_address[1]}", "gpus": [0], "proc": SimpleNamespace(poll=lambda: None)}]
        lost = MultiReplicaVllmSynth("m", 1, servers=only_dead, max_attempts=2).process_conversations_across_replicas(
            [[{"role": "user", "content": "x"}]])
        assert lost[0]["response"] is None and lost[0]["error"].startswith("HTTP 500")
        assert synth.extract_messages_from_responses(lost)[0]["choices"] == []
        dead.shutdown()

        # a server process that died is an error at once, not a time-out
        gone = [{"url": "http://127.0.0.1:9", "gpus": [3], "proc": SimpleNamespace(poll=lambda: 1, returncode=1)}]
        with pytest.raises(RuntimeError, match="exited"):
            wait_until_healthy(gone, timeout_s=5, poll_s=0.1)
    finally:
        good.shutdown()
        flaky.shutdown()
