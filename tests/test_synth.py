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
