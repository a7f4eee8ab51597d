# SPDX-License-Identifier: Apache-2.0
"""Speculator data generation: prompt cutting, sharding, job scripts, the GPU-queue runner (with `echo` jobs on CPU),
merging, and training on the merged dataset with ``process: false``."""
import importlib.util
from pathlib import Path

import pytest
import yaml

ROOT = Path(__file__).resolve().parent.parent
GEN = ROOT / "projects" / "arctic_lstm_speculator" / "data_generation"


def _load(name):
    spec = importlib.util.spec_from_file_location(f"_specgen_{name}", GEN / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Tok:
    """Whitespace tokenizer with a trivial chat template."""

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False):
        text = " ".join(f"<{m['role']}> {m['content']}" for m in messages) + (" <assistant>" if add_generation_prompt else "")
        return self(text)["input_ids"] if tokenize else text

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [hash(w) % 1000 for w in text.split()]}


def test_prompt_cutting_and_sharding():
    g = _load("vllm_data_generation")
    assert g.chunk_prompts(list(range(10)), 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert g.chunk_prompts([1, 2], 4) == []
    covered = [i for s in range(3) for i in g.shard_range(10, s, 3)]
    assert covered == list(range(10))
    with pytest.raises(ValueError):
        g.shard_range(10, 3, 3)
    assert g.resolve_dataset("ultrachat")[0] == "HuggingFaceH4/ultrachat_200k"
    assert g.resolve_dataset("aya_french")[1] == "french"
    assert g.resolve_dataset("org/data:validation") == ("org/data", None, "validation", None)
    conv = g.as_conversation({"problem": "q", "solution": "a"}, ("problem", "solution"))
    assert [m["role"] for m in conv] == ["user", "assistant"]
    msgs = [{"role": "user", "content": "a b c"}, {"role": "assistant", "content": "d e"},
            {"role": "user", "content": "f"}, {"role": "assistant", "content": "g h i j"}]
    chunks = g.build_prompts([msgs], _Tok(), "chunks", 4, 100)
    assert len(chunks) == 14 // 4 and all(len(c) == 4 for c in chunks)
    turns = g.build_prompts([msgs], _Tok(), "turns", 4, 100)
    assert len(turns) == 2 and len(turns[0]) < len(turns[1])
    assert g.build_prompts([msgs], _Tok(), "turns", 4, 6) == turns[:1]  # the longer prompt exceeds the limit


def test_generation_files_merge_and_train(tiny_recipe, tmp_path):
    g, c = _load("vllm_data_generation"), _load("concat_generated_datasets")
    prompts = [[1, 2, 3, 4]] * 5
    n = g.write_generations(str(tmp_path / "raw" / "ultrachat" / "0_2.jsonl"), prompts,
                            lambda part: [[10 + i for i in range(24)] for _ in part], batch=2)
    g.write_generations(str(tmp_path / "raw" / "magicoder" / "0_2.jsonl"), prompts[:3],
                        lambda part: [[40 + i for i in range(24)] for _ in part])
    with open(tmp_path / "raw" / "magicoder" / "0_2.jsonl", "a") as f:
        f.write('{"input": [1, 2], "outp')  # a writer that was killed mid-line
    assert n == 5
    files = c.find_generation_files([str(tmp_path / "raw")])
    assert len(files) == 2
    cols = c.read_generations(files)
    assert len(cols["input_ids"]) == 8 and cols["input_ids"] == cols["labels"]
    with_prompt = c.read_generations(files, with_prompt=True)
    assert with_prompt["labels"][0][:4] == [-100] * 4 and len(with_prompt["input_ids"][0]) == 28

    from datasets import Dataset

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    Dataset.from_dict(cols).save_to_disk(str(tmp_path / "all"))
    model = {"name_or_path": "tiny-llama", "dtype": "fp32", "n_speculator_heads": 2, "speculator_width": "32",
             "proj_dim": "32", "emb_dim": "32", "method": "sum_lstm", "speculator_tie_weights": True,
             "tie_lstm_embs": True, "disable_activation_checkpoint": True}
    r = tiny_recipe(type="arctic-lstm-speculator", code=str(ROOT / "projects" / "arctic_lstm_speculator" / "train.py"),
                    model=model, exit_iteration=2, micro_batch_size=2)
    r["data"]["sources"] = [{"type": "huggingface", "name_or_path": str(tmp_path / "all"), "process": False}]
    r["data"].update(filter_samples=False, pack_samples=False)
    r["deepspeed"] = {"zero_optimization": {"stage": 2}}
    p = tmp_path / "r.yaml"
    p.write_text(yaml.safe_dump(r))
    tr = get_registered_trainer(get_config(p).type)(get_config(p))
    tr.train()
    assert tr.global_step == 2


def test_job_scripts_and_gpu_queue(tmp_path):
    m, r = _load("make_datagen_jobs"), _load("multigpu_runner")
    paths = m.write_jobs("org/model", str(tmp_path / "raw"), str(tmp_path / "jobs"), ["ultrachat", "aya_french"], 2,
                         tensor_parallel=2, temperature=0.0, extra=["--gen-tokens", "128"])
    assert len(paths) == 4
    text = open(paths[0]).read()
    assert "--shard 0 --num-shards 2" in text and "--tensor-parallel 2" in text and "--gen-tokens 128" in text
    assert "VLLM_CACHE_ROOT" in text and str(tmp_path / "raw" / "ultrachat" / "0_2.jsonl") in text

    assert r.gpu_groups(range(8), 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert r.gpu_groups([2, 3, 5], 1, jobs_per_group=2) == [[2], [2], [3], [3], [5], [5]]
    with pytest.raises(ValueError):
        r.gpu_groups([0], 2)

    jobs = tmp_path / "q"
    jobs.mkdir()
    log = tmp_path / "log"
    for i in range(5):
        (jobs / f"j{i}.sh").write_text(f'echo "j{i} $CUDA_VISIBLE_DEVICES" >> {log}\n')
    (jobs / "bad.sh").write_text("exit 3\n")
    with pytest.raises(SystemExit, match="bad"):
        r.main([str(jobs), "--gpus", "0,1,2,3", "-n", "2"])
    lines = sorted(open(log).read().split("\n")[:-1])
    assert [ln.split()[0] for ln in lines] == [f"j{i}" for i in range(5)]
    assert {ln.split()[1] for ln in lines} <= {"0,1", "2,3"}
    # a second run skips what finished and retries only the failed job
    assert [name for name, _ in r.folder_jobs(str(jobs))] == ["bad"]
    (jobs / "bad.sh").write_text("true\n")
    r.main([str(jobs), "--gpus", "0"])
    assert r.folder_jobs(str(jobs)) == []
    # the watch mode picks up scripts that appear later
    calls = []

    def more():
        calls.append(1)
        if len(calls) == 1:
            return [("late", f"echo late >> {log}")]
        raise KeyboardInterrupt

    assert r.run_queue([], [[0]], more_jobs=more, poll_s=0.01) == []
    assert "late" in open(log).read()
