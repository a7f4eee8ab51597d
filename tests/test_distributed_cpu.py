# SPDX-License-Identifier: Apache-2.0
"""Multi-process tests on CPU (Gloo): ZeRO sharding, resume, launcher supervision, trainer equivalence
across parallel layouts.  Pattern of the reference's multi-GPU tests (tests/trainer/test_ulysses_alst.py):
same data, two layouts, compare the losses."""

import json
import socket
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch
import yaml

ROOT = Path(__file__).resolve().parent.parent
WORKER = str(ROOT / "tests" / "dist_worker.py")


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(world, *worker_args, timeout=300, expect_fail=False):
    cmd = [sys.executable, "-m", "arctictraining_b200.launcher.local", "--num_gpus", str(world), "--master_port",
           str(free_port()), "--", sys.executable, "-u", WORKER, *map(str, worker_args)]
    env = {"PATH": "/usr/bin:/bin", "PYTHONPATH": str(ROOT), "AT_LOG_LEVEL": "WARNING", "CUDA_VISIBLE_DEVICES": ""}
    import os

    env = {**os.environ, **env}
    t0 = time.time()
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    if expect_fail:
        return res, time.time() - t0
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res, time.time() - t0


@pytest.fixture(scope="module")
def single_process_reference():
    sys.path.insert(0, str(ROOT / "tests"))
    import dist_worker as w

    engine = w.make_engine(0)
    losses = []
    for b in w.global_batches(3, 2):
        out = engine(**b)
        engine.backward(out.loss)
        engine.step()
        losses.append(float(out.loss))
    return losses, {n: t.clone() for n, t in engine.iter_full_named_parameters()}


@pytest.mark.parametrize("stage", [0, 1, 2, 3])
def test_two_ranks_match_single_process(tmp_path, single_process_reference, stage):
    ref_losses, ref_params = single_process_reference
    launch(2, f"zero{stage}", tmp_path)
    got = torch.load(tmp_path / f"zero{stage}.pt", weights_only=False)
    assert got["losses"] == pytest.approx(ref_losses, rel=1e-5)
    for n, p in ref_params.items():
        assert (got["params"][n] - p).abs().mean() < 2e-5, n
    if stage == 3:
        assert all(got["released"]), "stage 3 must release the layer buffers after use"
    assert got["norm"] > 0


def test_layers_that_keep_activations_match_under_stage3(tmp_path, single_process_reference):
    """Stage 3 on two ranks with the last two layers keeping their activations (parameters gathered again before
    their backward, possibly into another pool buffer) gives the single-process result."""
    ref_losses, ref_params = single_process_reference
    launch(2, "zero3keep", tmp_path)
    got = torch.load(tmp_path / "zero3.pt", weights_only=False)
    assert got["losses"] == pytest.approx(ref_losses, rel=1e-5)
    for n, p in ref_params.items():
        assert (got["params"][n] - p).abs().mean() < 2e-5, n
    assert all(got["released"])


def test_sharded_checkpoint_resume_two_ranks(tmp_path):
    launch(2, "resume", tmp_path)
    res = json.loads((tmp_path / "resume.json").read_text())
    assert res["ok"], res


def test_launcher_stops_all_ranks_when_one_fails(tmp_path):
    res, elapsed = launch(2, "rank_failure", tmp_path, expect_fail=True, timeout=120)
    assert res.returncode != 0
    assert elapsed < 45, "the surviving rank was not terminated promptly"
    assert "injected failure" in res.stderr


def _recipe(tmp_path, name, **over):
    r = {
        "type": "sft", "micro_batch_size": 1, "epochs": 1, "exit_iteration": 4, "seed": 7,
        "model": {"name_or_path": "tiny-llama", "dtype": "fp32", "attn_implementation": "sdpa"},
        "data": {"sources": [{"type": "synthetic", "num_samples": 16, "min_length": 64, "max_length": 64}],
                 "cache_dir": str(tmp_path / "cache"), "max_length": 64, "dl_num_workers": 0},
        "optimizer": {"lr": 1e-3},
        "deepspeed": {"zero_optimization": {"stage": 3}},
        "train_log_metrics_path": str(tmp_path / f"{name}.jsonl"),
        "kill_switch_path": str(tmp_path / "kill"),
    }
    r.update(over)
    p = tmp_path / f"{name}.yaml"
    p.write_text(yaml.safe_dump(r))
    return p


def _losses(path):
    return [json.loads(line)["loss"] for line in Path(path).read_text().splitlines() if line.strip()]


def test_sequence_parallel_matches_data_parallel(tmp_path):
    """DP=2 vs SP=2 with GAS=2 (the same two samples feed every optimizer step), plus tiled MLP."""
    dp = _recipe(tmp_path, "dp")
    sp = _recipe(tmp_path, "sp", sequence_parallel_size=2, gradient_accumulation_steps=2, exit_iteration=2,
                 tiled_mlp_compute=True)
    launch(2, "trainer", tmp_path, dp)
    launch(2, "trainer", tmp_path, sp)
    l_dp, l_sp = _losses(tmp_path / "dp.jsonl"), _losses(tmp_path / "sp.jsonl")
    assert len(l_dp) >= 2 and len(l_sp) >= 2
    assert l_sp[0] == pytest.approx(l_dp[0], rel=1e-5, abs=1e-6)
    assert l_sp[1] == pytest.approx(l_dp[1], rel=2e-3)


def _read_safetensors_dir(d):
    from safetensors.torch import load_file

    out = {}
    for f in sorted(Path(d).glob("*.safetensors")):
        out.update(load_file(str(f)))
    return out


def test_expert_parallel_run_matches_unsharded_experts_and_exports_all_experts(tmp_path):
    """Pattern of the reference's MoE test (tests/trainer/test_moe.py:56-239) on two Gloo ranks: the same tiny
    Qwen3-MoE model trained with EP=1 (every rank holds all experts) and with EP=2 (each rank holds half of them), each
    stopped after two steps and resumed for two more.  The four losses agree, the per-(expert-parallel rank, layer)
    expert files exist, and the Hugging Face exports after steps 2 and 4 hold the same tensors for every expert."""
    runs = {}
    for name, ep in (("ep1", 1), ("ep2", 2)):
        out = tmp_path / name
        over = dict(
            model={"name_or_path": "tiny-qwen3-moe", "dtype": "fp32", "attn_implementation": "sdpa"},
            arctic_moe=True, expert_parallel_size=ep, optimizer={"type": "fused_adam_moe", "lr": 1e-3},
            deepspeed={"zero_optimization": {"stage": 2}},
            checkpoint=[
                {"type": "deepspeed", "output_dir": str(out / "ds"), "save_every_n_steps": 2, "auto_resume": True},
                {"type": "huggingface", "output_dir": str(out / "hf"), "save_every_n_steps": 2},
            ],
            exit_iteration=0, exit_iteration_this_run=2,
        )
        recipe = _recipe(tmp_path, name, **over)
        launch(2, "trainer", tmp_path, recipe)   # steps 1-2, checkpoint
        launch(2, "trainer", tmp_path, recipe)   # resume, steps 3-4
        runs[name] = _losses(tmp_path / f"{name}.jsonl")
        assert len(runs[name]) == 4, runs[name]
    assert runs["ep2"] == pytest.approx(runs["ep1"], rel=2e-4)
    tag_dirs = sorted((tmp_path / "ep2" / "ds").glob("*global_step_4"))
    assert tag_dirs and sorted(p.name for p in tag_dirs[0].glob("ep_rank_*_moe_layer_*_model_states.pt"))[:2] == [
        "ep_rank_0_moe_layer_0_model_states.pt", "ep_rank_0_moe_layer_1_model_states.pt"]
    assert list(tag_dirs[0].glob("ep_rank_1_moe_layer_0_model_states.pt"))
    for step in (2, 4):
        a = _read_safetensors_dir(tmp_path / "ep1" / "hf" / f"global_step_{step}")
        b = _read_safetensors_dir(tmp_path / "ep2" / "hf" / f"global_step_{step}")
        assert set(a) == set(b) and any(".experts.3." in k for k in b)
        for k in a:
            # AdamW turns rounding differences of near-zero gradients into full learning-rate steps: compare each
            # tensor as a whole tightly and single elements within a few steps of the learning rate (1e-3)
            assert float((b[k] - a[k]).norm() / (a[k].norm() + 1e-12)) < 3e-2, (k, step)
            torch.testing.assert_close(b[k], a[k], atol=2e-3 * step + 1e-4, rtol=0, msg=lambda m: f"{k} at step {step}: {m}")


def test_gathered_parameters_of_the_stand_in_engine_package_two_ranks(tmp_path):
    launch(2, "shim", tmp_path)
    r0, r1 = (torch.load(tmp_path / f"shim_rank{r}.pt", weights_only=True) for r in (0, 1))
    for r in (r0, r1):
        assert torch.all(r["seen"] == 0.125) and torch.all(r["inside"] == 0.125)
        # one AdamW step at lr 1e-2 moves every element by at most about lr (+ weight decay): the update started from
        # the value rank 0 wrote, not from the initial weights
        assert (r["after"] - 0.125).abs().max() < 0.03
    torch.testing.assert_close(r0["after"], r1["after"])


@pytest.mark.parametrize("world", [2, 4])
def test_library_model_attention_under_sequence_parallelism(tmp_path, world):
    """Ulysses through the attention registry of the transformers library (one key/value head, so it is replicated
    over the ranks; two packed samples): loss and summed gradients equal the single-process run."""
    launch(world, "ulysses_hf", tmp_path)
    r = torch.load(tmp_path / "ulysses_hf.pt", weights_only=True)
    assert r["calls"] >= 2 and r["registered_by_name_matches"]
    torch.testing.assert_close(r["loss"], r["ref_loss"], rtol=1e-5, atol=1e-6)
    for name, want in r["ref_grads"].items():
        torch.testing.assert_close(r["grads"][name], want, rtol=2e-4, atol=2e-6, msg=lambda m, n=name: f"{n}: {m}")


def test_library_model_trains_under_sequence_parallelism_like_data_parallel(tmp_path):
    """An architecture without an own implementation (OLMo-2 from the transformers library, random weights): DP=2 vs
    SP=2 with GAS=2 through the trainer - the same two samples feed every optimizer step, so the losses agree."""
    from transformers import Olmo2Config

    arch = tmp_path / "tiny-olmo2"
    Olmo2Config(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=256).save_pretrained(arch)
    model = {"name_or_path": str(arch), "dtype": "fp32", "attn_implementation": "sdpa",
             "hf_config_kwargs": {"num_hidden_layers": 2}}  # a changed depth means random initialisation
    common = dict(model=model, tokenizer={"type": "fake", "name_or_path": "tiny-llama"})
    dp = _recipe(tmp_path, "lib_dp", **common)
    sp = _recipe(tmp_path, "lib_sp", sequence_parallel_size=2, gradient_accumulation_steps=2, exit_iteration=2, **common)
    launch(2, "trainer", tmp_path, dp)
    launch(2, "trainer", tmp_path, sp)
    l_dp, l_sp = _losses(tmp_path / "lib_dp.jsonl"), _losses(tmp_path / "lib_sp.jsonl")
    assert len(l_dp) >= 2 and len(l_sp) >= 2
    assert l_sp[0] == pytest.approx(l_dp[0], rel=1e-5, abs=1e-6)
    assert l_sp[1] == pytest.approx(l_dp[1], rel=2e-3)
