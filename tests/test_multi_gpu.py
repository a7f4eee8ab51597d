# SPDX-License-Identifier: Apache-2.0
"""Multi-GPU tests (child processes, one per GPU, NCCL + peer memory); skipped when fewer than 2 GPUs are visible."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def launch(world, *args, timeout=600):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "arctictraining_b200.launcher.local", "--num_gpus", str(world), "--master_port", str(port),
           "--", sys.executable, "-u", str(ROOT / "tests" / "gpu_worker.py"), *map(str, args)]
    env = {**os.environ, "PYTHONPATH": str(ROOT), "AT_LOG_LEVEL": "WARNING", "NCCL_NVLS_ENABLE": "0"}
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]


def test_peer_memory_path_matches_nccl(tmp_path):
    launch(2, "fused_vs_nccl", tmp_path)
    res = json.loads((tmp_path / "fused_vs_nccl.json").read_text())
    for stage, r in res.items():
        assert r["fused"] == pytest.approx(r["nccl"], rel=2e-3), stage
        assert r["max_param_diff"] < 2e-2, stage


def test_partly_frozen_units_take_one_communication_path_on_every_rank(tmp_path):
    launch(2, "partly_frozen", tmp_path)
    per_rank = json.loads((tmp_path / "partly_frozen.json").read_text())
    # the premise: the last rank holds no trainable element of the partly frozen units, the first one does
    assert all(n > 0 for n in per_rank[0]["clip1.0"]["local_train_len"])
    assert all(n == 0 for n in per_rank[-1]["clip1.0"]["local_train_len"])
    for r in per_rank:
        for name, v in r.items():
            assert v["fused"] == pytest.approx(v["nccl"], rel=2e-3), name
            assert v["max_param_diff"] < 2e-2, name
            assert v["bit_identical_reruns"], name


def test_parameter_gather_inside_the_consuming_gemm_matches_the_pull_gather(tmp_path):
    launch(2, "gather_gemm", tmp_path)
    for per_rank in json.loads((tmp_path / "gather_gemm.json").read_text()):
        for name, r in per_rank.items():
            assert r["weight_equal"] and r["outside_untouched"] and r["out_equal"], (name, r)
            assert r["rel_err_vs_fp32"] < 1e-2, (name, r)


def test_bounded_barrier_reports_a_missing_peer(tmp_path):
    launch(2, "barrier_timeout", tmp_path)
    assert json.loads((tmp_path / "barrier_timeout.json").read_text())["ok"]


def test_peer_memory_ulysses_exchange_matches_nccl(tmp_path):
    launch(2, "ulysses_peer", tmp_path)
    for per_rank in json.loads((tmp_path / "ulysses_peer.json").read_text()):
        assert per_rank["kv_split"]["out_diff"] == 0.0 and per_rank["kv_split"]["grad_diff"] == 0.0
        r = per_rank["kv_replicated"]
        assert r["out_diff"] == 0.0 and r["grad_diff"] <= 2e-2 * r["grad_scale"]
        assert per_rank["kv_split_proj_err"] < 1e-2 and per_rank["kv_replicated_proj_err"] < 1e-2


def test_peer_memory_moe_exchange_matches_all_to_all(tmp_path):
    launch(2, "moe_peer", tmp_path)
    for per_rank in json.loads((tmp_path / "moe_peer.json").read_text()):
        for name, err in per_rank.items():
            assert err < 2e-2, (name, err)


def test_attention_block_with_exchanges_inside_the_gemms(tmp_path):
    launch(2, "fused_attention_block", tmp_path)
    for per_rank in json.loads((tmp_path / "fused_attention_block.json").read_text()):
        for name, err in per_rank.items():
            assert err < 1e-2, (name, err)
