# SPDX-License-Identifier: Apache-2.0
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# a world of one process for everything that is not launched as a subprocess
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", "29511")
os.environ.setdefault("RANK", "0")
os.environ.setdefault("LOCAL_RANK", "0")
os.environ.setdefault("WORLD_SIZE", "1")
os.environ.setdefault("AT_LOG_LEVEL", "WARNING")


def pytest_addoption(parser):
    from arctictraining_b200.testing_utils import pytest_addoption_shared

    pytest_addoption_shared(parser)


def pytest_terminal_summary(terminalreporter):
    from arctictraining_b200.testing_utils import pytest_terminal_summary_main

    report_id = terminalreporter.config.getoption("--make-reports")
    if report_id:
        pytest_terminal_summary_main(terminalreporter, id=report_id)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no GPU")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def tiny_recipe(tmp_path):
    """A complete SFT recipe on the tiny Llama preset with synthetic tokens (no files, no network)."""

    def make(**overrides):
        cfg = {
            "type": "sft",
            "micro_batch_size": 2,
            "epochs": 1,
            "exit_iteration": 4,
            "seed": 7,
            "model": {"name_or_path": "tiny-llama", "dtype": "fp32", "attn_implementation": "sdpa"},
            "data": {
                "sources": [{"type": "synthetic", "num_samples": 32, "min_length": 64, "max_length": 64}],
                "cache_dir": str(tmp_path / "cache"),
                "max_length": 64,
                "dl_num_workers": 0,
            },
            "optimizer": {"lr": 1e-3},
            "deepspeed": {"zero_optimization": {"stage": 0}},
            "train_log_metrics_path": str(tmp_path / "metrics.jsonl"),
            "kill_switch_path": str(tmp_path / "kill"),
        }
        for k, v in overrides.items():
            if isinstance(v, dict) and isinstance(cfg.get(k), dict):
                cfg[k] = {**cfg[k], **v}
            else:
                cfg[k] = v
        return cfg

    return make
