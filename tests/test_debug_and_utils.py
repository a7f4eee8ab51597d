# SPDX-License-Identifier: Apache-2.0
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.nn as nn

from arctictraining_b200.debug.underflow_overflow import DebugGradients
from arctictraining_b200.debug.underflow_overflow import DebugUnderflowOverflow
from arctictraining_b200.testing_utils import CaptureStd
from arctictraining_b200.testing_utils import get_unique_port_number
from arctictraining_b200.testing_utils import mockenv_context
from arctictraining_b200.utils.misc import human_format_base10_number
from arctictraining_b200.utils.misc import human_format_secs


def test_overflow_tracer_aborts_with_frames():
    class Boom(nn.Module):
        def forward(self, x):
            return x * float("inf")

    model = nn.Sequential(nn.Linear(4, 4), Boom())
    DebugUnderflowOverflow(model, max_frames_to_save=5)
    with pytest.raises(ValueError, match="inf/nan detected"):
        model(torch.ones(2, 4))


def test_overflow_tracer_passes_clean_batches_and_can_be_removed():
    model = nn.Sequential(nn.Linear(4, 4), nn.ReLU())
    dbg = DebugUnderflowOverflow(model, trace_batch_nums=[])
    model(torch.ones(2, 4))
    model(torch.ones(2, 4))
    assert dbg.batch_number == 2 and dbg.total_calls == 6
    dbg.remove()
    model(torch.ones(2, 4))
    assert dbg.total_calls == 6


def test_gradient_tracer_detects_nan_gradient():
    model = nn.Sequential(nn.Linear(4, 4))
    DebugGradients(model)
    out = model(torch.ones(2, 4))
    with pytest.raises(ValueError, match="gradient detected"):
        (out * float("nan")).sum().backward()


def test_small_helpers(capsys):
    assert human_format_base10_number(1234567) == "1.23M"
    assert human_format_secs(0.0123) == "12.3ms" and human_format_secs(3661) == "01:01:01"
    with mockenv_context("HOME", ATB_TEST_VAR="1"):
        import os

        assert os.environ["ATB_TEST_VAR"] == "1" and "HOME" not in os.environ
    assert "ATB_TEST_VAR" not in __import__("os").environ
    with CaptureStd(replay=False) as cs:
        print("hello")
        print("10%\r100% done", file=sys.stderr)
    assert cs.out.strip() == "hello"
    assert cs.err == "100% done\n" and cs.combined == "hello\n100% done\n" and "stderr: 100% done" in repr(cs)
    assert get_unique_port_number() >= 10999


def test_host_adamw_extension_matches_reference_update():
    import torch

    from arctictraining_b200.ops import _ext_cpu
    from arctictraining_b200.ops import reference as ref

    if not _ext_cpu.available():
        import pytest

        pytest.skip("no C++ compiler for the host extension")
    torch.manual_seed(0)
    n = 200_003  # not a multiple of the chunk or vector width
    p, g, m = torch.randn(n), torch.randn(n) * 0.1, torch.randn(n) * 0.01
    v = torch.rand(n) * 0.01
    lp = torch.empty(n, dtype=torch.bfloat16)
    p2, m2, v2 = p.clone(), m.clone(), v.clone()
    lp2 = torch.empty(n, dtype=torch.bfloat16)
    for step in (1, 2, 3):
        _ext_cpu.ops().cpu_adamw_step(p, g, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
        ref.adamw_step(p2, g, m2, v2, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5, lp2)
    assert torch.allclose(p, p2, atol=1e-6, rtol=1e-5)
    assert torch.allclose(m, m2, atol=1e-7, rtol=1e-5) and torch.allclose(v, v2, atol=1e-9, rtol=1e-5)
    assert (lp.float() - lp2.float()).abs().max() <= 2 ** -7 * p.abs().max()


def test_testing_helpers_env_paths_logger_and_seed(tmp_path, monkeypatch):
    import logging
    import random
    import sys

    from arctictraining_b200 import testing_utils as tu

    monkeypatch.setenv("ATB_FLAG", "Yes")
    monkeypatch.setenv("ATB_INT", "12")
    assert tu.parse_flag_from_env("ATB_FLAG") is True and tu.parse_flag_from_env("ATB_UNSET", True) is True
    assert tu.parse_int_from_env("ATB_INT") == 12 and tu.parse_int_from_env("ATB_UNSET", 3) == 3
    monkeypatch.setenv("ATB_FLAG", "maybe")
    with pytest.raises(ValueError, match="yes or no"):
        tu.parse_flag_from_env("ATB_FLAG")
    monkeypatch.setenv("ATB_INT", "x")
    with pytest.raises(ValueError, match="int"):
        tu.parse_int_from_env("ATB_INT")

    tu.set_seed(7)
    a = (random.random(), torch.rand(1).item())
    tu.set_seed(7)
    assert a == (random.random(), torch.rand(1).item())
    assert tu.get_gpu_count() == torch.cuda.device_count()
    assert tu.get_tests_dir() == str(Path(__file__).resolve().parent)
    assert tu.get_tests_dir("data").endswith("tests/data")
    assert tu.apply_print_resets("10%\r50%\r done\nnext") == " done\nnext"

    f = tmp_path / "a" / "b.txt"
    tu.write_file(f, "alpha beta")
    tu.replace_str_in_file(f, "beta", "gamma")
    assert f.read_text() == "alpha gamma"

    log = logging.getLogger("atb200-test-capture")
    with tu.CaptureLogger(log) as cl:
        log.warning("look here")
    assert cl.out == "look here\n" and "look here" in repr(cl)
    with tu.ExtendSysPath(tmp_path):
        assert sys.path[0] == str(tmp_path)
    assert str(tmp_path) not in sys.path

    for mark in (tu.require_torch, tu.require_deepspeed, tu.require_torch_no_gpus, tu.require_torch_up_to_2_gpus,
                 tu.require_flash_attn, tu.require_flash_attn_3):
        assert callable(mark(lambda: None))

    class Case(tu.TestCasePlus):
        def runTest(self):
            pass

    case = Case()
    case.setUp()
    assert case.test_file_path == Path(__file__).resolve() and case.tests_dir_str.endswith("tests")
    assert (case.src_dir / "arctictraining_b200").is_dir() and case.repo_root_dir_str == str(case.tests_dir.parent)
    assert case.get_env()["PYTHONPATH"].split(":")[0] == case.src_dir_str
    d = case.get_auto_remove_tmp_dir_str()
    assert Path(d).is_dir()
    case.tearDown()
    assert not Path(d).exists()


def test_make_reports_writes_one_file_per_kind(tmp_path):
    """A small suite with a pass, a failure, a skip and a warning, run with ``--make-reports``."""
    import subprocess
    import sys

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "conftest.py").write_text(
        "import arctictraining_b200.testing_utils as tu\n"
        "def pytest_addoption(parser):\n    tu.pytest_addoption_shared(parser)\n"
        "def pytest_terminal_summary(terminalreporter):\n"
        "    rid = terminalreporter.config.getoption('--make-reports')\n"
        "    if rid:\n        tu.pytest_terminal_summary_main(terminalreporter, id=rid)\n")
    (tmp_path / "test_toy.py").write_text(
        "import time, warnings, pytest\n"
        "def test_ok():\n    time.sleep(0.06)\n"
        "def helper():\n    assert 1 == 2, 'numbers differ'\n"
        "def test_bad():\n    helper()\n"
        "def test_warn():\n    warnings.warn('careful', UserWarning)\n"
        "@pytest.mark.skip(reason='not today')\ndef test_skip():\n    pass\n")
    env = dict(os.environ, PYTHONPATH=str(root))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--make-reports=toy", "test_toy.py"],
                       cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 1, r.stdout + r.stderr
    rep = tmp_path / "reports" / "toy"
    assert sorted(p.name for p in rep.iterdir()) == [
        "durations.txt", "errors.txt", "failures_line.txt", "failures_long.txt", "failures_short.txt", "stats.txt",
        "summary_short.txt", "warnings.txt"]
    assert "test_toy.py::test_ok" in (rep / "durations.txt").read_text()
    assert "numbers differ" in (rep / "failures_line.txt").read_text()
    long, short = (rep / "failures_long.txt").read_text(), (rep / "failures_short.txt").read_text()
    assert "def test_bad" in long and "numbers differ" in short and len(short) < len(long)
    assert "careful" in (rep / "warnings.txt").read_text()
    summary = (rep / "summary_short.txt").read_text()
    assert "FAILED test_toy.py::test_bad" in summary and "SKIPPED test_toy.py::test_skip" in summary
    assert (rep / "stats.txt").read_text().strip() == "2 passed, 1 failed, 1 skipped, 1 warnings"


def test_device_id_follows_visible_devices_and_nvml_reads_that_device(monkeypatch):
    import sys
    from types import SimpleNamespace

    from arctictraining_b200.debug import utils as du

    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    assert du.get_device_id(2) == 2
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,6,7")
    assert du.get_device_id(1) == 6
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "GPU-abc, GPU-def")
    assert du.get_device_id(1) == "GPU-def"
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    assert du.get_device_id(0) is None

    asked = []
    fake = SimpleNamespace(
        nvmlInit=lambda: None,
        nvmlDeviceGetHandleByIndex=lambda i: asked.append(i) or ("idx", i),
        nvmlDeviceGetHandleByUUID=lambda u: asked.append(u) or ("uuid", u),
        nvmlDeviceGetMemoryInfo=lambda h: SimpleNamespace(used=3 * 2**30))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setattr(du, "_nvml_handle", None)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "5")
    monkeypatch.setenv("LOCAL_RANK", "0")
    assert du.get_nvml_mem() == 3 * 2**30 and asked == [5]
    assert du.get_nvml_mem() == 3 * 2**30 and asked == [5]  # the handle is kept
    monkeypatch.setattr(du, "_nvml_handle", None)
    fake.nvmlDeviceGetMemoryInfo = lambda h: (_ for _ in ()).throw(RuntimeError("not supported"))
    assert du.get_nvml_mem() == 0
    du.gc_empty_accelerator_cache()
    assert du.pr0 is du.print_rank0 and du.pr is du.print_rank
