# SPDX-License-Identifier: Apache-2.0
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
    assert cs.out.strip() == "hello"
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
