# SPDX-License-Identifier: Apache-2.0
"""Stand-in modules for the engine package the reference depends on, and the generic tiled autograd functions."""
import importlib.util
import sys
import time

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from arctictraining_b200.compat import deepspeed_shim
from arctictraining_b200.ops.tiled import TiledFusedLogitsLoss
from arctictraining_b200.ops.tiled import TiledMLP

REAL_PACKAGE = importlib.util.find_spec("deepspeed") is not None and "deepspeed" not in sys.modules


@pytest.fixture
def shim():
    if REAL_PACKAGE:
        pytest.skip("the real package is installed; the stand-ins stay out of its way")
    installed = deepspeed_shim.install()
    yield
    if installed:
        deepspeed_shim.uninstall()


def test_install_registers_modules_once_and_uninstall_removes_them():
    if REAL_PACKAGE:
        assert deepspeed_shim.install() is False
        return
    assert deepspeed_shim.install() is True
    try:
        assert deepspeed_shim.install() is False
        import deepspeed

        assert deepspeed.__atb200_shim__ and deepspeed.__version__.endswith("arctictraining_b200")
    finally:
        deepspeed_shim.uninstall()
    assert "deepspeed" not in sys.modules and "deepspeed.comm" not in sys.modules


def test_imports_of_reference_user_code_resolve(shim):
    import deepspeed
    import deepspeed.comm as dist
    from deepspeed import DeepSpeedEngine
    from deepspeed.accelerator import get_accelerator
    from deepspeed.ops.adam import DeepSpeedCPUAdam
    from deepspeed.ops.adam import FusedAdam
    from deepspeed.runtime.engine import DeepSpeedEngine as E2
    from deepspeed.runtime.sequence_parallel.ulysses_sp import TiledFusedLogitsLoss as L
    from deepspeed.runtime.sequence_parallel.ulysses_sp import TiledMLP as M
    from deepspeed.runtime.sequence_parallel.ulysses_sp import UlyssesSPDataLoaderAdapter  # noqa: F401
    from deepspeed.runtime.zero import GatheredParameters
    from deepspeed.runtime.zero.partition_parameters import ZeroParamStatus
    from deepspeed.utils.timer import SynchronizedWallClockTimer

    from arctictraining_b200.engine import TrainingEngine

    assert DeepSpeedEngine is TrainingEngine and E2 is TrainingEngine and L is TiledFusedLogitsLoss and M is TiledMLP
    assert dist.is_initialized is torch.distributed.is_initialized and dist.get_local_rank() == 0
    assert ZeroParamStatus.AVAILABLE.value == 1
    acc = get_accelerator()
    assert acc.device_name() in ("cpu", "cuda") and acc.memory_allocated() >= 0 and acc.current_device_name()
    acc.manual_seed_all(3)
    acc.empty_cache()
    with acc.stream(acc.Stream()):
        pass

    lin = nn.Linear(4, 4)
    for make in (FusedAdam, DeepSpeedCPUAdam):
        opt = make(lin.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
        assert opt.param_groups[0]["betas"] == (0.9, 0.95)
    with pytest.raises(ValueError):
        FusedAdam(lin.parameters(), amsgrad=True)

    timers = SynchronizedWallClockTimer()
    timers("fwd").start()
    time.sleep(0.01)
    timers("fwd").stop(record=True)
    assert timers.has("fwd") and timers("fwd").elapsed(reset=False) >= 9.0 and timers.get_mean(["fwd"])["fwd"] >= 9.0
    timers.log(["fwd", "missing"])
    assert timers("fwd").elapsed() == 0.0

    # parameters that no engine manages are whole already: the context is a no-op for them
    with GatheredParameters(lin, modifier_rank=0):
        lin.weight.data.zero_()
    assert torch.all(lin.weight == 0)

    # initialize() builds this package's engine; a gathered write reaches its master weights
    model = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8))
    engine, opt, _, _ = deepspeed.initialize(model=model, optimizer=FusedAdam(model.parameters(), lr=1e-2),
                                             config={"zero_optimization": {"stage": 2}})
    assert isinstance(engine, TrainingEngine) and opt is engine.optimizer
    with GatheredParameters([model[0].weight], modifier_rank=0):
        model[0].weight.data.fill_(0.5)
    full = dict(engine.iter_full_named_parameters())
    assert torch.all(full["0.weight"] == 0.5)
    unit = next(u for u in engine.units if any(p is model[0].weight for p in u.params))
    if unit.master is not None:
        assert (unit.master == 0.5).sum() >= model[0].weight.numel()


def test_tiled_functions_match_the_untiled_computation():
    torch.manual_seed(0)
    mlp = nn.Sequential(nn.Linear(16, 48), nn.GELU(), nn.Linear(48, 16))
    x = torch.randn(2, 37, 16, requires_grad=True)
    y = mlp(x)
    y.square().sum().backward()
    want = (y.detach(), x.grad.clone(), [p.grad.clone() for p in mlp.parameters()])
    x.grad = None
    mlp.zero_grad()
    y2 = TiledMLP.apply(lambda m, t: m(t), mlp, x, 5, list(mlp.parameters()))
    y2.square().sum().backward()
    torch.testing.assert_close(y2, want[0])
    torch.testing.assert_close(x.grad, want[1])
    for p, g in zip(mlp.parameters(), want[2]):
        torch.testing.assert_close(p.grad, g, rtol=1e-4, atol=1e-5)

    head = nn.Linear(16, 101, bias=False)
    labels = torch.randint(0, 101, (2, 37))
    labels[0, :5] = -100

    def ce_sum(m, h, lab, mask):
        return F.cross_entropy(m(h).float().view(-1, 101), lab.reshape(-1), ignore_index=-100, reduction="sum")

    x.grad = None
    ref = ce_sum(head, x, labels, None) * 0.5
    ref.backward()
    want = (ref.detach(), x.grad.clone(), head.weight.grad.clone())
    x.grad = None
    head.zero_grad()
    got = TiledFusedLogitsLoss.apply(ce_sum, head, x, labels, None, 4, [head.weight], "sum") * 0.5
    got.backward()
    torch.testing.assert_close(got, want[0])
    torch.testing.assert_close(x.grad, want[1])
    torch.testing.assert_close(head.weight.grad, want[2], rtol=1e-4, atol=1e-5)

    # "mean" with teacher states as the target, a mask and a ragged last tile (37 = 13 + 13 + 11)
    teacher = torch.randn(2, 37, 16)
    mask = torch.rand(2, 37) > 0.3

    def mse(m, h, t, msk):
        return ((h - t).square().mean(-1) * msk).sum() / h.shape[0] / h.shape[1]

    x.grad = None
    ref = mse(None, x, teacher, mask)
    ref.backward()
    want_dx = x.grad.clone()
    x.grad = None
    got = TiledFusedLogitsLoss.apply(mse, None, x, teacher, mask, 3, [], "mean")
    got.backward()
    torch.testing.assert_close(got, ref.detach())
    torch.testing.assert_close(x.grad, want_dx)
    with pytest.raises(ValueError):
        TiledFusedLogitsLoss.apply(mse, None, x, teacher, mask, 3, [], "median")
