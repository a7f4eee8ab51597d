# SPDX-License-Identifier: Apache-2.0
"""Single-GPU engine tests: bf16 model on the CUDA kernels against the same model in fp32 on the CPU, and the
engine's memory/speed options (direct bf16 gradients, layers that keep activations, native attention) against
each other."""

import copy
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from arctictraining_b200.engine import TrainingEngine  # noqa: E402
from arctictraining_b200.models.arch import load_arch_config  # noqa: E402
from arctictraining_b200.models.causal_lm import CausalLM  # noqa: E402
from arctictraining_b200.optimizer.adam import FusedAdamW  # noqa: E402
from arctictraining_b200.optimizer.factory import OptimizerFactory  # noqa: E402

ARCH = dict(hidden_size=256, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
            intermediate_size=512, vocab_size=1024)


def make_model(device, dtype, attn="sdpa"):
    cfg = load_arch_config("tiny-llama", ARCH)
    m = CausalLM(cfg, dtype=dtype)
    m.init_weights(seed=0)
    m.attn_impl = attn
    return m.to(device)


def make_engine(model, stage=3, **extra):
    opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(model, 0.1), lr=3e-3, betas=(0.9, 0.95))
    return TrainingEngine(model, opt, None, {"zero_optimization": {"stage": stage}, "gradient_clipping": 1.0,
                                             "bf16": {"enabled": next(model.parameters()).dtype == torch.bfloat16}, **extra})


def batches(n, device, bs=2, seq=256, vocab=1024):
    g = torch.Generator().manual_seed(0)
    out = []
    for _ in range(n):
        ids = torch.randint(8, vocab, (bs, seq), generator=g)
        labels = ids.clone()
        labels[:, : seq // 4] = -100
        out.append({"input_ids": ids.to(device), "labels": labels.to(device)})
    return out


def run(engine, data):
    losses = []
    for b in data:
        out = engine(**b)
        engine.backward(out.loss)
        engine.step()
        losses.append(float(out.loss.detach()))
    return losses


def test_bf16_gpu_engine_tracks_fp32_cpu_engine():
    cpu = run(make_engine(make_model("cpu", torch.float32), 0), batches(4, "cpu"))
    gpu = run(make_engine(make_model("cuda", torch.bfloat16)), batches(4, "cuda"))
    assert gpu == pytest.approx(cpu, rel=3e-2)
    assert int(torch.ops.atb200.read_and_clear_error_flag(torch.zeros(1, device="cuda"))) == 0


def test_direct_bf16_gradients_equal_fp32_accumulation(monkeypatch):
    data = batches(3, "cuda")
    a = make_engine(make_model("cuda", torch.bfloat16))
    assert all(u.direct_grad for u in a.units if u.grad_acc is not None)
    assert all(u.grad_acc.dtype == torch.bfloat16 for u in a.units if u.grad_acc is not None)
    la = run(a, data)
    monkeypatch.setenv("ATB200_DIRECT_GRADS", "0")
    b = make_engine(make_model("cuda", torch.bfloat16))
    assert all(u.grad_acc.dtype == torch.float32 for u in b.units if u.grad_acc is not None)
    lb = run(b, data)
    assert la == pytest.approx(lb, rel=1e-6)
    pa = dict(a.iter_full_named_parameters())
    for n, t in b.iter_full_named_parameters():
        assert torch.equal(pa[n], t), n
    assert float(a.get_global_grad_norm()) == pytest.approx(float(b.get_global_grad_norm()), rel=1e-4)


@pytest.mark.parametrize("keep", [0, 4])
def test_first_weight_gradient_stored_without_zeroing_equals_zero_then_accumulate(monkeypatch, keep):
    """Linear-layer weight gradients written by a storing GEMM epilogue into a gradient buffer that was not zeroed
    (the default at world size 1) against the zero-fill + accumulate path (``ATB200_STORE_FIRST_WGRAD=0``): bf16(0 + x) == bf16(x), so losses,
    gradient norm and parameters agree bit for bit, with and without recomputation of the layers."""
    data = batches(3, "cuda")
    extra = {"activation_checkpoint_keep": keep}
    monkeypatch.setenv("ATB200_STORE_FIRST_WGRAD", "0")
    a = make_engine(make_model("cuda", torch.bfloat16), **extra)
    la = run(a, data)
    monkeypatch.setenv("ATB200_STORE_FIRST_WGRAD", "1")
    b = make_engine(make_model("cuda", torch.bfloat16), **extra)
    # poison the gradient buffers: whatever they hold must not reach the update
    for u in b.units:
        if u.grad_acc is not None:
            u.grad_acc.fill_(float("nan"))
    lb = run(b, data)
    assert any(len(getattr(u, "_store_first_cache", ())) > 0 for u in b.units), "the store-first path did not engage"
    assert la == lb
    pa = dict(a.iter_full_named_parameters())
    for n, t in b.iter_full_named_parameters():
        assert torch.equal(pa[n], t), n
    assert float(a.get_global_grad_norm()) == float(b.get_global_grad_norm())


@pytest.mark.parametrize("keep", [2, "auto"])
def test_layers_keeping_activations_on_gpu(keep):
    data = batches(5, "cuda")
    a = run(make_engine(make_model("cuda", torch.bfloat16)), data)
    e = make_engine(make_model("cuda", torch.bfloat16), activation_checkpoint_keep=keep)
    b = run(e, data)
    assert b == pytest.approx(a, rel=1e-6)
    if keep == "auto":
        assert e._keep_state["phase"] == 2 and e._keep_state["kept_layers"] == 4  # a tiny model fits entirely


def test_native_attention_in_the_model_matches_sdpa():
    data = batches(3, "cuda")
    a = run(make_engine(make_model("cuda", torch.bfloat16, "sdpa")), data)
    b = run(make_engine(make_model("cuda", torch.bfloat16, "native")), data)
    assert b == pytest.approx(a, rel=2e-2)


@pytest.mark.parametrize("zero", [
    {"stage": 3, "offload_optimizer": {"device": "cpu"}},
    {"stage": 3, "offload_optimizer": {"device": "cpu", "ratio": 0.5}},
    {"stage": 3, "offload_optimizer": {"device": "cpu"}, "offload_param": {"device": "cpu"}},
    {"stage": 2, "offload_optimizer": {"device": "cpu"}},
])
def test_host_offload_of_optimizer_states_and_parameters_matches_the_device_engine(zero, monkeypatch):
    """Optimizer states (all, or a fraction) and parameter shards in pinned host memory: same losses and the same
    weights as with everything on the device (the host AdamW and the CUDA AdamW follow the same update rule; the
    comparison run keeps fp32 gradient shards so that both accumulate alike)."""
    monkeypatch.setenv("ATB200_DIRECT_GRADS", "0")
    data = batches(3, "cuda")
    base = make_engine(make_model("cuda", torch.bfloat16), zero["stage"])
    opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(m := make_model("cuda", torch.bfloat16), 0.1), lr=3e-3, betas=(0.9, 0.95))
    off = TrainingEngine(m, opt, None, {"zero_optimization": zero, "gradient_clipping": 1.0, "bf16": {"enabled": True}})
    hosted = [u for u in off.units if u.host_states]
    assert hosted and all(u.master.device.type == "cpu" and u.master.is_pinned() for u in hosted if u.master is not None)
    if "ratio" in zero["offload_optimizer"]:
        assert any(u.master is not None and u.master.is_cuda for u in off.units)
    if "offload_param" in zero:
        held = [u for u in off.units if u.host_params]
        assert held and all(u.shard.device.type == "cpu" and u.shard.is_pinned() and not u.persistent for u in held)
    la, lb = run(base, data), run(off, data)
    assert lb == pytest.approx(la, rel=2e-3)
    pa = dict(base.iter_full_named_parameters())
    for n, t in off.iter_full_named_parameters():
        # AdamW turns gradients near its epsilon into full-size steps of either sign, and the host kernel (exact
        # division and square root) and the CUDA kernel (fast-math) round differently there: allow a small fraction
        # of elements to differ by a few learning-rate steps, and require the tensors to agree as a whole
        a, b = t.float().cpu(), pa[n].float().cpu()
        bad = ((a - b).abs() > 2e-3 + 2e-2 * b.abs()).float().mean().item()
        assert bad < 0.01, (n, bad)
        assert float((a - b).abs().max()) <= 4 * 3e-3 * len(data), n
        assert float((a - b).norm() / (b.norm() + 1e-12)) < 2e-2, n
    assert float(off.get_global_grad_norm()) == pytest.approx(float(base.get_global_grad_norm()), rel=1e-2)
    assert int(torch.ops.atb200.read_and_clear_error_flag(torch.zeros(1, device="cuda"))) == 0
