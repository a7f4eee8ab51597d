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
