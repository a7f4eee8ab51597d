# SPDX-License-Identifier: Apache-2.0
import pytest
import torch

from arctictraining_b200.attention.moba import moba_attn_naive
from arctictraining_b200.attention.moba import moba_attn_varlen
from arctictraining_b200.ops import reference as ref


def test_moba_equals_full_causal_attention_when_topk_covers_all_blocks():
    torch.manual_seed(0)
    S, H, D = 96, 2, 16
    q, k, v = (torch.randn(S, H, D) for _ in range(3))
    cu = torch.tensor([0, 40, 96])
    out = moba_attn_naive(q, k, v, cu, 56, moba_chunk_size=16, moba_topk=64)
    full = ref.attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), cu_seqlens=cu)[0]
    assert torch.allclose(out, full, atol=1e-5)


def test_moba_varlen_matches_naive_with_sparse_topk():
    torch.manual_seed(0)
    S, H, D = 130, 3, 8
    q, k, v = (torch.randn(S, H, D) for _ in range(3))
    cu = torch.tensor([0, 70, 130])
    a = moba_attn_naive(q, k, v, cu, 70, moba_chunk_size=16, moba_topk=2)
    b = moba_attn_varlen(q, k, v, cu, 70, moba_chunk_size=16, moba_topk=2, query_chunk=32)
    assert torch.allclose(a, b, atol=1e-5)
    full = ref.attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), cu_seqlens=cu)[0]
    assert not torch.allclose(a, full, atol=1e-3)  # sparse selection really drops blocks


def test_moba_efficient_matches_naive_forward_and_backward():
    from arctictraining_b200.attention.moba import moba_attn_efficient

    torch.manual_seed(1)
    S, H, D = 150, 2, 8
    cu = torch.tensor([0, 90, 150])
    base = [torch.randn(S, H, D) for _ in range(3)]
    grads = []
    outs = []
    for fn in (moba_attn_naive, moba_attn_efficient):
        q, k, v = (t.clone().requires_grad_(True) for t in base)
        o = fn(q, k, v, cu, 90, moba_chunk_size=16, moba_topk=3)
        o.square().sum().backward()
        outs.append(o.detach())
        grads.append((q.grad, k.grad, v.grad))
    assert torch.allclose(outs[0], outs[1], atol=1e-5)
    for a, b in zip(*grads):
        assert torch.allclose(a, b, atol=1e-4)


def test_moba_trainer_is_the_swiftkv_distillation_with_block_attention(tiny_recipe, tmp_path):
    """The project trainer of the reference: SwiftKV self-distillation whose attention (teacher and student) is MoBA.
    With ``topk`` covering every block MoBA equals full attention, so the run must reproduce the plain SwiftKV run."""
    from pathlib import Path

    import yaml

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    root = Path(__file__).resolve().parent.parent

    def run(kind, **model_extra):
        r = tiny_recipe(
            type=kind, code=str(root / "projects" / ("moba_attention" if kind == "moba" else "swiftkv") / "train.py"),
            model={"name_or_path": "tiny-llama", "dtype": "fp32", "num_key_value_layers": 1, "key_value_group_size": 1,
                   "hf_config_kwargs": {"num_hidden_layers": 3}, **model_extra},
            exit_iteration=2, optimizer={"lr": 1e-2, "weight_decay": 0.0},
            train_log_metrics_path=str(tmp_path / f"{kind}.jsonl"),
        )
        p = tmp_path / f"{kind}.yaml"
        p.write_text(yaml.safe_dump(r))
        tr = get_registered_trainer(get_config(p).type)(get_config(p))
        batch = next(iter(tr.train_dataloader))
        return tr, float(tr.loss(dict(batch)).detach())

    moba, loss_all_blocks = run("moba", moba_chunk_size=16, moba_topk=64)
    assert type(moba.model_unwrapped.sp_context).__name__ == "MoBAContext"
    assert all("swiftkv" in n for n, p in moba.model_unwrapped.named_parameters() if p.requires_grad)
    _, loss_swiftkv = run("swiftkv")
    assert loss_all_blocks == pytest.approx(loss_swiftkv, rel=1e-4, abs=1e-6)
    _, loss_sparse = run("moba", moba_chunk_size=16, moba_topk=2)
    assert loss_sparse != pytest.approx(loss_swiftkv, rel=1e-6)   # dropping blocks changes teacher and student
    moba.train()
    assert moba.global_step == 2
