# SPDX-License-Identifier: Apache-2.0
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
