# SPDX-License-Identifier: Apache-2.0
"""ArcticMoE on CPU: routing semantics, permutation round trip, equivalence with a naive per-token MoE,
HF name conversion and a tiny MoE training run."""

import pytest
import torch
import torch.nn.functional as F

from arctictraining_b200.models.arch import load_arch_config
from arctictraining_b200.models.causal_lm import CausalLM
from arctictraining_b200.moe import ops as mops
from arctictraining_b200.moe.layer import ArcticMoE
from arctictraining_b200.moe.layer import MoEConfig
from arctictraining_b200.ops import reference as ref


def test_topk_gating_ties_go_to_lower_index_and_scores_normalise():
    logits = torch.tensor([[1.0, 1.0, 0.0, 1.0], [0.0, 2.0, 2.0, -1.0]])
    scores, experts, probs = mops.topk_gating(logits, 2, True)
    assert experts.tolist() == [[0, 1], [1, 2]]
    assert torch.allclose(scores.sum(-1), torch.ones(2))
    assert torch.allclose(probs.sum(-1), torch.ones(2))
    raw, _, _ = mops.topk_gating(logits, 2, False)
    assert torch.allclose(raw[0], probs[0, :2])


def test_slots_are_expert_major_stable_and_aligned():
    experts = torch.tensor([[2, 0], [0, 1], [2, 1], [0, 2]], dtype=torch.int32)
    slots, counts, offsets = mops.assign_slots(experts, 4, align=4)
    assert counts.tolist() == [3, 2, 3, 0]
    assert offsets.tolist() == [0, 4, 8, 12, 12]
    # pairs in (token, k) order: (0,2)(0,0)(1,0)(1,1)(2,2)(2,1)(3,0)(3,2)
    assert slots.tolist() == [[8, 0], [1, 4], [9, 5], [2, 10]]


def test_scatter_gather_round_trip_and_grads():
    torch.manual_seed(0)
    T, H, K, E = 6, 8, 2, 3
    x = torch.randn(T, H, requires_grad=True)
    experts = torch.randint(0, E, (T, K), dtype=torch.int32)
    slots, _, offsets = mops.assign_slots(experts, E, align=4)
    rows = int(offsets[-1])
    perm = mops.scatter_rows(x, slots, rows)
    scores = torch.rand(T, K, requires_grad=True)
    out = mops.gather_rows(perm, slots, scores)
    assert torch.allclose(out, x * scores.sum(-1, keepdim=True), atol=1e-6)
    out.sum().backward()
    assert torch.allclose(x.grad, scores.sum(-1, keepdim=True).expand_as(x).detach(), atol=1e-6)


def naive_moe(moe: ArcticMoE, x: torch.Tensor) -> torch.Tensor:
    probs = torch.softmax(F.linear(x, moe.router_gate).float(), -1)
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, : moe.top_k]
    sc = torch.gather(probs, 1, order)
    sc = sc / sc.sum(-1, keepdim=True)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(moe.top_k):
            e = int(order[t, j])
            h = ref.swiglu_interleaved(F.linear(x[t : t + 1], moe.expert_gate_up[e]))
            out[t] += sc[t, j] * F.linear(h, moe.expert_down[e])[0]
    return out


def make_moe(E=4, K=2, H=64, I=64, **kw):
    torch.manual_seed(0)
    moe = ArcticMoE(MoEConfig(model_dim=H, intermediate_dim=I, num_experts=E, top_k=K, loss_coeff=0.0, **kw), dtype=torch.float32)
    for p in moe.parameters():
        torch.nn.init.normal_(p, std=0.1)
    return moe


def test_arctic_moe_matches_naive_forward_and_backward():
    moe = make_moe()
    x = torch.randn(10, 64, requires_grad=True)
    y = moe(x)
    y.pow(2).sum().backward()
    g_fast = {n: p.grad.clone() for n, p in moe.named_parameters()}
    gx = x.grad.clone()
    moe.zero_grad()
    x.grad = None
    y2 = naive_moe(moe, x)
    y2.pow(2).sum().backward()
    assert torch.allclose(y, y2, atol=1e-5)
    assert torch.allclose(gx, x.grad, atol=1e-4)
    for n, p in moe.named_parameters():
        assert torch.allclose(g_fast[n], p.grad, atol=1e-4), n


def test_load_balancing_term_pushes_probability_away_from_busy_experts():
    moe = make_moe(E=4, K=1)
    moe._config.loss_coeff = 1.0
    moe.train()
    x = torch.randn(32, 64)
    moe(x).sum().backward()
    g_with = moe.router_gate.grad.clone()
    moe.zero_grad()
    moe._config.loss_coeff = 0.0
    moe(x).sum().backward()
    assert not torch.allclose(g_with, moe.router_gate.grad)


def test_routing_replay_reuses_recorded_assignments():
    moe = make_moe()
    moe._config.enable_routing_replay = True
    x = torch.randn(7, 64)
    y1 = moe(x)
    rec = moe.recorded_assignments.clone()
    with torch.no_grad():
        moe.router_gate.add_(torch.randn_like(moe.router_gate))  # would change the routing
    moe.replay_assignments = rec
    moe(x)
    assert torch.equal(moe.recorded_assignments, rec)
    assert y1.shape == x.shape


def test_hf_names_round_trip_for_moe_model():
    from arctictraining_b200.models import hf_io

    cfg = load_arch_config("tiny-qwen3-moe")
    m = CausalLM(cfg, dtype=torch.float32)
    m.init_weights(seed=1)
    hf = dict(hf_io.iter_hf_tensors(((n, p.data) for n, p in m.named_parameters()), cfg))
    assert "model.layers.0.mlp.experts.3.gate_proj.weight" in hf and "model.layers.0.mlp.gate.weight" in hf
    assert "model.layers.1.self_attn.q_norm.weight" in hf
    native = hf_io.hf_to_native_state_dict(hf, cfg)
    for n, p in m.named_parameters():
        assert torch.equal(native[n], p.data), n


def test_tiny_moe_model_trains(tiny_recipe):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    cfg = get_config(tiny_recipe(model={"name_or_path": "tiny-qwen3-moe", "dtype": "fp32"}, arctic_moe="auto",
                                 optimizer={"type": "fused_adam_moe", "lr": 1e-3}, exit_iteration=3))
    tr = get_registered_trainer(cfg.type)(cfg)
    assert tr.use_arctic_moe
    tr.train()
    assert tr.global_step == 3


def test_gpt_oss_stacked_expert_layout_round_trips_and_keeps_the_math():
    """gpt-oss stores all experts of a block in two stacked tensors with gate / up interleaved element-wise; the remap
    into ArcticMoE's stacks and back is lossless, and a block built from them computes gate * sigmoid(1.702 gate) * up."""
    from arctictraining_b200.models import hf_io
    from arctictraining_b200.moe.grouped import grouped_mlp_reference

    cfg = load_arch_config("tiny-qwen3-moe")
    cfg = type(cfg)({**cfg, "model_type": "gpt_oss"})
    E, H, I = 4, 64, 128
    g = torch.Generator().manual_seed(0)
    gu = torch.randn(E, H, 2 * I, generator=g)
    down = torch.randn(E, I, H, generator=g)
    hf = {"model.layers.0.mlp.experts.gate_up_proj": gu, "model.layers.0.mlp.experts.down_proj": down,
          "model.layers.0.mlp.router.weight": torch.randn(E, H, generator=g),
          "model.layers.0.mlp.experts.gate_up_proj_bias": torch.zeros(E, 2 * I)}
    native = hf_io.hf_to_native_state_dict(dict(hf), cfg)
    assert native["model.layers.0.mlp.expert_gate_up"].shape == (E, 2 * I, H)
    assert native["model.layers.0.mlp.expert_down"].shape == (E, H, I)
    back = dict(hf_io.iter_hf_tensors(native.items(), cfg))
    for k in ("model.layers.0.mlp.experts.gate_up_proj", "model.layers.0.mlp.experts.down_proj", "model.layers.0.mlp.router.weight"):
        assert torch.equal(back[k], hf[k]), k
    # the math of one expert, written out in the Hugging Face layout
    x = torch.randn(128, H, generator=g)
    offsets = torch.tensor([0, 128, 128, 128, 128], dtype=torch.int32)
    y = grouped_mlp_reference(x, offsets, native["model.layers.0.mlp.expert_gate_up"], native["model.layers.0.mlp.expert_down"],
                              act_fn="silu_alpha")
    z = x @ gu[0]
    gate, up = z[:, 0::2], z[:, 1::2]
    want = (gate * torch.sigmoid(1.702 * gate) * up) @ down[0]
    torch.testing.assert_close(y, want, atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("family", ["qwen3_moe", "qwen2_moe"])
def test_transformers_sparse_blocks_convert_to_arctic_moe_with_equal_logits(family):
    """A ``transformers`` model of the Qwen MoE families (the path other architectures take through the model factory)
    gives the same logits after its sparse blocks have been replaced by ArcticMoE blocks — router, experts, and for
    Qwen2-MoE / Qwen3-Next the sigmoid-gated shared expert."""
    transformers = pytest.importorskip("transformers")
    from arctictraining_b200.moe.convert import convert_hf_blocks_to_arctic_moe
    from arctictraining_b200.moe.layer import ArcticMoE

    common = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  vocab_size=256, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
                  decoder_sparse_step=1, mlp_only_layers=[], max_position_embeddings=128)
    if family == "qwen3_moe":
        cfg = transformers.Qwen3MoeConfig(**common, head_dim=16)
        model = transformers.Qwen3MoeForCausalLM(cfg)
    else:
        cfg = transformers.Qwen2MoeConfig(**common, shared_expert_intermediate_size=64)
        model = transformers.Qwen2MoeForCausalLM(cfg)
    torch.manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():
            p.normal_(0, 0.05)
    model = model.float().eval()
    ids = torch.randint(0, 256, (2, 10))
    with torch.no_grad():
        want = model(input_ids=ids).logits
        assert convert_hf_blocks_to_arctic_moe(model) == 2
        assert all(isinstance(layer.mlp, ArcticMoE) for layer in model.model.layers)
        model.eval()
        got = model(input_ids=ids).logits
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), float((got - want).abs().max())


def test_stage_timers_report_every_stage_once_enabled():
    from arctictraining_b200.moe.layer import ArcticMoE
    from arctictraining_b200.moe.layer import MoEConfig
    from arctictraining_b200.moe.timers import enable_moe_timers
    from arctictraining_b200.moe.timers import format_breakdown
    from arctictraining_b200.moe.timers import forward_breakdown

    torch.manual_seed(0)
    model = torch.nn.Sequential(
        ArcticMoE(MoEConfig(model_dim=32, intermediate_dim=64, num_experts=4, top_k=2, use_shared_expert=True,
                            shared_intermediate_dim=64, input_dtype=torch.float32), dtype=torch.float32),
        ArcticMoE(MoEConfig(model_dim=32, intermediate_dim=64, num_experts=4, top_k=2, input_dtype=torch.float32), dtype=torch.float32),
    )
    for p in model.parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(2, 6, 32)
    model(x)
    assert forward_breakdown(model) == {}          # off by default: nothing recorded, nothing synchronised
    assert enable_moe_timers(model) == 2
    model(x)
    model(x)
    report = forward_breakdown(model)
    assert set(report) == {"amoe e2e", "router", "dispatch", "experts", "combine", "shared-expert"}
    assert report["amoe e2e"] >= report["experts"] > 0
    assert model[0].timers.calls == {} and forward_breakdown(model) == {}   # the report resets the sums
    line = format_breakdown(report)
    assert line.startswith("AMoE time (ms) | amoe e2e: ") and "experts:" in line
    model[0].timers.record_token_counts([5, 9, 2], [4, 4, 8])
    assert forward_breakdown(model)["tokens/max_rcv_count_per_rank"] == 9
