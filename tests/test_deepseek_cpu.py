# SPDX-License-Identifier: Apache-2.0
"""The native DeepSeek-V2 family (multi-head latent attention, routed + shared experts) against the Hugging Face
implementation on a tiny random model, through the checkpoint converters in both directions."""

import pytest
import torch

from arctictraining_b200.models.arch import load_arch_config
from arctictraining_b200.models.deepseek import DeepseekV2ForCausalLM
from arctictraining_b200.models.deepseek import permute_rotary_rows
from arctictraining_b200.models.hf_io import hf_to_native_state_dict
from arctictraining_b200.models.hf_io import iter_hf_tensors
from arctictraining_b200.ops import reference as ref

transformers = pytest.importorskip("transformers")


def hf_model(cfg, **extra):
    from transformers import DeepseekV2Config
    from transformers import DeepseekV2ForCausalLM as HFModel

    keys = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size",
            "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "head_dim", "n_routed_experts",
            "num_experts_per_tok", "moe_intermediate_size", "n_shared_experts", "first_k_dense_replace", "norm_topk_prob",
            "routed_scaling_factor", "topk_method", "n_group", "topk_group", "rms_norm_eps", "max_position_embeddings")
    kw = {k: cfg[k] for k in keys}
    kw.update(extra)
    hf_cfg = DeepseekV2Config(**kw, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, attn_implementation="eager")
    torch.manual_seed(0)
    m = HFModel(hf_cfg).float().eval()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
        for n, p in m.named_parameters():
            if "norm" in n:
                p.fill_(1.0).add_(0.1 * torch.randn_like(p))
    return m


def per_expert_state_dict(m):
    """The hub layout: one gate/up/down triple per expert (the in-memory model of recent transformers stacks them)."""
    sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):
            pre = k[: -len("gate_up_proj")]
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, dim=0)
                sd[f"{pre}{e}.gate_proj.weight"], sd[f"{pre}{e}.up_proj.weight"] = g.clone(), u.clone()
        elif k.endswith("mlp.experts.down_proj"):
            pre = k[: -len("down_proj")]
            for e in range(v.shape[0]):
                sd[f"{pre}{e}.down_proj.weight"] = v[e].clone()
        else:
            sd[k] = v.clone()
    return sd


@pytest.mark.parametrize("variant", ["low_rank_q", "full_q_group_limited"])
def test_logits_match_hugging_face_and_export_round_trips(variant):
    over = {}
    if variant == "full_q_group_limited":
        over = dict(q_lora_rank=None, topk_method="group_limited_greedy", n_group=4, topk_group=2, routed_scaling_factor=2.5)
    cfg = load_arch_config("tiny-deepseek-v2", over)
    hf = hf_model(cfg)
    for layer in hf.model.layers:  # the library's group-limited branch reads an attribute its module never sets
        if hasattr(layer.mlp, "experts"):
            layer.mlp.num_experts = cfg["n_routed_experts"]
    sd = per_expert_state_dict(hf)
    native = DeepseekV2ForCausalLM(cfg, dtype=torch.float32)
    missing, unexpected = native.load_state_dict(hf_to_native_state_dict(dict(sd), cfg), strict=True), None
    native.eval()
    ids = torch.randint(0, cfg["vocab_size"], (2, 12))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = native(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())
    # export: native -> HF names gives back exactly what was loaded
    back = dict(iter_hf_tensors(((n, p.data) for n, p in native.named_parameters()), cfg))
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k]), k


def test_rotary_row_permutation_is_its_own_inverse_and_keeps_dot_products():
    cfg = load_arch_config("tiny-deepseek-v2")
    w = torch.randn(cfg["num_attention_heads"] * (cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"]), 5)
    assert torch.equal(permute_rotary_rows(permute_rotary_rows(w, cfg, "q"), cfg, "q", inverse=True), w)
    a = torch.randn(cfg["kv_lora_rank"] + cfg["qk_rope_head_dim"], 5)
    assert torch.equal(permute_rotary_rows(permute_rotary_rows(a, cfg, "kv_a"), cfg, "kv_a", inverse=True), a)
    assert torch.equal(permute_rotary_rows(a, cfg, "kv_a")[: cfg["kv_lora_rank"]], a[: cfg["kv_lora_rank"]])


def test_yarn_tables_match_hugging_face():
    from transformers import DeepseekV2Config
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    scaling = dict(rope_type="yarn", factor=40.0, original_max_position_embeddings=4096, beta_fast=32, beta_slow=1, mscale=0.707,
                   mscale_all_dim=0.707)
    hf_cfg = DeepseekV2Config(head_dim=64, qk_rope_head_dim=64, max_position_embeddings=163840,
                              rope_parameters=dict(scaling, rope_theta=10000.0))
    inv, amp = ROPE_INIT_FUNCTIONS["yarn"](hf_cfg, "cpu")
    pos = torch.tensor([[0, 1, 777, 50000]])
    cos, sin = ref.rope_cos_sin(pos, 64, 10000.0, scaling)
    ang = pos.float().unsqueeze(-1) * inv
    assert torch.allclose(cos, ang.cos() * amp, atol=1e-5) and torch.allclose(sin, ang.sin() * amp, atol=1e-5)
    assert abs(amp - 1.0) < 1e-6  # equal mscale and mscale_all_dim cancel; the softmax scale carries mscale^2 instead


def test_trains_and_generates(tmp_path):
    from arctictraining_b200.models.generation import generate

    cfg = load_arch_config("tiny-deepseek-v2")
    torch.manual_seed(0)
    m = DeepseekV2ForCausalLM(cfg, dtype=torch.float32)
    m.init_weights(seed=1)
    ids = torch.randint(0, cfg["vocab_size"], (2, 16))
    out = m(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.isfinite(out.loss) and all(p.grad is not None for n, p in m.named_parameters() if "expert_" not in n)
    m.eval()
    with torch.no_grad():
        gen, _ = generate(m, ids[:1, :8], max_new_tokens=3, do_sample=False)
        step = m(input_ids=gen[:, :-1]).logits.argmax(-1)
    assert torch.equal(gen[:, 8:], step[:, 7:])  # cached decoding equals re-scoring the whole prefix
