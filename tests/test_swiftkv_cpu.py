# SPDX-License-Identifier: Apache-2.0
from pathlib import Path

import pytest
import torch
import yaml

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture
def swiftkv_recipe(tiny_recipe, tmp_path):
    r = tiny_recipe(
        type="swiftkv",
        code=str(ROOT / "projects" / "swiftkv" / "train.py"),
        model={"name_or_path": "tiny-llama", "dtype": "fp32", "num_key_value_layers": 1, "key_value_group_size": 1,
               "hf_config_kwargs": {"num_hidden_layers": 3}},
        exit_iteration=3,
        optimizer={"lr": 1e-2, "weight_decay": 0.0},
    )
    r["deepspeed"] = {"zero_optimization": {"stage": 3}}
    p = tmp_path / "swiftkv.yaml"
    p.write_text(yaml.safe_dump(r))
    return p


def test_swiftkv_student_equals_teacher_at_init_and_trains(swiftkv_recipe):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    cfg = get_config(swiftkv_recipe)
    tr = get_registered_trainer(cfg.type)(cfg)
    model = tr.model_unwrapped
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("swiftkv" in n for n in trainable)

    batch = next(iter(tr.train_dataloader))
    batch.pop("packed_sample_seqlens")
    # key_value_group_size == 1 and copied projections: layer `nkv` itself reproduces the teacher exactly
    s_hidden, t_hidden = tr.forward(batch)
    assert torch.allclose(s_hidden[2], t_hidden[2], atol=1e-5)
    first = float(tr.loss(dict(batch)))
    before = {n: t.clone() for n, t in tr.model.iter_full_named_parameters()}
    tr.train()
    assert tr.global_step == 3
    after = dict(tr.model.iter_full_named_parameters())
    moved = [n for n in before if not torch.equal(before[n], after[n])]
    assert moved and all("swiftkv" in n for n in moved), "only SwiftKV parameters may change"
    assert first >= 0 and torch.isfinite(torch.tensor(first))


def test_swiftkv_hf_names(swiftkv_recipe):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.models import hf_io
    from arctictraining_b200.registry import get_registered_trainer

    cfg = get_config(swiftkv_recipe)
    tr = get_registered_trainer(cfg.type)(cfg)
    model = tr.model_unwrapped
    hf = dict(hf_io.iter_hf_tensors(tr.model.iter_full_named_parameters(), model.config))
    assert "model.layers.1.self_attn.k_proj_swiftkv.weight" in hf
    assert "model.layers.2.self_attn.q_proj_swiftkv.weight" in hf
    assert "model.norm_swiftkv.weight" in hf
    native = hf_io.hf_to_native_state_dict(hf, model.config)
    own = dict(tr.model.iter_full_named_parameters())
    assert set(native) == set(own)
    for n in own:
        assert torch.equal(native[n], own[n]), n


def test_sliding_window_layers_limit_the_keys_a_query_sees():
    """Qwen2-style configuration: layers from ``max_window_layers`` on attend to the last ``sliding_window`` keys only
    (the SwiftKV Qwen2 variant of the reference inherits this from the Qwen2 attention,
    projects/swiftkv/models/qwen2/modeling_qwen2_swiftkv.py)."""
    import torch

    from arctictraining_b200 import ops
    from arctictraining_b200.models.arch import load_arch_config
    from arctictraining_b200.models.causal_lm import CausalLM

    cfg = load_arch_config("tiny-llama", {"sliding_window": 8, "use_sliding_window": True, "max_window_layers": 1,
                                          "attention_bias": True})
    m = CausalLM(cfg, dtype=torch.float32)
    assert m.model.layers[0].self_attn.window is None and m.model.layers[1].self_attn.window == 8
    assert m.model.layers[0].self_attn.qkv_proj.bias is not None
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 32, 4, 16) for _ in range(3))
    full = ops.attention(q, k, v)
    win = ops.attention(q, k, v, window=8)
    assert torch.allclose(full[:, :8], win[:, :8], atol=1e-6)          # the first 8 queries see everything anyway
    assert not torch.allclose(full[:, 20:], win[:, 20:], atol=1e-4)
    # a far-away key has no influence inside the window
    k2, v2 = k.clone(), v.clone()
    k2[:, 0], v2[:, 0] = 5.0, -3.0
    assert torch.allclose(ops.attention(q, k2, v2, window=8)[:, 16:], win[:, 16:], atol=1e-6)
    cu = torch.tensor([0, 12, 32])
    packed = ops.attention(q, k, v, cu_seqlens=cu, window=8)
    assert torch.allclose(packed[:, 12:], ops.attention(q[:, 12:], k[:, 12:], v[:, 12:], window=8), atol=1e-6)


def test_swiftkv_on_the_deepseek_v2_latent_attention_family(tiny_recipe, tmp_path):
    """DeepSeek-V2 variant (projects/swiftkv/models/deepseek_v2/modeling_deepseek_swiftkv.py in the reference): the
    shared branch is the latent key/value projection; with groups of one the student equals the teacher at start."""
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.models import hf_io
    from arctictraining_b200.registry import get_registered_trainer

    r = tiny_recipe(
        type="swiftkv", code=str(ROOT / "projects" / "swiftkv" / "train.py"),
        model={"name_or_path": "tiny-deepseek-v2", "dtype": "fp32", "num_key_value_layers": 1, "key_value_group_size": 2},
        exit_iteration=2, optimizer={"lr": 1e-2, "weight_decay": 0.0},
    )
    r["deepspeed"] = {"zero_optimization": {"stage": 3}}
    p = tmp_path / "swiftkv_ds.yaml"
    p.write_text(yaml.safe_dump(r))
    cfg = get_config(p)
    tr = get_registered_trainer(cfg.type)(cfg)
    model = tr.model_unwrapped
    assert type(model).__name__ == "MLASwiftKVForCausalLM"
    trainable = [n for n, p_ in model.named_parameters() if p_.requires_grad]
    assert trainable and all("swiftkv" in n for n in trainable)
    hf = dict(hf_io.iter_hf_tensors(tr.model.iter_full_named_parameters(), model.config))
    for key in ("model.layers.1.self_attn.kv_a_proj_with_mqa_swiftkv.weight", "model.layers.1.self_attn.kv_b_proj_swiftkv.weight",
                "model.layers.1.self_attn.kv_a_layernorm_swiftkv.weight", "model.layers.2.self_attn.q_b_proj_swiftkv.weight",
                "model.layers.2.self_attn.q_a_layernorm_swiftkv.weight", "model.norm_swiftkv.weight",
                "model.layers.1.mlp.experts.0.gate_proj.weight", "model.layers.1.mlp.shared_experts.down_proj.weight"):
        assert key in hf, key
    assert "model.layers.2.self_attn.kv_b_proj_swiftkv.weight" not in hf  # layer 2 shares the branch of layer 1
    native = hf_io.hf_to_native_state_dict(dict(hf), model.config)
    own = dict(tr.model.iter_full_named_parameters())
    assert set(native) == set(own)
    assert all(torch.equal(native[n], own[n]) for n in own)

    batch = next(iter(tr.train_dataloader))
    batch.pop("packed_sample_seqlens")
    s_hidden, t_hidden = tr.forward(batch)
    # layer 1 is the first of its group: its keys/values are the mean of layers 1 and 2, so no exact equality; the
    # student must still be close to the teacher and the loss finite
    assert s_hidden[1] is t_hidden[1] or torch.equal(s_hidden[1], t_hidden[1])
    before = {n: t.clone() for n, t in tr.model.iter_full_named_parameters()}
    tr.train()
    after = dict(tr.model.iter_full_named_parameters())
    moved = [n for n in before if not torch.equal(before[n], after[n])]
    assert moved and all("swiftkv" in n for n in moved)
