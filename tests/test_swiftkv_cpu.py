import sys
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
