# SPDX-License-Identifier: Apache-2.0
from pathlib import Path

import pytest
import torch
import yaml

ROOT = Path(__file__).resolve().parent.parent


def test_speculator_shapes_and_tied_weights():
    from arctictraining_b200.speculator import Speculator
    from arctictraining_b200.speculator import SpeculatorConfig

    for method, tie in (("sum_rnn", False), ("sum_rnn", True), ("sum_lstm", True)):
        cfg = SpeculatorConfig("x", 32, "48", "48", "48", 100, 3, tie_weights=tie, scale_input=True, method=method,
                               tie_lstm_embs=True)
        sp = Speculator(cfg)
        sp.reset_parameters()
        state = torch.randn(2, 10, 32)
        inds = torch.randint(0, 100, (2, 13))
        logits = sp(state, inds)
        assert logits.shape == (3, 2, 10, 100)
        if tie:
            assert sp.head[1].weight is sp.head[0].weight


@pytest.mark.parametrize("kind", ["arctic-lstm-speculator", "spec-decode"])
def test_speculator_trainer_runs_saves_and_only_trains_the_heads(tiny_recipe, tmp_path, kind):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    proj = "arctic_lstm_speculator" if kind == "arctic-lstm-speculator" else "mlp_speculator"
    model = {"name_or_path": "tiny-llama", "dtype": "fp32", "n_speculator_heads": 2, "speculator_width": 32,
             "disable_activation_checkpoint": True}
    if kind == "arctic-lstm-speculator":
        model.update(speculator_width="32", proj_dim="32", emb_dim="32", method="sum_lstm", speculator_tie_weights=True,
                     tie_lstm_embs=True)
    r = tiny_recipe(type=kind, code=str(ROOT / "projects" / proj / "train.py"), model=model, exit_iteration=3,
                    checkpoint=[{"type": kind, "output_dir": str(tmp_path / "spec"), "save_end_of_training": True}])
    r["deepspeed"] = {"zero_optimization": {"stage": 2}}
    p = tmp_path / "r.yaml"
    p.write_text(yaml.safe_dump(r))
    cfg = get_config(p)
    tr = get_registered_trainer(cfg.type)(cfg)
    before = {n: t.clone() for n, t in tr.model.iter_full_named_parameters()}
    tr.train()
    after = dict(tr.model.iter_full_named_parameters())
    moved = [n for n in before if not torch.equal(before[n], after[n])]
    assert moved and all(n.startswith("speculator.") for n in moved)
    saved = torch.load(tmp_path / "spec" / "pytorch_model.bin", weights_only=True)
    assert set(saved) == set(tr.model_unwrapped.speculator.state_dict())
    assert (tmp_path / "spec" / "config.json").exists()


def _spec_trainer(tiny_recipe, tmp_path, **extra):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    model = {"name_or_path": "tiny-llama", "dtype": "fp32", "n_speculator_heads": 2, "speculator_width": 32,
             "disable_activation_checkpoint": True}
    r = tiny_recipe(type="spec-decode", code=str(ROOT / "projects" / "mlp_speculator" / "train.py"), model=model, **extra)
    r["deepspeed"] = {"zero_optimization": {"stage": 3}}
    p = tmp_path / "r.yaml"
    p.write_text(yaml.safe_dump(r))
    cfg = get_config(p)
    return get_registered_trainer(cfg.type)(cfg)


def test_cached_generation_matches_full_reforward(tiny_recipe, tmp_path):
    """Greedy decoding with the key/value cache picks the tokens that re-running the whole sequence picks, and the
    hidden states it returns are those of a plain forward over the finished sequence."""
    tr = _spec_trainer(tiny_recipe, tmp_path, exit_iteration=1)
    prompts = torch.randint(8, 1000, (3, 9), generator=torch.Generator().manual_seed(0))
    want = tr.generate_continuations(prompts, 7)
    got, hidden = tr.generate(prompts, 7, do_sample=False)
    assert torch.equal(got, want)
    assert hidden.shape[:2] == (3, 9 + 7 - 1)
    full = tr.base_hidden_states({"input_ids": got})
    torch.testing.assert_close(hidden, full[:, : hidden.shape[1]], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("simple", [True, False])
def test_speculator_generation_modes_update_the_heads(tiny_recipe, tmp_path, simple):
    """``gen_train_simple``: one update per generated batch.  Otherwise one generation of ``gen_micro_batch_size``
    sequences feeds ``gen_micro_batch_size / gen_train_micro_batch_size`` speculator updates per data batch."""
    extra = dict(gen_train=True, gen_train_simple=simple, gen_prompt_length=8, gen_seq_length=12, exit_iteration=4,
                 micro_batch_size=2)
    extra.update(dict(gen_micro_batch_size=2, gen_train_micro_batch_size=2) if simple
                 else dict(gen_micro_batch_size=8, gen_train_micro_batch_size=4))
    tr = _spec_trainer(tiny_recipe, tmp_path, **extra)
    before = {n: t.clone() for n, t in tr.model.iter_full_named_parameters()}
    batch = next(iter(tr.train_dataloader))
    batch.pop("packed_sample_seqlens", None)
    steps0 = tr.model.global_steps
    tr.step(batch)
    assert tr.model.global_steps - steps0 == (1 if simple else 2)
    tr.metrics.values.clear()
    tr.step(batch)  # the learning rate of the very first update is zero (warm-up)
    after = dict(tr.model.iter_full_named_parameters())
    moved = [n for n in before if not torch.equal(before[n], after[n])]
    assert moved and all(n.startswith("speculator.") for n in moved)
