# SPDX-License-Identifier: Apache-2.0
"""Trainer smoke tests and checkpoint round trips on CPU (pattern of the reference's tests/trainer and
tests/checkpoint: a few iterations on a tiny random model; rebuild and compare weights bit for bit)."""

import json
from pathlib import Path

import pytest
import torch

from arctictraining_b200.config.trainer import get_config
from arctictraining_b200.registry import get_registered_trainer


def build(recipe):
    cfg = get_config(recipe)
    return get_registered_trainer(cfg.type)(cfg)


def test_sft_trainer_runs_and_logs_metrics(tiny_recipe, tmp_path):
    tr = build(tiny_recipe(exit_iteration=3))
    tr.train()
    assert tr.global_step == 3 and tr.early_stop
    rows = [json.loads(line) for line in Path(tr.config.train_log_metrics_path).read_text().splitlines()]
    assert [r["iter"] for r in rows] == [1, 2, 3]
    assert {"loss", "lr", "iter_time", "step_time", "seqlen", "epoch"} <= set(rows[0])


def test_overfit_first_batch_reduces_loss(tiny_recipe):
    tr = build(tiny_recipe(overfit_first_batch=True, exit_iteration=12, optimizer={"lr": 5e-3, "weight_decay": 0.0},
                           scheduler={"name": "constant"}))
    tr.train()
    rows = [json.loads(line) for line in Path(tr.config.train_log_metrics_path).read_text().splitlines()]
    assert rows[-1]["loss"] < rows[0]["loss"] - 0.5


def test_eval_interval_and_gradient_accumulation(tiny_recipe, tmp_path):
    data = {"sources": [{"type": "synthetic", "num_samples": 32, "min_length": 32, "max_length": 32}],
            "train_eval_split": [0.75, 0.25], "cache_dir": str(tmp_path / "c"), "max_length": 32, "dl_num_workers": 0}
    tr = build(tiny_recipe(data=data, eval_interval=2, gradient_accumulation_steps=2, exit_iteration=4))
    tr.train()
    assert tr.global_step == 4 and tr.train_batch_idx >= 8
    assert "loss/eval" in tr.metrics.summary_dict


def test_kill_switch_stops_training(tiny_recipe, tmp_path):
    tr = build(tiny_recipe(exit_iteration=0))
    Path(tr.config.kill_switch_path).write_text("stop")
    tr.train()
    assert tr.early_stop and "kill switch" in tr.early_stop_reason and tr.global_step == 0


def test_causal_trainer(tiny_recipe, tmp_path):
    from datasets import Dataset

    ds_dir = tmp_path / "text_ds"
    Dataset.from_dict({"text": [" ".join(f"w{i + j}" for j in range(60)) for i in range(24)]}).save_to_disk(str(ds_dir))
    data = {"sources": [{"type": "huggingface_causal", "name_or_path": str(ds_dir)}], "cache_dir": str(tmp_path / "c"),
            "max_length": 32, "dl_num_workers": 0}
    tr = build(tiny_recipe(type="causal", data=data, exit_iteration=2))
    batch = next(iter(tr.train_dataloader))
    assert batch["input_ids"].shape == (2, 32) and torch.equal(batch["input_ids"], batch["labels"])
    tr.train()
    assert tr.global_step == 2


def test_dpo_trainer(tiny_recipe, tmp_path):
    r = tiny_recipe(type="dpo", micro_batch_size=1, ref_model={"name_or_path": "tiny-llama", "dtype": "fp32"},
                    data={"sources": [{"type": "synthetic_dpo", "num_samples": 16, "words_per_message": 6}],
                          "cache_dir": str(tmp_path / "c"), "max_length": 64, "dl_num_workers": 0},
                    exit_iteration=2, beta=0.5)
    tr = build(r)
    batch = next(iter(tr.train_dataloader))
    first = float(tr.loss(batch))
    assert first == pytest.approx(0.6931, abs=1e-3)  # policy == reference at the start: -log(sigmoid(0))
    tr.train()
    assert tr.global_step == 2


def test_dpo_fused_logprobs_match_plain_logits(tiny_recipe, tmp_path):
    from arctictraining_b200.trainer.dpo import get_logprobs

    r = tiny_recipe(type="dpo", micro_batch_size=1, ref_model={"name_or_path": "tiny-llama", "dtype": "fp32"},
                    data={"sources": [{"type": "synthetic_dpo", "num_samples": 8, "words_per_message": 6}],
                          "cache_dir": str(tmp_path / "c"), "max_length": 64, "dl_num_workers": 0})
    tr = build(r)
    batch = next(iter(tr.train_dataloader))
    lp, n = tr.sequence_logprobs(tr.model, batch)
    logits = tr.model(input_ids=batch["input_ids"], return_logits=True).logits.float()
    ref_lp, ref_n = get_logprobs(logits, batch["labels"], -100)
    assert torch.allclose(lp, ref_lp, atol=1e-3) and torch.equal(n, ref_n)


def _force_checkpoint(tr):
    tr.global_step_this_run = 1
    tr.training_finished = True
    tr.checkpoint()


@pytest.mark.parametrize("stage", [0, 2, 3])
def test_sharded_checkpoint_resume_is_bit_exact(tiny_recipe, tmp_path, stage):
    ck = [{"type": "deepspeed", "output_dir": str(tmp_path / "ck"), "auto_resume": True, "save_every_n_steps": 2}]
    a = build(tiny_recipe(checkpoint=ck, exit_iteration=2, deepspeed={"zero_optimization": {"stage": stage}}))
    a.train()
    assert (tmp_path / "ck" / "latest").read_text().startswith("epoch_0_global_step_2")
    b = build(tiny_recipe(checkpoint=ck, exit_iteration=4, seed=99, deepspeed={"zero_optimization": {"stage": stage}}))
    assert b.is_resume is False or b.global_step == 2  # resume consumed
    assert b.global_step == 2 and b.model.global_steps == 2
    pa = dict(a.model.iter_full_named_parameters())
    pb = dict(b.model.iter_full_named_parameters())
    assert all(torch.equal(pa[n], pb[n]) for n in pa)
    b.train()
    assert b.global_step == 4


def test_hf_checkpoint_reloads_into_an_identical_model(tiny_recipe, tmp_path):
    ck = [{"type": "huggingface", "output_dir": str(tmp_path / "hf"), "save_end_of_training": True}]
    a = build(tiny_recipe(checkpoint=ck, exit_iteration=2, deepspeed={"zero_optimization": {"stage": 3}}))
    a.train()
    out = tmp_path / "hf" / "global_step_2"
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    from safetensors.torch import load_file

    names = set(load_file(str(out / "model.safetensors")))
    assert "model.layers.0.self_attn.q_proj.weight" in names and "model.layers.1.mlp.up_proj.weight" in names
    b = build(tiny_recipe(model={"name_or_path": str(out), "dtype": "fp32"}, seed=5))
    pa = dict(a.model.iter_full_named_parameters())
    pb = dict(b.model.iter_full_named_parameters())
    assert all(torch.equal(pa[n], pb[n]) for n in pa)


def test_lora_trains_only_adapters_and_exports_them(tiny_recipe, tmp_path):
    """Adapters of the requested Hugging Face modules only (k_proj shares a fused weight with q_proj and v_proj and must
    stay untouched), exported as ``adapter_model.safetensors`` + ``adapter_config.json`` in the PEFT key layout; the
    exported A / B pairs reproduce the update the model applies."""
    import json

    from safetensors.torch import load_file

    from arctictraining_b200.models.peft import merged_weight_delta

    ck = [{"type": "huggingface", "output_dir": str(tmp_path / "hf"), "save_end_of_training": True}]
    tr = build(tiny_recipe(model={"peft_config": {"peft_type": "LORA", "r": 4, "lora_alpha": 8,
                                                  "target_modules": ["q_proj", "v_proj", "down_proj", "up_proj"]}},
                           checkpoint=ck, exit_iteration=2, optimizer={"lr": 1e-2}))
    trainable = [n for n, p in tr.model_unwrapped.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    assert not any(n.endswith(("lora_A.k_proj", "lora_A.gate_proj")) for n in trainable)
    tr.train()
    out = tmp_path / "hf" / "global_step_2"
    saved = load_file(str(out / "adapter_model.safetensors"))
    cfg = json.loads((out / "adapter_config.json").read_text())
    assert cfg["peft_type"] == "LORA" and cfg["r"] == 4 and sorted(cfg["target_modules"]) == ["down_proj", "q_proj", "up_proj", "v_proj"]
    assert not (out / "model.safetensors").exists()
    key = "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"
    assert key in saved and saved[key].shape[0] == 4
    assert "base_model.model.model.layers.0.mlp.up_proj.lora_B.weight" in saved
    assert not any(".k_proj." in k or ".gate_proj." in k or "qkv_proj" in k for k in saved)
    # B A * alpha / r from the file equals the update of the live model, module by module
    want = merged_weight_delta(tr.model_unwrapped)
    assert want
    for mod, delta in want.items():
        a = saved[f"base_model.model.{mod}.lora_A.weight"].float()
        b = saved[f"base_model.model.{mod}.lora_B.weight"].float()
        if delta.numel():
            torch.testing.assert_close(b @ a * (8 / 4), delta.cpu(), atol=1e-6, rtol=1e-5)
    assert any(float(saved[k].abs().max()) > 0 for k in saved if ".lora_B." in k), "the adapters did not train"


def test_lora_update_touches_only_the_rows_of_the_requested_projections():
    from arctictraining_b200.models.arch import load_arch_config
    from arctictraining_b200.models.causal_lm import CausalLM
    from arctictraining_b200.models.peft import apply_lora

    m = CausalLM(load_arch_config("tiny-llama", {}), dtype=torch.float32)
    m.init_weights(seed=0)
    attn = m.model.layers[0].self_attn
    x = torch.randn(2, 8, attn.qkv_proj.weight.shape[1])
    before = attn.qkv_proj(x)
    apply_lora(m, {"r": 2, "target_modules": ["v_proj"]})
    lora = m.model.layers[0].self_attn.qkv_proj
    with torch.no_grad():
        lora.lora_B["v_proj"].normal_()
    after = lora(x)
    hq, hkv, d = attn.hq, attn.hkv, attn.d
    changed = (after - before).abs().amax(dim=(0, 1)) > 0
    assert not changed[: (hq + hkv) * d].any() and changed[(hq + hkv) * d :].all()


def test_callbacks_declared_on_a_custom_trainer_fire(tiny_recipe):
    from arctictraining_b200 import SFTTrainer

    seen = []

    class CountingTrainer(SFTTrainer):
        name = "counting-sft-test"

        def post_step_callback(self):
            seen.append(self.global_step)

        def pre_loss_callback(self, batch):
            seen.append("loss")
            return batch

    tr = build(tiny_recipe(type="counting-sft-test", exit_iteration=2))
    tr.train()
    assert seen == ["loss", 1, "loss", 2]


def test_cli_run_with_autocast_and_bf16_states(tiny_recipe, tmp_path):
    """The reference's autocast test (tests/trainer/test_autocast.py:30-113) through the real command line: ZeRO-3,
    bf16 master weights / gradients / optimizer states and ``torch_autocast``; both iterations are logged and the first
    loss is sane."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    import yaml

    root = Path(__file__).resolve().parent.parent
    r = tiny_recipe(exit_iteration=2, train_log_iter_interval=1, micro_batch_size=1, logger={"level": "INFO"})
    r["deepspeed"] = {"zero_optimization": {"stage": 3},
                      "bf16": {"enabled": True, "bf16_master_weights_and_grads": True, "bf16_optimizer_states": True},
                      "torch_autocast": {"enabled": True, "dtype": "torch.bfloat16"}}
    r["model"]["dtype"] = "bf16"
    path = tmp_path / "autocast.yaml"
    path.write_text(yaml.safe_dump(r))
    res = subprocess.run([sys.executable, "-m", "arctictraining_b200.cli", str(path), "--num_gpus", "1", "--master_port", "29733"],
                         cwd=root, env={**os.environ, "PYTHONPATH": str(root)}, capture_output=True, text=True, timeout=600)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-3000:]
    assert "iter: 1/2" in out and "iter: 2/2" in out and "iter: 3/2" not in out
    logs = [json.loads(x) for x in Path(r["train_log_metrics_path"]).read_text().splitlines() if x.strip()]
    assert logs[0]["iter"] == 1 and 0 < logs[0]["loss"] < 20


def test_damaged_checkpoints_are_refused_with_the_file_named(tiny_recipe, tmp_path):
    """Host-side failure injection: a shard cut short by a job that died while copying it, and a ``latest`` tag that
    names a directory which is gone.  Resuming must stop with the offending file in the message, not continue on
    fresh weights; and a save leaves no temporary files behind."""
    from arctictraining_b200.exceptions import CheckpointError

    ck = [{"type": "deepspeed", "output_dir": str(tmp_path / "ck"), "auto_resume": True, "save_every_n_steps": 2}]
    a = build(tiny_recipe(checkpoint=ck, exit_iteration=2))
    a.train()
    tag = (tmp_path / "ck" / "latest").read_text().strip()
    d = tmp_path / "ck" / tag
    assert not list(d.glob("*.tmp"))
    shard = next(d.glob("zero_pp_rank_0_*optim_states.pt"))
    whole = shard.read_bytes()
    shard.write_bytes(whole[: len(whole) // 3])
    with pytest.raises(CheckpointError, match="zero_pp_rank_0"):
        build(tiny_recipe(checkpoint=ck, exit_iteration=4))
    shard.write_bytes(whole)
    build(tiny_recipe(checkpoint=ck, exit_iteration=4))        # intact again: resumes
    (tmp_path / "ck" / "latest").write_text("epoch_9_global_step_99")
    with pytest.raises(CheckpointError, match="epoch_9_global_step_99"):
        build(tiny_recipe(checkpoint=ck, exit_iteration=4))


def test_eval_loss_is_reported_or_kept_according_to_the_log_interval(tiny_recipe, tmp_path):
    """``eval_interval: 1``: the evaluation loss of the last step is in the summary and no longer pending.  With
    ``eval_log_iter_interval: 2`` and three steps the loss of step 3 was recorded but not reported (pattern of the
    reference's tests/trainer/test_sft_trainer.py)."""
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    def run(**extra):
        r = tiny_recipe(**{"exit_iteration": 2, "eval_interval": 1, **extra})
        r["data"]["train_eval_split"] = [0.8, 0.2]
        r["data"]["cache_dir"] = str(tmp_path / f"cache{len(extra)}")
        trainer = get_registered_trainer("sft")(get_config(r))
        trainer.train()
        return trainer

    t = run()
    assert t.metrics.summary_dict["loss/eval"] > 0 and "loss/eval" not in t.metrics.values
    t = run(exit_iteration=3, eval_log_iter_interval=2)
    assert "loss/eval" in t.metrics.values and "loss/eval" not in t.metrics.summary_dict


def test_train_iters_sets_the_horizon_and_runs_over_epoch_boundaries(tiny_recipe):
    """``train_iters`` replaces ``epochs``: 32 samples at batch 2 are 16 steps per epoch; 20 steps need a second epoch."""
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    r = tiny_recipe(train_iters=20, exit_iteration=0, epochs=1)
    trainer = get_registered_trainer("sft")(get_config(r))
    assert trainer.training_horizon == 20 and len(trainer.train_dataloader) == 16
    trainer.train()
    assert trainer.global_step == 20 and trainer.epoch_idx >= 1


def test_loss_log_interval_and_epoch_checkpoints(tiny_recipe, tmp_path):
    """``loss_log_interval: 2`` logs the loss of every second step; ``save_every_n_epochs: 1`` writes one export at the
    end of each epoch (the directory is named after the global step)."""
    from loguru import logger as loguru_logger

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    r = tiny_recipe(exit_iteration=0, epochs=2, loss_log_interval=2,
                    checkpoint=[{"type": "huggingface", "output_dir": str(tmp_path / "hf"), "save_every_n_epochs": 1}])
    r["data"]["sources"][0]["num_samples"] = 8  # 4 steps per epoch
    lines = []
    sink = loguru_logger.add(lambda m: lines.append(str(m)), level="INFO")
    try:
        trainer = get_registered_trainer("sft")(get_config(r))
        trainer.train()
    finally:
        loguru_logger.remove(sink)
    assert trainer.global_step == 8
    logged = sorted(int(ln.split("Global Step: ")[1].split("/")[0]) for ln in lines if "Global Step:" in ln)
    assert logged and all(step % 2 == 0 for step in logged)
    assert sorted(p.name for p in (tmp_path / "hf").iterdir() if p.is_dir()) == ["global_step_4", "global_step_8"]


def test_entrypoint_profile_option_prints_a_profile_and_trains(tiny_recipe, tmp_path, capsys, monkeypatch):
    import yaml

    from arctictraining_b200 import entrypoint

    r = tiny_recipe(exit_iteration=2)
    path = tmp_path / "r.yaml"
    path.write_text(yaml.safe_dump(r))
    monkeypatch.setenv("LOCAL_RANK", "0")
    entrypoint.launch(["--config", str(path), "--python_profile", "tottime"])
    out = capsys.readouterr().out
    assert "function calls" in out and "tottime" in out
    assert (tmp_path / "metrics.jsonl").read_text().count("\n") >= 2


def test_library_architecture_trains_checkpoints_and_reloads(tiny_recipe, tmp_path):
    """An architecture this package has no own implementation of (OLMo-2 through the transformers library): ZeRO-3
    training with tiled MLP and LoRA off, Hugging Face export, and the export loads back into the library's class with
    the trained weights."""
    from transformers import AutoModelForCausalLM
    from transformers import Olmo2Config

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    arch = tmp_path / "tiny-olmo2"
    Olmo2Config(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=256).save_pretrained(arch)
    r = tiny_recipe(
        exit_iteration=3, tiled_mlp_compute=True,
        model={"name_or_path": str(arch), "dtype": "fp32", "attn_implementation": "sdpa",
               "hf_config_kwargs": {"num_hidden_layers": 2}},
        tokenizer={"type": "fake", "name_or_path": "tiny-llama"},
        checkpoint=[{"type": "huggingface", "output_dir": str(tmp_path / "hf"), "save_end_of_training": True}])
    r["deepspeed"] = {"zero_optimization": {"stage": 3}}
    trainer = get_registered_trainer("sft")(get_config(r))
    assert type(trainer.model_unwrapped).__name__ == "Olmo2ForCausalLM"
    before = {n: t.clone() for n, t in trainer.model.iter_full_named_parameters()}
    trainer.train()
    after = {n: t.clone() for n, t in trainer.model.iter_full_named_parameters()}
    assert any(not torch.equal(before[n], after[n]) for n in before)
    out = next((tmp_path / "hf").iterdir())
    reloaded = AutoModelForCausalLM.from_pretrained(out)
    assert reloaded.config.num_hidden_layers == 2
    state = reloaded.state_dict()
    for n, t in after.items():
        torch.testing.assert_close(state[n].float(), t.float(), msg=lambda m, n=n: f"{n}: {m}")


def test_library_model_layers_are_computed_twice_per_step_and_inputs_go_through_the_store(tiny_recipe, tmp_path):
    """The engine checkpoints the decoder layers of a transformers model itself: one forward and one recomputation per
    step (the library's own checkpointing flag must not add a third), and with the offload switch the layer inputs are
    handed to the activation store."""
    from transformers import Olmo2Config

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    arch = tmp_path / "tiny-olmo2"
    Olmo2Config(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=256).save_pretrained(arch)
    r = tiny_recipe(exit_iteration=2, activation_checkpoint_cpu_offload=True,
                    model={"name_or_path": str(arch), "dtype": "fp32", "attn_implementation": "sdpa",
                           "hf_config_kwargs": {"num_hidden_layers": 2}},
                    tokenizer={"type": "fake", "name_or_path": "tiny-llama"})
    trainer = get_registered_trainer("sft")(get_config(r))
    calls, saved = [0], [0]
    trainer.model_unwrapped.model.layers[0].mlp.register_forward_hook(lambda *a: calls.__setitem__(0, calls[0] + 1))
    store = trainer.model.act_store
    original_save = store.save
    store.save = lambda x: (saved.__setitem__(0, saved[0] + 1), original_save(x))[1]
    trainer.train()
    assert calls[0] == 2 * trainer.global_step
    assert saved[0] >= 2 * trainer.global_step  # two layers per step


def test_custom_model_factory_builds_a_library_model_from_the_architecture_config(tiny_recipe, tmp_path):
    """Pattern of the reference's test helper (tests/helpers.py: a model factory that overrides ``create_model`` and
    builds a random-weight model through the transformers library): the architecture config converts with ``to_hf()``,
    and the resulting Llama model of the library trains on this package's engine."""
    from transformers import AutoModelForCausalLM

    from arctictraining_b200 import HFModelFactory
    from arctictraining_b200 import SFTTrainer
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import RegistryMeta
    from arctictraining_b200.registry import get_registered_trainer

    class RandomWeightHFModelFactory(HFModelFactory):
        name = "random-weight-hf-test"

        def create_model(self, model_config):
            torch.manual_seed(11)
            assert self.config.dtype == torch.float32 and self.config.dtype == "fp32"
            return AutoModelForCausalLM.from_config(model_config.to_hf(), attn_implementation="sdpa",
                                                    dtype=self.config.dtype.value)

    class LibraryLlamaTrainer(SFTTrainer):
        name = "sft-library-llama-test"
        model_factory: RandomWeightHFModelFactory

    try:
        r = tiny_recipe(type="sft-library-llama-test", exit_iteration=3, model={"type": "random-weight-hf-test"})
        trainer = get_registered_trainer("sft-library-llama-test")(get_config(r))
        assert type(trainer.model_unwrapped).__module__.startswith("transformers.")
        assert trainer.model_unwrapped.config.num_hidden_layers == trainer.model_unwrapped.config.num_hidden_layers > 0
        trainer.train()
        assert trainer.global_step == 3
    finally:
        RegistryMeta._registry["ModelFactory"].pop("random-weight-hf-test", None)
        RegistryMeta._registry["Trainer"].pop("sft-library-llama-test", None)


def test_trainers_without_sequence_parallel_support_refuse_the_setting(tiny_recipe, tmp_path):
    """A trainer whose loss needs whole sequences (DPO, speculators, biencoder) says so instead of training on slices."""
    r = tiny_recipe(type="dpo", micro_batch_size=1, ref_model={"name_or_path": "tiny-llama", "dtype": "fp32"},
                    data={"sources": [{"type": "synthetic_dpo", "num_samples": 16, "words_per_message": 6}],
                          "cache_dir": str(tmp_path / "c"), "max_length": 64, "dl_num_workers": 0},
                    sequence_parallel_size=2)
    with pytest.raises(ValueError, match="does not support sequence_parallel_size=2"):
        build(r)
    from arctictraining_b200 import CausalTrainer
    from arctictraining_b200 import DPOTrainer
    from arctictraining_b200 import SFTTrainer

    assert SFTTrainer.supports_sequence_parallel and CausalTrainer.supports_sequence_parallel
    assert not DPOTrainer.supports_sequence_parallel


def test_export_of_a_package_wrapped_adapter_model_hands_gathered_tensors_to_its_writer(tmp_path):
    """A transformers model wrapped by the adapter package is exported by that package's ``save_pretrained``; it gets
    the trainable tensors as gathered by the engine, not the module's own (possibly released) parameters."""
    from types import SimpleNamespace

    from arctictraining_b200.checkpoint.hf import HFCheckpointEngine

    calls = {}

    class Wrapped(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.base = torch.nn.Linear(4, 4)
            self.lora_A = torch.nn.Parameter(torch.ones(2, 4))
            self.base.weight.requires_grad_(False)
            self.base.bias.requires_grad_(False)

        def save_pretrained(self, out_dir, state_dict=None, safe_serialization=True):
            calls.update(out_dir=out_dir, names=sorted(state_dict), safe=safe_serialization,
                         value=state_dict["lora_A"].clone())

    Wrapped.__module__ = "peft.peft_model"
    module = Wrapped()
    engine_view = SimpleNamespace(module=module, iter_full_named_parameters=lambda: iter(
        [("base.weight", module.base.weight.data), ("base.bias", module.base.bias.data), ("lora_A", torch.full((2, 4), 7.0))]))
    fake_self = SimpleNamespace(trainer=SimpleNamespace(tokenizer=None, config=SimpleNamespace(model=SimpleNamespace(name_or_path="x"))))
    HFCheckpointEngine._save_adapter(fake_self, engine_view, module, tmp_path / "out", True)
    assert calls["names"] == ["lora_A"] and calls["safe"] is True and calls["out_dir"] == str(tmp_path / "out")
    assert torch.all(calls["value"] == 7.0)  # the gathered tensor, not the module's parameter


def test_liger_type_puts_own_ops_into_a_library_model_without_changing_the_numbers(tiny_recipe, tmp_path):
    """``model.type: liger`` on a transformers architecture: RMSNorm modules call this package's op and the loss comes
    from the fused output projection + cross-entropy; losses and updated weights equal the plain ``huggingface`` run."""
    from transformers import Olmo2Config

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    arch = tmp_path / "tiny-olmo2"
    Olmo2Config(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=256).save_pretrained(arch)

    def run(kind):
        r = tiny_recipe(exit_iteration=3,
                        model={"type": kind, "name_or_path": str(arch), "dtype": "fp32", "attn_implementation": "sdpa",
                               "hf_config_kwargs": {"num_hidden_layers": 2}},
                        tokenizer={"type": "fake", "name_or_path": "tiny-llama"})
        r["data"]["cache_dir"] = str(tmp_path / "cache")
        r["train_log_metrics_path"] = str(tmp_path / f"{kind}.jsonl")
        trainer = get_registered_trainer("sft")(get_config(r))
        trainer.train()
        losses = [json.loads(line)["loss"] for line in (tmp_path / f"{kind}.jsonl").read_text().splitlines() if line.strip()]
        return trainer, losses, {n: t.clone() for n, t in trainer.model.iter_full_named_parameters()}

    plain, plain_losses, plain_params = run("huggingface")
    fused, fused_losses, fused_params = run("liger")
    assert not getattr(plain.model_unwrapped, "_atb_fused_loss", False) and fused.model_unwrapped._atb_fused_loss
    patched = [m for m in fused.model_unwrapped.modules() if getattr(m, "_atb_eps", None) is not None]
    assert len(patched) >= 5  # two per layer and the final norm
    assert fused_losses == pytest.approx(plain_losses, rel=1e-5)
    for n, t in plain_params.items():
        torch.testing.assert_close(fused_params[n], t, rtol=1e-4, atol=1e-6, msg=lambda m, n=n: f"{n}: {m}")
