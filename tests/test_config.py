# SPDX-License-Identifier: Apache-2.0
import textwrap

import pytest
import torch
import yaml
from pydantic import BaseModel
from pydantic import ValidationError

from arctictraining_b200.config.enums import DType
from arctictraining_b200.config.trainer import get_config
from arctictraining_b200.config.utils import HumanFloat
from arctictraining_b200.config.utils import HumanInt
from arctictraining_b200.config.utils import UniqueKeyLoader
from arctictraining_b200.config.utils import parse_human_val


@pytest.mark.parametrize(
    "text,expected",
    [("1k", 1e3), ("1.5K", 1500), ("2M", 2e6), ("1B", 1e9), ("1Ki", 1024), ("2Mi", 2 * 2**20), ("1Gi", 2**30),
     ("1e6", 1e6), ("1.5e3", 1500), ("10^6", 1e6), ("2^10", 1024), ("1_000", 1000), ("2.5%", 0.025), ("-3k", -3000),
     ("-2^2", -4), (7, 7), (0.5, 0.5), ("42", 42)],
)
def test_human_numbers(text, expected):
    assert parse_human_val(text) == pytest.approx(expected)


@pytest.mark.parametrize("bad", ["abc", "1kk", "k1", "1 k b", "^3"])
def test_invalid_human_numbers(bad):
    with pytest.raises(ValueError):
        parse_human_val(bad)


def test_human_types_in_pydantic_models():
    class M(BaseModel):
        a: HumanInt
        b: HumanFloat

    m = M(a="4Ki", b="1.5%")
    assert m.a == 4096 and m.b == pytest.approx(0.015)
    with pytest.raises(ValidationError):
        M(a="1.5", b=1)


@pytest.mark.parametrize("alias,dtype", [("bf16", torch.bfloat16), ("bfloat16", torch.bfloat16), ("fp16", torch.float16),
                                         ("half", torch.float16), ("float32", torch.float32), ("FP32", torch.float32)])
def test_dtype_aliases(alias, dtype):
    assert DType(alias).value == dtype
    assert DType(dtype).value == dtype


def test_dtype_rejects_unknown():
    with pytest.raises(ValueError):
        DType("int7")


def test_duplicate_yaml_keys_are_rejected():
    with pytest.raises(ValueError, match="Duplicate"):
        yaml.load("a: 1\nb: 2\na: 3\n", Loader=UniqueKeyLoader)


def test_get_config_fills_defaults_and_engine_section(tiny_recipe):
    recipe = tiny_recipe()
    recipe["deepspeed"] = {}
    cfg = get_config(recipe)
    assert cfg.type == "sft"
    assert cfg.model.type == "huggingface" and cfg.data.type == "sft"
    assert cfg.optimizer.type == "fused_adam" and cfg.scheduler.type == "huggingface"
    assert cfg.tokenizer.name_or_path == "tiny-llama"
    ds = cfg.deepspeed
    assert ds["train_micro_batch_size_per_gpu"] == 2 and ds["gradient_accumulation_steps"] == 1
    assert ds["zero_optimization"]["stage"] == 2  # default stage
    assert ds["zero_optimization"]["reduce_bucket_size"] == 64 * 64
    assert ds["gradient_clipping"] == 1.0
    assert cfg.data.sources[0].type == "synthetic" and cfg.data.sources[0].split == "train"


def test_max_length_defaults_to_model_positions(tiny_recipe):
    r = tiny_recipe()
    del r["data"]["max_length"]
    assert get_config(r).data.max_length == 2048


def test_incompatible_subconfig_type_is_rejected_unless_validation_is_skipped(tiny_recipe):
    r = tiny_recipe(data={"type": "dpo"})
    with pytest.raises(ValidationError):
        get_config(r)


def test_human_numbers_inside_engine_dict(tiny_recipe):
    cfg = get_config(tiny_recipe(deepspeed={"zero_optimization": {"stage": 3, "reduce_bucket_size": "5e8"}}))
    assert cfg.deepspeed["zero_optimization"]["reduce_bucket_size"] == 5e8
    assert cfg.zero_3_enabled


def test_extra_fields_are_forbidden(tiny_recipe):
    with pytest.raises(ValidationError):
        get_config(tiny_recipe(not_a_field=1))


def test_only_one_engine_may_auto_resume(tiny_recipe, tmp_path):
    ck = [{"type": "deepspeed", "output_dir": str(tmp_path / "a"), "auto_resume": True},
          {"type": "deepspeed", "output_dir": str(tmp_path / "b"), "auto_resume": True}]
    with pytest.raises((ValidationError, AssertionError)):
        get_config(tiny_recipe(checkpoint=ck))


def test_packing_requires_micro_batch_one(tiny_recipe):
    with pytest.raises((ValidationError, AssertionError)):
        get_config(tiny_recipe(data={"pack_samples": True}, micro_batch_size=2))


def test_user_module_next_to_recipe_is_imported_with_sibling_imports(tiny_recipe, tmp_path):
    (tmp_path / "helper_mod_xyz.py").write_text("VALUE = 41\n")
    (tmp_path / "train.py").write_text(textwrap.dedent("""
        from helper_mod_xyz import VALUE
        from arctictraining_b200 import SFTTrainer

        class MyTrainer(SFTTrainer):
            name = "my-sft-from-user-module"
            extra = VALUE + 1
    """))
    recipe = tiny_recipe(type="my-sft-from-user-module")
    path = tmp_path / "recipe.yaml"
    path.write_text(yaml.safe_dump(recipe))
    cfg = get_config(path)
    from arctictraining_b200.registry import get_registered_trainer

    assert cfg.type == "my-sft-from-user-module"
    assert get_registered_trainer(cfg.type).extra == 42


def test_missing_custom_code_file_raises(tiny_recipe):
    with pytest.raises(FileNotFoundError):
        get_config(tiny_recipe(code="/definitely/not/here.py"))


def test_every_shipped_recipe_validates(tmp_path, monkeypatch):
    """All recipes under projects/ build a typed config (trainer class found, sub-configs resolved, engine section
    built); only recipes that point at a checkpoint produced by an earlier stage are skipped."""
    import glob
    from pathlib import Path

    from arctictraining_b200.config.trainer import get_config

    root = Path(__file__).resolve().parent.parent
    monkeypatch.chdir(tmp_path)
    recipes = sorted(glob.glob(str(root / "projects" / "**" / "*.y*ml"), recursive=True))
    assert len(recipes) >= 20
    for path in recipes:
        if "/data/" in Path(path).read_text() and "excot" in path and "dpo" in Path(path).name:
            continue
        cfg = get_config(path)
        assert cfg.type, path
        assert cfg.deepspeed["train_micro_batch_size_per_gpu"] == cfg.micro_batch_size, path


def test_model_factory_works_with_a_stand_in_trainer():
    """Pattern of the reference's tests/model/test_hf_factory.py: the factory is built around a plain namespace that
    only carries the model config, and still creates the (LoRA-wrapped) model."""
    from types import SimpleNamespace

    from arctictraining_b200.config.model import ModelConfig

    config = ModelConfig(type="huggingface", name_or_path="tiny-llama", dtype="fp32",
                         peft_config={"peft_type": "Lora", "r": 4, "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj"]})
    assert config.peft_config_obj.r == 4
    model = config.factory(SimpleNamespace(config=SimpleNamespace(model=config)))()
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    with pytest.raises(ValueError):
        ModelConfig(type="huggingface", name_or_path="tiny-llama", peft_config={"peft_type": "invalid"})
