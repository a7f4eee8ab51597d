# SPDX-License-Identifier: Apache-2.0
from abc import ABC
from abc import abstractmethod

import pytest

from arctictraining_b200.exceptions import RegistryError
from arctictraining_b200.exceptions import RegistryValidationError
from arctictraining_b200.registry import RegistryMeta
from arctictraining_b200.registry import _get_class_attr_type_hints
from arctictraining_b200.registry import _validate_class_attribute_type
from arctictraining_b200.registry import _validate_class_method
from arctictraining_b200.registry import get_registered_class
from arctictraining_b200.registry import register


def make_base(base_name):
    ns = {
        "_validate_subclass": classmethod(lambda cls: None),
        "work": abstractmethod(lambda self, x: x),
    }
    return RegistryMeta(base_name, (ABC,), ns)


def test_subclasses_register_under_their_root_and_name():
    Base = make_base("RegBaseA")

    class One(Base):
        name = "one"

        def work(self, x):
            return x

    class Two(One):
        name = "two"

    assert get_registered_class("RegBaseA", "one") is One
    assert get_registered_class("RegBaseA", "two") is Two
    with pytest.raises(RegistryError):
        get_registered_class("RegBaseA", "three")
    with pytest.raises(RegistryError):
        get_registered_class("NoSuchBase", "one")


def test_base_class_is_not_registered_and_name_is_required():
    Base = make_base("RegBaseB")
    assert "RegBaseB" not in RegistryMeta._registry or not RegistryMeta._registry["RegBaseB"]
    with pytest.raises(RegistryValidationError):

        class Nameless(Base):
            def work(self, x):
                return x


def test_duplicate_name_is_rejected():
    Base = make_base("RegBaseC")

    class First(Base):
        name = "dup"

    with pytest.raises(RegistryValidationError):

        class Second(Base):
            name = "dup"


def test_validate_subclass_hook_runs_with_signature_and_type_checks():
    class Cfg:
        pass

    class OtherCfg:
        pass

    class Base(ABC, metaclass=RegistryMeta):
        name: str
        config: Cfg

        @classmethod
        def _validate_subclass(cls):
            _validate_class_attribute_type(cls, "config", Cfg)
            _validate_class_method(cls, "run", ["self", "batch"])

        def run(self, batch):
            return batch

    class Good(Base):
        name = "good-sig"
        config: Cfg

    with pytest.raises(RegistryValidationError):

        class BadSig(Base):
            name = "bad-sig"

            def run(self, batch, extra):
                return batch

    with pytest.raises(RegistryValidationError):

        class BadType(Base):
            name = "bad-type"
            config: OtherCfg

    assert get_registered_class("Base", "good-sig") is Good


def test_union_type_hints_are_flattened():
    from typing import Union

    class A:
        pass

    class B:
        pass

    class Holder:
        thing: Union[A, B]
        single: A

    assert _get_class_attr_type_hints(Holder, "thing") == (A, B)
    assert _get_class_attr_type_hints(Holder, "single") == (A,)
    assert _get_class_attr_type_hints(Holder, "missing") == ()


def test_multiple_inheritance_with_mixin_registers_once():
    Base = make_base("RegBaseD")

    class Mixin:
        def helper(self):
            return 1

    class Impl(Mixin, Base):
        name = "mixed"

    assert get_registered_class("RegBaseD", "mixed") is Impl


def test_register_decorator_is_a_noop():
    class Plain:
        pass

    assert register(Plain) is Plain
    assert register()(Plain) is Plain


def test_builtin_names_are_registered():
    import arctictraining_b200  # noqa: F401
    from arctictraining_b200 import registry as r

    assert r.get_registered_trainer("sft").__name__ == "SFTTrainer"
    assert r.get_registered_trainer("causal").__name__ == "CausalTrainer"
    assert r.get_registered_trainer("dpo").__name__ == "DPOTrainer"
    for n in ("huggingface", "liger"):
        r.get_registered_model_factory(n)
    for n in ("sft", "causal", "dpo"):
        r.get_registered_data_factory(n)
    for n in ("huggingface", "huggingface_instruct", "huggingface_causal", "snowflake", "ProjectGutenbergSFT",
              "HuggingFaceH4/ultrafeedback_binarized", "synthetic"):
        r.get_registered_data_source(n)
    for n in ("deepspeed", "huggingface"):
        r.get_registered_checkpoint_engine(n)
    for n in ("fused_adam", "cpu_adam", "fused_adam_moe", "cpu_adam_moe"):
        r.get_registered_optimizer_factory(n)
    for n in ("huggingface", "wds"):
        r.get_registered_scheduler_factory(n)
    for n in ("huggingface", "fake"):
        r.get_registered_tokenizer_factory(n)


def test_module_paths_of_the_reference_resolve_to_this_package():
    """User code imports the reference by its module paths; every one of them yields the (once registered) class of
    this package."""
    import importlib

    import arctic_training
    import arctictraining_b200 as impl
    import arctictraining_b200.synth  # noqa: F401 - the sub-package is not loaded by the top-level import

    pairs = [
        ("arctic_training.trainer.sft_trainer", "SFTTrainer", impl.SFTTrainer),
        ("arctic_training.trainer.causal_trainer", "CausalTrainer", impl.CausalTrainer),
        ("arctic_training.trainer.dpo_trainer", "DPOTrainer", impl.DPOTrainer),
        ("arctic_training.trainer.trainer", "Trainer", impl.Trainer),
        ("arctic_training.checkpoint.ds_engine", "DSCheckpointEngine", impl.DSCheckpointEngine),
        ("arctic_training.checkpoint.hf_engine", "HFCheckpointEngine", impl.HFCheckpointEngine),
        ("arctic_training.checkpoint.engine", "CheckpointEngine", impl.CheckpointEngine),
        ("arctic_training.model.hf_factory", "HFModelFactory", impl.HFModelFactory),
        ("arctic_training.model.liger_factory", "LigerModelFactory", impl.LigerModelFactory),
        ("arctic_training.model.factory", "ModelFactory", impl.ModelFactory),
        ("arctic_training.data.sft_factory", "SFTDataFactory", impl.SFTDataFactory),
        ("arctic_training.data.hf_instruct_source", "HFDataSourceInstruct", impl.HFDataSourceInstruct),
        ("arctic_training.data.snowflake_source", "SnowflakeDataSource", impl.SnowflakeDataSource),
        ("arctic_training.optimizer.adam_factory", "FusedAdamOptimizerFactory", impl.FusedAdamOptimizerFactory),
        ("arctic_training.scheduler.wsd_factory", "WSDSchedulerFactory", None),
        ("arctic_training.tokenizer.hf_factory", "HFTokenizerFactory", impl.HFTokenizerFactory),
        ("arctic_training.config.trainer", "TrainerConfig", impl.TrainerConfig),
        ("arctic_training.testing_utils", "TestCasePlus", None),
        ("arctic_training.model.moe.moe", "ArcticMoE", None),
        ("arctic_training.model.moe.moe_gemm", "group_gemm_fn", None),
        ("arctic_training.monkey_patches", "monkey_patch_checkpoint_function_with_cpu_offload", None),
        ("arctic_training.trainer.parallel_groups", "ParallelGroups", None),
        ("arctic_training.synth.base_caller", "BatchProcessor", impl.synth.BatchProcessor),
        ("arctic_training.synth.vllm_callers", "MultiReplicaVllmSynth", impl.synth.MultiReplicaVllmSynth),
        ("arctic_training.synth.vllm_utils", "launch_vllm_servers", None),
        ("arctic_training.synth.vllm_utils", "check_vllm_servers_health", None),
        ("arctic_training.synth.vllm_utils", "kill_processes", None),
        ("arctic_training.synth.utils", "recursive_to_dict", None),
        ("arctic_training.debug.utils", "print_rank0", None),
    ]
    for mod, name, expect in pairs:
        obj = getattr(importlib.import_module(mod), name)
        assert expect is None or obj is expect, (mod, name)
    assert arctic_training.CheckpointEngine is impl.CheckpointEngine
    with pytest.raises(ImportError):
        importlib.import_module("arctic_training.no_such_module")
