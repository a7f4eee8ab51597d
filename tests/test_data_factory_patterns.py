# SPDX-License-Identifier: Apache-2.0
"""The reference's data-factory test patterns (tests/data/test_sft_factory.py, test_source.py, test_factory.py), run
offline: a stand-in trainer object (plain namespace) around a data config, the hash tokenizer, synthetic sources, and
the reference's import paths."""
from types import SimpleNamespace

import pytest

from arctic_training.config.tokenizer import TokenizerConfig
from arctic_training.registry import _get_class_attr_type_hints
from arctic_training.registry import get_registered_data_factory


def create_data_factory(data_config_kwargs):
    from arctictraining_b200.tokenizer.factory import FakeTokenizer

    data_config_kwargs["type"] = data_config_kwargs.get("type", "sft")
    factory_cls = get_registered_data_factory(data_config_kwargs["type"])
    data_config_cls = _get_class_attr_type_hints(factory_cls, "config")[0]
    data_config = data_config_cls(**data_config_kwargs)
    trainer = SimpleNamespace(
        config=SimpleNamespace(micro_batch_size=1, data=data_config, seed=42, gradient_accumulation_steps=1,
                               tokenizer=TokenizerConfig(type="huggingface", name_or_path="tiny-llama"),
                               min_iterations=0, train_log_iter_interval=0, sequence_parallel_size=1),
        tokenizer=FakeTokenizer(1024), _set_seeds=lambda seed: None)
    return data_config.factory(trainer=trainer)


def test_padding_that_cannot_be_met_is_refused():
    with pytest.raises(ValueError, match=r"You have requested padding sequences"):
        create_data_factory(dict(type="sft", sources=["HuggingFaceH4/ultrachat_200k"], pad_to="max_length",
                                 max_length=13, div_length=7))


def test_cache_paths_are_unique_per_source_set_and_per_split(tmp_path):
    names = ["HuggingFaceH4/ultrachat_200k", "Open-Orca/SlimOrca"]
    both = create_data_factory(dict(type="sft", sources=names, eval_sources=names, cache_dir=tmp_path))
    one = create_data_factory(dict(type="sft", sources=names[:1], cache_dir=tmp_path))
    path_both = both.cache_path(both._get_data_sources(both.config.sources))
    path_one = one.cache_path(one._get_data_sources(one.config.sources))
    assert path_both != path_one
    per_source = [s.cache_path for s in both._get_data_sources(both.config.sources)] + [
        s.cache_path for s in both._get_data_sources(both.config.eval_sources)]
    assert len(per_source) == 4 and len(set(per_source)) == 4


def test_min_iterations_replicates_a_tiny_dataset(tmp_path):
    factory = create_data_factory(dict(
        type="sft", cache_dir=tmp_path, max_length=4096, pack_samples=False,
        sources=[{"type": "synthetic_messages", "num_samples": 1}]))
    factory.trainer.config.min_iterations = 20
    train_dl, eval_dl = factory()
    assert len(train_dl) == 20 and eval_dl is None


def test_generated_data_is_reproducible(tmp_path):
    """Same sources, two cache directories: the token streams are identical (a checksum of all ids)."""
    sums = []
    for sub in ("a", "b"):
        factory = create_data_factory(dict(
            type="sft", cache_dir=tmp_path / sub, max_length=4096,
            sources=[{"type": "synthetic_messages", "num_samples": 24}]))
        train_dl, _ = factory()
        pad = factory.tokenizer.pad_token_id
        sums.append(sum(int(x) for b in train_dl for x in b["input_ids"].flatten() if x != pad))
    assert sums[0] == sums[1] > 0


def _toy_conversations(n=20):
    from datasets import Dataset

    rows = [{"messages": [{"role": "user", "content": f"question number {i} about topic {i % 3}"},
                          {"role": "assistant", "content": f"answer number {i} with some more words"}],
             "prompt_id": str(i)} for i in range(n)]
    return Dataset.from_list(rows)


@pytest.mark.parametrize("with_split", [True, False])
def test_local_dataset_through_the_instruct_source(tmp_path, with_split):
    """A dataset saved to disk, with a ``train`` split or as a bare dataset, read through ``huggingface_instruct`` with a
    ``messages.role.<value>`` role mapping (tests/data/test_hf_source.py of the reference)."""
    from datasets import DatasetDict

    path = tmp_path / "local_chat"
    data = _toy_conversations()
    (DatasetDict(dict(train=data)) if with_split else data).save_to_disk(path.as_posix())
    factory = create_data_factory(dict(
        type="sft", cache_dir=tmp_path / "cache", max_length=4096, pack_samples=False,
        sources=[dict(type="huggingface_instruct", name_or_path=path.as_posix(),
                      role_mapping={"user": "messages.role.user", "assistant": "messages.role.assistant"})]))
    train_dl, _ = factory()
    assert len(train_dl) == 20
    batch = next(iter(train_dl))
    labels = batch["labels"][0]
    assert (labels == -100).any() and (labels != -100).any()  # the user turn is masked, the assistant turn is trained on
