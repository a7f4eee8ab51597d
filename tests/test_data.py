# SPDX-License-Identifier: Apache-2.0
"""Data layer: SFT tokenisation and masking, packing, padding, causal slicing, DPO pairs, caches, sources."""

from types import SimpleNamespace

import pytest
import torch

from arctictraining_b200.data.causal import slice_and_pack_causal_batch
from arctictraining_b200.data.hf_sources import HFDataSourceConfigInstruct
from arctictraining_b200.data.hf_sources import extract_messages
from arctictraining_b200.data.sft import DataCollatorForCausalLM
from arctictraining_b200.data.sft import SFTDataFactory
from arctictraining_b200.data.sft import pack_sft_batch
from arctictraining_b200.data.sft import pad
from arctictraining_b200.tokenizer.fake import FakeTokenizer

MESSAGES = [
    {"role": "user", "content": "what is two plus two"},
    {"role": "assistant", "content": "it is four"},
    {"role": "user", "content": "and three plus three"},
    {"role": "assistant", "content": "six of course"},
]


def test_assistant_only_labels_include_end_of_turn_token():
    tok = FakeTokenizer(1024)
    enc = SFTDataFactory.tokenize_messages(MESSAGES, tok, mask_inputs=True)
    ids, labels = enc["input_ids"], enc["labels"]
    assert len(ids) == len(labels)
    trained = [i for i, lab in enumerate(labels) if lab != -100]
    assert all(labels[i] == ids[i] for i in trained)
    n_assistant_words = len("it is four".split()) + len("six of course".split())
    assert len(trained) == n_assistant_words + 2  # plus one end-of-turn token after each assistant message
    assert tok.eos_token_id in [ids[i] for i in trained]
    unmasked = SFTDataFactory.tokenize_messages(MESSAGES, tok, mask_inputs=False)
    assert unmasked["labels"] == unmasked["input_ids"]


def test_ignore_empty_think_prefix():
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "<think>\n</think>\nhello there"}]
    tok = FakeTokenizer(1024)
    a = SFTDataFactory.tokenize_messages(msgs, tok, ignore_empty_think=False)
    b = SFTDataFactory.tokenize_messages(msgs, tok, ignore_empty_think=True)
    assert sum(x != -100 for x in b["labels"]) < sum(x != -100 for x in a["labels"])


def test_pad_to_multiple_and_to_max():
    ts = [torch.tensor([1, 2, 3]), torch.tensor([4, 5])]
    out = pad(ts, padding_value=0, divisible_by=4)
    assert out.tolist() == [[1, 2, 3, 0], [4, 5, 0, 0]]
    assert pad(ts, padding_value=9, max_seq=6).shape == (2, 6)
    pos = pad([torch.arange(3), torch.arange(2)], is_position_id=True, divisible_by=4)
    assert pos.tolist() == [[0, 1, 2, 3], [0, 1, 2, 3]]
    assert pad(ts, padding_value=0, padding_side="left", divisible_by=4).tolist() == [[0, 1, 2, 3], [0, 0, 4, 5]]


def test_packing_restarts_positions_and_respects_max_length():
    batch = {"input_ids": [[1] * 5, [2] * 4, [3] * 6, [4] * 2], "labels": [[1] * 5, [2] * 4, [3] * 6, [4] * 2],
             "attention_mask": [[1] * 5, [1] * 4, [1] * 6, [1] * 2]}
    out = pack_sft_batch(batch, max_length=10, always_max_length=False, drop_last=False, fuse_positions_prob=0.0, seed=0)
    assert out["packed_sample_seqlens"] == [[5, 4], [6, 2]]
    assert out["position_ids"][0] == list(range(5)) + list(range(4))
    assert all(len(x) <= 10 for x in out["input_ids"])
    dropped = pack_sft_batch(batch, 10, False, True, 0.0, 0)
    assert dropped["packed_sample_seqlens"] == [[5, 4]]
    fused = pack_sft_batch(batch, 10, False, False, 1.0, 0)
    assert fused["position_ids"][0] == list(range(9))


def test_collator_pads_labels_with_ignore_index():
    cfg = SimpleNamespace(pad_to="div_length", div_length=8, max_length=32)
    col = DataCollatorForCausalLM(FakeTokenizer(64), cfg)
    out = col([{"input_ids": [5, 6, 7], "labels": [-100, 6, 7]}, {"input_ids": [8] * 9, "labels": [8] * 9}])
    assert out["input_ids"].shape == (2, 16) and out["labels"][0, 3:].eq(-100).all()
    assert out["packed_sample_seqlens"] == [[3], [9]]
    assert out["position_ids"][0].tolist() == list(range(16))


def test_causal_slicing_carries_leftovers_across_calls():
    overflow = []
    a = slice_and_pack_causal_batch({"input_ids": [list(range(25)), list(range(100, 107))]}, 10, overflow)
    assert [len(x) for x in a["input_ids"]] == [10, 10, 10]
    assert a["packed_sample_seqlens"][2] == [5, 5]  # tail of doc 1 + head of doc 2
    assert a["position_ids"][2] == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4]
    assert overflow == [[105, 106]]
    b = slice_and_pack_causal_batch({"input_ids": [list(range(200, 208))]}, 10, overflow)
    assert b["input_ids"] == [[105, 106] + list(range(200, 208))] and overflow == []


def test_role_mapping_paths():
    ex = {"system_prompt": "be brief", "question": "q1", "response": "a1"}
    msgs = extract_messages(ex, {"system": "system_prompt", "user": "question", "assistant": "response"}, None)
    assert [m["role"] for m in msgs] == ["system", "user", "assistant"]
    conv = {"conversations": [{"from": "human", "value": "u1"}, {"from": "gpt", "value": "g1"},
                              {"from": "human", "value": "u2"}, {"from": "gpt", "value": "g2"}]}
    msgs = extract_messages(conv, {"user": "conversations.from.human", "assistant": "conversations.from.gpt"}, None)
    assert [m["content"] for m in msgs] == ["u1", "g1", "u2", "g2"]
    with pytest.raises(ValueError):
        HFDataSourceConfigInstruct(type="huggingface_instruct", name_or_path="x", role_mapping={"user": "a.b"})
    known = HFDataSourceConfigInstruct(type="huggingface_instruct", name_or_path="Open-Orca/SlimOrca:train[:10]")
    assert known.split == "train[:10]" and known.role_mapping["user"] == "conversations.from.human"


def test_sft_pipeline_through_factory_with_messages_and_cache(tiny_recipe, tmp_path):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    data = {"sources": [{"type": "synthetic_messages", "num_samples": 40, "turns": 2, "words_per_message": 8}],
            "cache_dir": str(tmp_path / "cache"), "max_length": 96, "pack_samples": True, "dl_num_workers": 0}
    cfg = get_config(tiny_recipe(data=data, micro_batch_size=1))
    tr = get_registered_trainer(cfg.type)(cfg, mode="process-data")
    batch = next(iter(tr.train_dataloader))
    assert batch["input_ids"].shape[1] % 256 == 0 or batch["input_ids"].shape[1] <= 256
    assert sum(batch["packed_sample_seqlens"][0]) <= 96
    assert (batch["labels"] != -100).any()
    n_cache_entries = len(list((tmp_path / "cache").iterdir()))
    tr2 = get_registered_trainer(cfg.type)(cfg, mode="process-data")  # second build hits the cache
    assert len(list((tmp_path / "cache").iterdir())) == n_cache_entries
    b2 = next(iter(tr2.train_dataloader))
    assert torch.equal(b2["input_ids"], batch["input_ids"])


def test_min_iterations_replicates_data(tiny_recipe, tmp_path):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    data = {"sources": [{"type": "synthetic", "num_samples": 6, "min_length": 16, "max_length": 16}],
            "cache_dir": str(tmp_path / "c"), "max_length": 16, "dl_num_workers": 0}
    cfg = get_config(tiny_recipe(data=data, min_iterations=20, micro_batch_size=1))
    tr = get_registered_trainer(cfg.type)(cfg, mode="process-data")
    assert len(tr.train_dataloader) == 20


def test_dpo_tokenisation_masks_prompt_and_pairs_rows(tiny_recipe, tmp_path):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    r = tiny_recipe(type="dpo", micro_batch_size=2, ref_model={"name_or_path": "tiny-llama", "dtype": "fp32"},
                    data={"sources": [{"type": "synthetic_dpo", "num_samples": 16, "words_per_message": 6}],
                          "cache_dir": str(tmp_path / "c"), "max_length": 64, "dl_num_workers": 0})
    cfg = get_config(r)
    assert cfg.deepspeed["train_micro_batch_size_per_gpu"] == 4
    tr = get_registered_trainer(cfg.type)(cfg, mode="process-data")
    b = next(iter(tr.train_dataloader))
    assert b["input_ids"].shape[0] == 4  # chosen rows then rejected rows
    n_prompt = len(b["prompt"][0])
    assert (b["labels"][0, :n_prompt] == -100).all() and (b["labels"][0, n_prompt] != -100)
    assert torch.equal(b["input_ids"][0, :n_prompt], b["input_ids"][2, :n_prompt])
