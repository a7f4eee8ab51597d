# SPDX-License-Identifier: Apache-2.0
"""Preference (DPO) data: prompt / chosen / rejected tokenisation and the paired collator.

Behaviour parity: arctic_training/data/dpo_factory.py:36-308 — the prompt is tokenised as part of
``prompt + answer`` so that tokenizer merges at the boundary are handled (the prompt may lose its last
token to the answer), BOS is prepended and EOS appended when the tokenizer defines them, over-long
prompts are truncated (``keep_start`` / ``keep_end``) before answers are, labels mask the prompt, and a
batch is the chosen rows followed by the rejected rows.
"""

from __future__ import annotations

from typing import Any
from typing import Dict
from typing import List
from typing import Literal
from typing import Optional
from typing import Tuple

import torch

from ..config.data import DataConfig
from ..config.utils import HumanInt
from .factory import DataFactory
from .sft import IGNORE_INDEX
from .sft import pad

Tokens = Dict[str, List[int]]


class DPODataConfig(DataConfig):
    max_prompt_length: HumanInt = 4096
    """ Maximum prompt length. """

    dpo_prompt_truncation_mode: Literal["keep_start", "keep_end"] = "keep_start"
    """ Which end of an over-long prompt survives truncation. """


def _check_prompts_agree(prompt: Tokens, chosen: Tokens, rejected: Tokens) -> None:
    c, r = chosen["prompt_input_ids"], rejected["prompt_input_ids"]
    keep = min(len(c), len(r))
    for k in list(prompt):
        prompt[k] = prompt[k][:keep]
    differing = sum(a != b for a, b in zip(c, r))
    if differing > 1 or abs(len(c) - len(r)) > 1:
        raise ValueError("Chosen and rejected prompts may only differ in their last token (tokenizer merges).")


def add_bos_token_if_needed(bos_token_id: Optional[int], tokens: Tokens) -> Tokens:
    if bos_token_id is None:
        return tokens
    ids = tokens["prompt_input_ids"]
    if not ids or ids[0] != bos_token_id:
        ids.insert(0, bos_token_id)
        tokens["prompt_attention_mask"].insert(0, 1)
    return tokens


def add_eos_token_if_needed(eos_token_id: Optional[int], tokens: Tokens) -> Tokens:
    if eos_token_id is None:
        return tokens
    ids = tokens["input_ids"]
    if not ids or ids[-1] != eos_token_id:
        ids.append(eos_token_id)
        tokens["attention_mask"].append(1)
    elif len(ids) > 1 and ids[-2] == eos_token_id:
        tokens["input_ids"], tokens["attention_mask"] = ids[:-1], tokens["attention_mask"][:-1]
    return tokens


def _sequence(tokens: Tokens, prefix: str) -> Tokens:
    n_prompt = len(tokens["prompt_input_ids"])
    ids = tokens["prompt_input_ids"] + tokens["input_ids"]
    return {
        f"{prefix}_input_ids": ids,
        f"{prefix}_attention_mask": tokens["prompt_attention_mask"] + tokens["attention_mask"],
        f"{prefix}_labels": [IGNORE_INDEX] * n_prompt + ids[n_prompt:],
    }


class DataCollatorForPref:
    def __init__(self, tokenizer: Any) -> None:
        self.tokenizer = tokenizer

    def __call__(self, instances: List[Dict[str, Any]]) -> Dict[str, Any]:
        def both(key: str) -> List[torch.Tensor]:
            return [torch.as_tensor(ex[f"chosen_{key}"], dtype=torch.long) for ex in instances] + [
                torch.as_tensor(ex[f"rejected_{key}"], dtype=torch.long) for ex in instances
            ]

        pad_id = getattr(self.tokenizer, "pad_token_id", 0) or 0
        return {
            "input_ids": pad(both("input_ids"), padding_value=pad_id),
            "labels": pad(both("labels"), padding_value=IGNORE_INDEX),
            "attention_mask": pad(both("attention_mask"), padding_value=0),
            "prompt": [ex["prompt_input_ids"] for ex in instances],
            "prompt_text": [ex["prompt_text"] for ex in instances],
            "chosen_text": [ex["chosen_text"] for ex in instances],
            "rejected_text": [ex["rejected_text"] for ex in instances],
        }


class DPODataFactory(DataFactory):
    name = "dpo"
    config: DPODataConfig

    def convert_text(self, tokenizer: Any, conversations: List[Dict[str, str]]) -> str:
        return tokenizer.apply_chat_template(conversation=conversations, tokenize=False)

    def process(self, dataset):
        missing = [c for c in ("prompt", "chosen", "rejected") if c not in dataset.column_names]
        if missing:
            raise ValueError(f"DPODataFactory needs 'prompt', 'chosen' and 'rejected' columns; missing {missing}")
        dataset = dataset.select_columns(["prompt", "chosen", "rejected"])
        tok = self.tokenizer
        nproc = min(self.config.num_proc, max(1, len(dataset) // 64))
        return dataset.map(
            lambda ex: self.tokenize_messages(ex["prompt"], ex["chosen"], ex["rejected"], tok),
            num_proc=nproc if nproc > 1 else None, desc="Tokenizing preference pairs",
        )

    def process_prompt(self, tokenizer: Any, prompt_text: str) -> Tokens:
        enc = tokenizer(prompt_text, add_special_tokens=False)
        return {f"prompt_{k}": list(enc[k]) for k in ("input_ids", "attention_mask")}

    def process_answer(self, tokenizer: Any, prompt: str, answer: str) -> Tokens:
        full = tokenizer(prompt + answer, add_special_tokens=False)
        alone = list(tokenizer(prompt, add_special_tokens=False)["input_ids"])
        full_ids, full_mask = list(full["input_ids"]), list(full["attention_mask"])
        start = len(alone)
        if alone != full_ids[:start]:
            start -= 1  # the prompt's last token merged with the beginning of the answer
        return {
            "prompt_input_ids": full_ids[:start],
            "prompt_attention_mask": full_mask[:start],
            "input_ids": full_ids[len(alone):],
            "attention_mask": full_mask[len(alone):],
        }

    def _truncate_tokens(self, chosen: Tokens, rejected: Tokens, prompt: Tokens) -> Tuple[Tokens, Tokens, Tokens]:
        cfg = self.config
        longest = max(len(chosen["input_ids"]), len(rejected["input_ids"]))
        for t in (chosen, rejected, prompt):
            if len(t["prompt_input_ids"]) + longest > cfg.max_length:
                for k in ("prompt_input_ids", "prompt_attention_mask"):
                    t[k] = t[k][: cfg.max_prompt_length] if cfg.dpo_prompt_truncation_mode == "keep_start" else t[k][-cfg.max_prompt_length:]
        for t in (chosen, rejected):
            if len(t["prompt_input_ids"]) + longest > cfg.max_length:
                room = max(1, cfg.max_length - len(t["prompt_input_ids"]))
                for k in ("input_ids", "attention_mask"):
                    t[k] = t[k][:room]
        return chosen, rejected, prompt

    def tokenize_messages(self, prompt, chosen, rejected, tokenizer: Any) -> Dict[str, Any]:
        prompt_text = self.convert_text(tokenizer, prompt)
        chosen_text = self.convert_text(tokenizer, prompt + chosen)[len(prompt_text):]
        rejected_text = self.convert_text(tokenizer, prompt + rejected)[len(prompt_text):]
        p = self.process_prompt(tokenizer, prompt_text)
        c = self.process_answer(tokenizer, prompt_text, chosen_text)
        r = self.process_answer(tokenizer, prompt_text, rejected_text)
        _check_prompts_agree(p, c, r)
        bos, eos = getattr(tokenizer, "bos_token_id", None), getattr(tokenizer, "eos_token_id", None)
        p, c, r = (add_bos_token_if_needed(bos, t) for t in (p, c, r))
        c, r = add_eos_token_if_needed(eos, c), add_eos_token_if_needed(eos, r)
        c, r, p = self._truncate_tokens(c, r, p)
        row: Dict[str, Any] = {}
        row.update(p)
        row.update(_sequence(c, "chosen"))
        row.update(_sequence(r, "rejected"))
        row.update(prompt_text=prompt_text, chosen_text=chosen_text, rejected_text=rejected_text)
        return row

    def collate_fn(self):
        return DataCollatorForPref(tokenizer=self.tokenizer)
