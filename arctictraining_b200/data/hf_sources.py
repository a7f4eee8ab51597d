# SPDX-License-Identifier: Apache-2.0
"""Data sources backed by the ``datasets`` library: generic, instruction (SFT), causal text, and two
named datasets.  Parity: arctic_training/data/hf_source.py:33-170, hf_instruct_source.py:32-224,
hf_causal_source.py:21-48."""

from __future__ import annotations

from pathlib import Path
from typing import Any
from typing import Dict
from typing import List
from typing import Optional

from pydantic import Field
from pydantic import field_validator
from pydantic import model_validator
from typing_extensions import Self

from ..config.data import DataSourceConfig
from .source import DataSource

# datasets whose split names or loader options are known
KNOWN_HF_DATASETS: Dict[str, Dict[str, Any]] = {
    "HuggingFaceH4/ultrachat_200k": {"split_mapping": {"train": "train_sft", "eval": "test_sft"}},
    "HuggingFaceH4/ultrafeedback_binarized": {"split_mapping": {"train": "train_prefs", "eval": "test_prefs"}},
    "nvidia/AceMath-Instruct-Training-Data": {
        "split_mapping": {"train": "general_sft_stage2"}, "kwargs": {"verification_mode": "no_checks"},
    },
}

_CONV = {"user": "messages.role.user", "assistant": "messages.role.assistant"}
KNOWN_HF_INSTRUCT_DATASETS: Dict[str, Dict[str, Any]] = {
    "nvidia/AceMath-Instruct-Training-Data": {"role_mapping": dict(_CONV)},
    "HuggingFaceH4/ultrachat_200k": {"role_mapping": dict(_CONV)},
    "THUDM/LongAlign-10k": {"role_mapping": dict(_CONV)},
    "Open-Orca/OpenOrca": {"role_mapping": {"system": "system_prompt", "user": "question", "assistant": "response"}},
    "Yukang/LongAlpaca-12k": {"role_mapping": {"user": "instruction", "assistant": "output"}},
    "Open-Orca/SlimOrca": {"role_mapping": {
        "system": "conversations.from.system", "user": "conversations.from.human", "assistant": "conversations.from.gpt"}},
    "meta-math/MetaMathQA": {"role_mapping": {"user": "query", "assistant": "response"}},
    "ise-uiuc/Magicoder-OSS-Instruct-75K": {"role_mapping": {"user": "problem", "assistant": "solution"}},
    "lmsys/lmsys-chat-1m": {"role_mapping": {"user": "conversation.role.user", "assistant": "conversation.role.assistant"}},
}


class HFDataSourceConfig(DataSourceConfig):
    name_or_path: str
    """ Dataset name or local path; ``name:split`` and ``name:split[10:20]`` are accepted. """

    kwargs: Dict[str, Any] = Field(default_factory=dict)
    """ Extra keyword arguments for ``datasets.load_dataset``. """

    split_mapping: Dict[str, str] = Field(default_factory=dict)
    """ Standard split name (train/eval) -> split name of this dataset. """

    @model_validator(mode="after")
    def _fill_from_name(self) -> Self:
        if ":" in self.name_or_path:
            name, split = self.name_or_path.split(":", 1)
            object.__setattr__(self, "name_or_path", name)
            object.__setattr__(self, "split", split)
        known = KNOWN_HF_DATASETS.get(self.name_or_path, {})
        if not self.split_mapping and "split_mapping" in known:
            object.__setattr__(self, "split_mapping", dict(known["split_mapping"]))
        for k, v in known.get("kwargs", {}).items():
            self.kwargs.setdefault(k, v)
        return self


class HFDataSource(DataSource):
    name = "huggingface"
    config: HFDataSourceConfig

    def pre_load_callback(self, split: str) -> str:
        mapping = self.config.split_mapping
        if not mapping:
            return split
        base, bracket, rest = split.partition("[")
        if base in set(mapping.values()) or base not in mapping:
            return split
        return mapping[base] + bracket + rest

    def load(self, config: HFDataSourceConfig, split: str):
        from datasets import DatasetDict
        from datasets import load_dataset
        from datasets import load_from_disk

        if Path(config.name_or_path).exists():
            ds = load_from_disk(config.name_or_path, **config.kwargs)
            if isinstance(ds, DatasetDict):
                ds = ds[split]
            return ds
        return load_dataset(config.name_or_path, split=split, **config.kwargs)


class HFDataSourceConfigInstruct(HFDataSourceConfig):
    role_mapping: Dict[str, str] = Field(default_factory=lambda: {"user": "user", "assistant": "assistant"})
    """ Role -> where its text lives: a column name (``question``) or ``array.field.value``
    (``conversations.from.human``: items of ``conversations`` whose ``from`` equals ``human``). """

    content_key: Optional[str] = None
    """ Key of the text inside conversation items (auto-detected among content/text/message/value). """

    @field_validator("role_mapping", mode="before")
    @classmethod
    def _paths_have_three_parts(cls, v: Dict[str, str]) -> Dict[str, str]:
        for role, spec in v.items():
            if "." in spec and len(spec.split(".")) != 3:
                raise ValueError(f"Invalid conversation path for role '{role}': expected 'array.field.value'")
        return v

    @model_validator(mode="after")
    def _fill_known_role_mapping(self) -> Self:
        known = KNOWN_HF_INSTRUCT_DATASETS.get(str(self.name_or_path).split(":")[0])
        if known:
            if "role_mapping" not in self.model_fields_set and "role_mapping" in known:
                object.__setattr__(self, "role_mapping", dict(known["role_mapping"]))
            if "content_key" not in self.model_fields_set and "content_key" in known:
                object.__setattr__(self, "content_key", known["content_key"])
        return self


def _item_text(item: Dict[str, Any], key: Optional[str]) -> Optional[str]:
    if key:
        v = item.get(key)
        return None if v is None else str(v)
    for cand in ("content", "text", "message", "value"):
        if item.get(cand) is not None:
            return str(item[cand])
    return None


def extract_messages(example: Dict[str, Any], role_mapping: Dict[str, str], content_key: Optional[str]) -> List[Dict[str, str]]:
    """Turn one raw record into a list of chat messages, interleaving roles turn by turn."""
    per_role: Dict[str, List[Dict[str, str]]] = {}
    for role, spec in role_mapping.items():
        texts: List[str] = []
        if "." not in spec:
            if example.get(spec) is not None:
                texts = [str(example[spec])]
        else:
            arr, field, value = spec.split(".")
            conv = example.get(arr)
            if isinstance(conv, list):
                for item in conv:
                    if isinstance(item, dict) and item.get(field) == value:
                        t = _item_text(item, content_key)
                        if t is not None:
                            texts.append(t)
        msgs = [{"role": role, "content": t} for t in texts if t]
        if msgs:
            per_role[role] = msgs
    return [m for turn in zip(*per_role.values()) for m in turn]


class HFDataSourceInstruct(HFDataSource):
    name = "huggingface_instruct"
    config: HFDataSourceConfigInstruct

    def post_load_callback(self, dataset):
        mapping, key = self.config.role_mapping, self.config.content_key

        def to_messages(example: Dict[str, Any]) -> Dict[str, Any]:
            msgs = extract_messages(example, mapping, key)
            if not msgs:
                raise ValueError(f"Could not extract messages using role_mapping {mapping}; columns: {sorted(example)}")
            return {"messages": msgs}

        if self.config.name_or_path == "nvidia/AceMath-Instruct-Training-Data":
            dataset = dataset.map(lambda ex: {"messages": ex["messages"] + [{"role": "assistant", "content": ex["answer"]}]})
        nproc = min(self.data_factory.config.num_proc, max(1, len(dataset) // 64))
        return dataset.map(to_messages, num_proc=nproc if nproc > 1 else None, desc=f"Loading {self.config.name_or_path}")


class HFDataSourceConfigCausal(HFDataSourceConfig):
    column: str = "text"
    """ Column that holds the raw text. """


class HFDataSourceCausal(HFDataSource):
    name = "huggingface_causal"
    config: HFDataSourceConfigCausal

    def post_load_callback(self, dataset):
        col = self.config.column
        if col != "text":
            dataset = dataset.rename_column(col, "text")
        return dataset.select_columns(["text"])


class ProjectGutenbergSFT(HFDataSource):
    """Each book becomes a single user message (prompt-only distillation data, e.g. for SwiftKV)."""

    name = "ProjectGutenbergSFT"

    def post_load_callback(self, dataset):
        return dataset.map(lambda ex: {"messages": [{"role": "user", "content": ex["text"]}]}, desc="Project Gutenberg")


class UltraFeedbackBinarized(HFDataSource):
    name = "HuggingFaceH4/ultrafeedback_binarized"

    def post_load_callback(self, dataset):
        return dataset.select_columns(["chosen", "rejected"]).map(self.split_prompt_content, desc="ultrafeedback")

    @staticmethod
    def split_prompt_content(example: Dict[str, List]) -> Dict[str, List]:
        """The shared leading messages of chosen/rejected form the prompt."""
        n = min(len(example["chosen"]), len(example["rejected"]))
        idx = 0
        while idx < n and example["chosen"][idx]["content"] == example["rejected"][idx]["content"]:
            idx += 1
        idx = min(idx, n - 1) if n else 0
        return {"prompt": example["chosen"][:idx], "chosen": example["chosen"][idx:], "rejected": example["rejected"][idx:]}
