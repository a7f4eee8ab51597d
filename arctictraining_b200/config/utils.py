# SPDX-License-Identifier: Apache-2.0
"""Helpers shared by the config classes: rank look-ups, human-readable numbers, strict YAML loading.

Behaviour parity: arctic_training/config/utils.py:25-92.
"""

from __future__ import annotations

import os
import re
from typing import Annotated
from typing import Union

import yaml
from pydantic.functional_validators import BeforeValidator


def get_local_rank() -> int:
    return int(os.getenv("LOCAL_RANK", 0))


def get_global_rank() -> int:
    return int(os.getenv("RANK", 0))


def get_world_size() -> int:
    return int(os.getenv("WORLD_SIZE", 1))


class UniqueKeyLoader(yaml.SafeLoader):
    """SafeLoader that refuses a mapping in which the same key appears twice."""

    def construct_mapping(self, node, deep=False):
        seen = set()
        for key_node, _ in node.value:
            key = self.construct_object(key_node, deep=deep)
            if key in seen:
                raise ValueError(f"Duplicate '{key}' key found in YAML on line {key_node.start_mark.line + 1}.")
            seen.add(key)
        return super().construct_mapping(node, deep)


_NUM = r"(-?\d+\.?\d*)"
_DEC = {"k": 1e3, "m": 1e6, "b": 1e9, "t": 1e12}
_BIN = {"ki": 2**10, "mi": 2**20, "gi": 2**30, "ti": 2**40}
_RE_POW = re.compile(rf"^{_NUM}\^{_NUM}$")
_RE_SCI = re.compile(rf"^{_NUM}e{_NUM}$")
_RE_SUF = re.compile(rf"^{_NUM}(ki|mi|gi|ti|k|m|b|t)$")


def parse_human_val(value: Union[str, int, float]) -> Union[int, float]:
    """Turn ``"1.5K"``, ``"1Ki"``, ``"10^6"``, ``"1e6"``, ``"2.5%"`` or ``"1_000"`` into a number."""
    if isinstance(value, (int, float)):
        return value
    if not isinstance(value, str):
        raise ValueError("only strings and numbers can be parsed")
    text = value.replace("_", "").strip().lower()
    if text.endswith("%"):
        return float(text[:-1]) / 100.0
    m = _RE_POW.match(text)
    if m:
        base, exp = float(m.group(1)), float(m.group(2))
        return (-1.0 if base < 0 else 1.0) * abs(base) ** exp
    m = _RE_SCI.match(text)
    if m:
        return float(m.group(1)) * 10 ** float(m.group(2))
    m = _RE_SUF.match(text)
    if m:
        mult = _BIN.get(m.group(2)) or _DEC[m.group(2)]
        return float(m.group(1)) * mult
    return float(text)


HumanInt = Annotated[int, BeforeValidator(parse_human_val)]
HumanFloat = Annotated[float, BeforeValidator(parse_human_val)]
