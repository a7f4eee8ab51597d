# SPDX-License-Identifier: Apache-2.0
"""JSON-lines helpers and human-readable number formatting.  Parity: arctic_training/utils.py:22-90."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any
from typing import List


def read_json_file(path) -> List[Any]:
    """Read a ``.json`` file (one document) or a ``.jsonl`` file (one document per line)."""
    path = Path(path)
    text = path.read_text()
    if path.suffix == ".jsonl":
        return [json.loads(line) for line in text.splitlines() if line.strip()]
    return json.loads(text)


def write_json_file(path, data, append: bool = False) -> None:
    path = Path(path)
    if path.suffix == ".jsonl":
        rows = data if isinstance(data, list) else [data]
        with open(path, "a" if append else "w") as fh:
            for row in rows:
                fh.write(json.dumps(row) + "\n")
    else:
        with open(path, "w") as fh:
            json.dump(data, fh, indent=2)


def append_json_file(path, data) -> None:
    write_json_file(path, data, append=True)


def human_format_base2_number(num: float, suffix: str = "") -> str:
    for unit in ("", "Ki", "Mi", "Gi", "Ti", "Pi"):
        if abs(num) < 1024.0:
            return f"{num:3.2f}{unit}{suffix}"
        num /= 1024.0
    return f"{num:.2f}Ei{suffix}"


def human_format_base10_number(num: float, suffix: str = "") -> str:
    for unit in ("", "K", "M", "B", "T", "Qa"):
        if abs(num) < 1000.0:
            return f"{num:3.2f}{unit}{suffix}"
        num /= 1000.0
    return f"{num:.2f}Qi{suffix}"


def human_format_secs(secs: float) -> str:
    secs = float(secs)
    if secs < 1:
        return f"{secs * 1e3:.1f}ms"
    if secs < 60:
        return f"{secs:.3f}s"
    m, s = divmod(int(round(secs)), 60)
    h, m = divmod(m, 60)
    return f"{h:02d}:{m:02d}:{s:02d}"
