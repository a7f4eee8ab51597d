# SPDX-License-Identifier: Apache-2.0
"""Rewrite user trainer / factory code written against the old class-attribute style to annotations.

    python ci/upgrade_user_code.py my_trainer.py [more.py ...] [--check]

``config_type = MyConfig`` becomes ``config: MyConfig`` and ``data_factory_type = [A, B]`` becomes
``data_factory: Union[A, B]`` (adding the ``typing`` import when needed); likewise for the model, checkpoint-engine,
optimizer, scheduler and tokenizer attributes.  ``--check`` only reports files that would change (exit 1).
Counterpart of scripts/upgrade_user_code.py in the reference.
"""

import re
import sys
from pathlib import Path
from typing import Tuple

ATTRS = ("config", "data_factory", "model_factory", "checkpoint_engine", "optimizer_factory", "scheduler_factory",
         "tokenizer_factory")
_NAME = r"[A-Za-z_][A-Za-z0-9_.]*"
_SINGLE = re.compile(rf"^(?P<ind>[ \t]*)(?P<attr>{'|'.join(ATTRS)})_type[ \t]*=[ \t]*(?P<cls>{_NAME})[ \t]*(?P<tail>#.*)?$", re.M)
_LIST = re.compile(rf"^(?P<ind>[ \t]*)(?P<attr>{'|'.join(ATTRS)})_type[ \t]*=[ \t]*\[(?P<items>[^\]]*)\][ \t]*(?P<tail>#.*)?$", re.M)


def upgrade_source(text: str) -> Tuple[str, int]:
    """Returns the rewritten text and the number of rewritten attributes."""
    n_union = 0

    def as_union(m: "re.Match") -> str:
        nonlocal n_union
        items = [x.strip() for x in m["items"].replace("\n", " ").split(",") if x.strip()]
        tail = f"  {m['tail']}" if m["tail"] else ""
        if len(items) == 1:
            return f"{m['ind']}{m['attr']}: {items[0]}{tail}"
        n_union += 1
        return f"{m['ind']}{m['attr']}: Union[{', '.join(items)}]{tail}"

    text, n_list = _LIST.subn(as_union, text)
    text, n_single = _SINGLE.subn(lambda m: f"{m['ind']}{m['attr']}: {m['cls']}" + (f"  {m['tail']}" if m["tail"] else ""), text)
    if n_union and not re.search(r"^\s*from typing import .*\bUnion\b|^\s*import typing\b", text, re.M):
        lines = text.split("\n")
        at = 0
        if lines and lines[0].startswith(('"""', "'''")):  # keep a module docstring first
            quote = lines[0][:3]
            at = next((i for i, ln in enumerate(lines) if ln.rstrip().endswith(quote) and (i > 0 or len(ln.strip()) > 3)), 0) + 1
        while at < len(lines) and (lines[at].startswith("#") or lines[at].startswith("from __future__") or not lines[at].strip()) and at < 30:
            at += 1
        lines.insert(at, "from typing import Union")
        text = "\n".join(lines)
    return text, n_list + n_single


def main(argv) -> int:
    check = "--check" in argv
    paths = [Path(a) for a in argv if not a.startswith("--")]
    if not paths:
        print(__doc__)
        return 2
    changed = 0
    for p in paths:
        if not p.exists():
            print(f"{p}: not found")
            return 2
        new, n = upgrade_source(p.read_text())
        if n:
            changed += 1
            print(f"{p}: {n} attribute(s) {'would be ' if check else ''}rewritten")
            if not check:
                p.write_text(new)
    return 1 if (check and changed) else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
