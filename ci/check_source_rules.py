# SPDX-License-Identifier: Apache-2.0
"""Repository hygiene checks run by CI: every Python / CUDA source compiles or at least parses, no source names one of
the driver API calls that are closed on the target hosts, no TMA / bulk load with cluster multicast, and recipes parse
as YAML with unique keys.  Exits non-zero with one line per violation."""

import ast
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BATCH_COPY = re.compile(r"cu(da)?Memcpy(3D)?Batch" + "Async")
MULTICAST_LOAD = re.compile(r"cp\.async\.bulk[\w.:]*\.multi" + "cast::" + "cluster")  # pattern split so that this file does not match itself


def main() -> int:
    problems = []
    for path in ROOT.rglob("*"):
        rel = path.relative_to(ROOT)
        if rel.parts[0].startswith(("_", "gpu")) or any(part in {".git", "baseline", "build", "__pycache__"} for part in rel.parts):
            continue
        if path.suffix == ".py":
            try:
                ast.parse(path.read_text())
            except SyntaxError as e:
                problems.append(f"{rel}: {e}")
        if path.suffix in {".py", ".cu", ".cuh", ".cpp", ".h"}:
            text = path.read_text(errors="ignore")
            if BATCH_COPY.search(text):
                problems.append(f"{rel}: names a batched memcpy driver call")
            if MULTICAST_LOAD.search(text):
                problems.append(f"{rel}: bulk / TMA load with cluster multicast")
        if path.suffix in {".yml", ".yaml"} and ".github" not in rel.parts:
            import yaml

            sys.path.insert(0, str(ROOT))
            from arctictraining_b200.config.utils import UniqueKeyLoader

            try:
                yaml.load(path.read_text(), Loader=UniqueKeyLoader)
            except Exception as e:  # noqa: BLE001
                problems.append(f"{rel}: {e}")
    print("\n".join(problems) if problems else "source rules: ok")
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
