# SPDX-License-Identifier: Apache-2.0
"""Install optional dependency groups declared in ``pyproject.toml`` without installing the package itself.

    python ci/install_extras.py dev embed [--dry-run] [--pip-args="--no-index --find-links /wheels"]

A group may refer to another group of this project (``arctictraining_b200[dev]``); references are followed, cycles
are tolerated.  Counterpart of scripts/install_deps.py in the reference.
"""

import argparse
import shlex
import subprocess
import sys
import tomllib
from pathlib import Path
from typing import Dict
from typing import List

ROOT = Path(__file__).resolve().parent.parent


def load_groups(pyproject: Path = ROOT / "pyproject.toml") -> Dict[str, List[str]]:
    with open(pyproject, "rb") as f:
        project = tomllib.load(f).get("project", {})
    groups = dict(project.get("optional-dependencies", {}))
    groups["__name__"] = [project.get("name", "")]
    return groups


def resolve(wanted: List[str], groups: Dict[str, List[str]]) -> List[str]:
    own = groups.get("__name__", [""])[0].replace("-", "_")
    seen, out, todo = set(), set(), list(wanted)
    while todo:
        g = todo.pop()
        if g in seen:
            continue
        seen.add(g)
        if g not in groups or g == "__name__":
            known = ", ".join(k for k in groups if k != "__name__")
            raise SystemExit(f"unknown dependency group {g!r}; known groups: {known}")
        for dep in groups[g]:
            head = dep.split("[")[0].strip().replace("-", "_")
            if "[" in dep and head == own:
                todo.extend(x.strip() for x in dep.split("[", 1)[1].rstrip("]").split(","))
            else:
                out.add(dep)
    return sorted(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("groups", nargs="+")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--pip-args", default="")
    args = ap.parse_args(argv)
    deps = resolve(args.groups, load_groups())
    if not deps:
        print("nothing to install")
        return 0
    cmd = [sys.executable, "-m", "pip", "install", *shlex.split(args.pip_args), *deps]
    print(" ".join(cmd))
    return 0 if args.dry_run else subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
