# SPDX-License-Identifier: Apache-2.0
"""Every tracked source file must carry the project's licence identifier in its first lines.

    python ci/check_license.py            # exit 1 and list the files that lack it
    python ci/check_license.py --fix      # insert it (after a shebang / encoding line if present)
    python ci/check_license.py FILE ...   # check only these (the form a pre-commit hook uses)

Counterpart of scripts/check_license.py in the reference, which compares against its full header text; one SPDX line
is what licence scanners read.
"""

import subprocess
import sys
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parent.parent
SPDX = "SPDX-License-Identifier: Apache-2.0"
COMMENT = {".py": "# ", ".sh": "# ", ".yaml": "# ", ".yml": "# ", ".cu": "// ", ".cuh": "// ", ".cpp": "// ", ".h": "// "}
CHECKED = {".py", ".sh", ".cu", ".cuh", ".cpp", ".h"}
HEAD_LINES = 5


def tracked_sources() -> List[Path]:
    out = subprocess.run(["git", "ls-files"], cwd=ROOT, capture_output=True, text=True, check=True).stdout.split("\n")
    return [ROOT / p for p in out if p and Path(p).suffix in CHECKED]


def has_identifier(path: Path) -> bool:
    with open(path, "r", errors="ignore") as f:
        return any(SPDX in f.readline() for _ in range(HEAD_LINES))


def insert_identifier(path: Path) -> None:
    lines = path.read_text().split("\n")
    at = 0
    while at < len(lines) and (lines[at].startswith("#!") or "coding" in lines[at][:20]):
        at += 1
    lines.insert(at, COMMENT[path.suffix] + SPDX)
    path.write_text("\n".join(lines))


def main(argv: List[str]) -> int:
    fix = "--fix" in argv
    named = [Path(a).resolve() for a in argv if not a.startswith("--")]
    files = [p for p in (named or tracked_sources()) if p.suffix in CHECKED and p.exists() and p.stat().st_size > 0]
    missing = [p for p in files if not has_identifier(p)]
    for p in missing:
        if fix:
            insert_identifier(p)
        print(f"{'added to' if fix else 'missing in'} {p.relative_to(ROOT) if p.is_relative_to(ROOT) else p}")
    return 0 if fix or not missing else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
