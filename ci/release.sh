#!/usr/bin/env bash
# SPDX-License-Identifier: Apache-2.0
# Build the wheel (CUDA extension compiled for sm_100a in-tree first) and upload it to the package index.
#   ci/release.sh            build + upload (needs ~/.pypirc)
#   ci/release.sh --no-upload   build only
set -euo pipefail
cd "$(dirname "$0")/.."

python ci/check_source_rules.py
python ci/check_license.py
python -c "import __graft_entry__ as g; g.build()"
python -m pip wheel --no-deps --no-build-isolation -w dist .

if [[ "${1:-}" == "--no-upload" ]]; then
  ls -l dist
  exit 0
fi
if [[ ! -f "$HOME/.pypirc" ]]; then
  echo "create ~/.pypirc to upload" >&2
  exit 1
fi
python -m twine upload dist/*
