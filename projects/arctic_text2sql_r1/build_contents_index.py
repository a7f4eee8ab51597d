# SPDX-License-Identifier: Apache-2.0
"""Build the value index (BM25 over text cells) of every database under ``--db-root``.

    python projects/arctic_text2sql_r1/build_contents_index.py --db-root dev_databases --index-root db_contents_index
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from text2sql.value_index import build_indexes  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--db-root", required=True)
    ap.add_argument("--index-root", required=True)
    args = ap.parse_args()
    done = build_indexes(args.db_root, args.index_root)
    print(f"indexed {len(done)} databases into {args.index_root}")
