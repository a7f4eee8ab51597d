# SPDX-License-Identifier: Apache-2.0
"""Turn a benchmark file (BIRD, Spider and variants, synthetic) into model input / target pairs.

    python projects/arctic_text2sql_r1/process_dataset.py -i dev.json -o dev_bird.json -d dev_databases \\
        -t dev_tables.json -s bird -m dev -v 2 -c db_contents_index
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from text2sql.evaluate import load_json  # noqa: E402
from text2sql.prompting import SOURCES  # noqa: E402
from text2sql.prompting import build_examples  # noqa: E402
from text2sql.prompting import write_examples  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--input_data_file", required=True)
    ap.add_argument("-o", "--output_data_file", required=True)
    ap.add_argument("-d", "--db_path", required=True)
    ap.add_argument("-t", "--tables", required=True)
    ap.add_argument("-s", "--source", required=True, choices=sorted(SOURCES))
    ap.add_argument("-m", "--mode", default="dev", choices=["train", "dev", "test"])
    ap.add_argument("-v", "--value_limit_num", type=int, default=2)
    ap.add_argument("-c", "--db_content_index_path", default=None)
    args = ap.parse_args()
    examples = build_examples(load_json(args.input_data_file), load_json(args.tables), args.db_path, args.source, args.mode,
                              args.value_limit_num, args.db_content_index_path)
    write_examples(examples, args.output_data_file)
    print(f"wrote {len(examples)} examples to {args.output_data_file}")
