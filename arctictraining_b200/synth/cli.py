# SPDX-License-Identifier: Apache-2.0
"""``arctic_synth`` command line: inspect, download or cancel batch tasks kept in a work directory.
Parity: arctic_training/synth/cli.py:27-133."""

from __future__ import annotations

import argparse
import json
import sys
from typing import List
from typing import Optional


def main(argv: Optional[List[str]] = None) -> int:
    p = argparse.ArgumentParser(prog="arctic_synth")
    p.add_argument("action", choices=["status", "download", "cancel", "extract"])
    p.add_argument("-w", "--work_dir", required=True)
    p.add_argument("-t", "--task_name", required=True)
    p.add_argument("-c", "--credential_path", default=None)
    p.add_argument("--provider", choices=["openai", "azure"], default="openai")
    args = p.parse_args(argv)
    from .openai_callers import AzureOpenAISynth
    from .openai_callers import OpenAIBatchProcessor
    from .openai_callers import OpenAISynth

    make = AzureOpenAISynth if args.provider == "azure" else OpenAISynth
    client = make(work_dir=args.work_dir, credential_path=args.credential_path)
    if args.action == "status":
        client.retrieve_batch_task(args.task_name, print_status=True)
    elif args.action == "download":
        print(f"downloaded {len(client.download_batch_task(args.task_name))} responses")
    elif args.action == "cancel":
        client.cancel_batch_task(args.task_name)
    else:
        res = client.download_batch_task(args.task_name)
        json.dump(OpenAIBatchProcessor.extract_messages_from_responses(res), sys.stdout, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
