# SPDX-License-Identifier: Apache-2.0
"""Run a list of shell commands over the GPUs of one node, each command on its own group of GPUs, starting the next
command as soon as a group becomes free.  Used to fan `vllm_data_generation.py` shards out over 8 GPUs.

    python multigpu_runner.py --gpus-per-job 1 --commands jobs.txt

Every line of `jobs.txt` is one command; `CUDA_VISIBLE_DEVICES` is set for it.  A failing command is reported and does
not stop the others.  Reference: projects/arctic_lstm_speculator/multigpu_runner.py.
"""

import argparse
import os
import subprocess
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--commands", required=True)
    ap.add_argument("--gpus-per-job", type=int, default=1)
    ap.add_argument("--num-gpus", type=int, default=0, help="0 = all visible GPUs")
    args = ap.parse_args()
    n = args.num_gpus
    if not n:
        import torch

        n = torch.cuda.device_count()
    groups = [list(range(i, i + args.gpus_per_job)) for i in range(0, n - args.gpus_per_job + 1, args.gpus_per_job)]
    jobs = [line.strip() for line in open(args.commands) if line.strip() and not line.startswith("#")]
    running = {}
    failed = []
    while jobs or running:
        for gi, g in enumerate(groups):
            if gi not in running and jobs:
                cmd = jobs.pop(0)
                env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(map(str, g)))
                running[gi] = (subprocess.Popen(cmd, shell=True, env=env), cmd)
        for gi in list(running):
            proc, cmd = running[gi]
            if proc.poll() is not None:
                if proc.returncode != 0:
                    failed.append(cmd)
                del running[gi]
        time.sleep(1.0)
    if failed:
        raise SystemExit("failed:\n" + "\n".join(failed))


if __name__ == "__main__":
    main()
