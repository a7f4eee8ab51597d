# SPDX-License-Identifier: Apache-2.0
"""Run a queue of shell jobs over the GPUs of one node: every job gets its own group of GPUs through
`CUDA_VISIBLE_DEVICES`, and the next job starts as soon as a group becomes free.  Used to fan
`vllm_data_generation.py` shards out over a node.

    python multigpu_runner.py jobs/                      # every jobs/*.sh, one GPU each, all visible GPUs
    python multigpu_runner.py jobs/ -n 4 --max-gpus 8    # 4 GPUs per job (tensor-parallel generation)
    python multigpu_runner.py --commands jobs.txt        # one command per line instead of a folder of scripts

A job that ended with exit code 0 leaves a marker `<folder>_done/<name>`; a second run of the same folder skips those
jobs, so an interrupted generation resumes where it stopped.  A failing job is reported at the end and does not stop
the others.  `--watch` keeps polling the folder for new scripts until interrupted.
Reference: projects/arctic_lstm_speculator/multigpu_runner.py.
"""

from __future__ import annotations

import argparse
import glob
import os
import subprocess
import time
from typing import Callable
from typing import Dict
from typing import List
from typing import Optional
from typing import Sequence
from typing import Tuple


def gpu_groups(gpus: Sequence[int], gpus_per_job: int, jobs_per_group: int = 1) -> List[List[int]]:
    """Disjoint groups of `gpus_per_job` devices (left-over devices stay idle), each listed `jobs_per_group` times."""
    whole = len(gpus) // gpus_per_job * gpus_per_job
    groups = [list(gpus[i:i + gpus_per_job]) for i in range(0, whole, gpus_per_job)]
    if not groups:
        raise ValueError(f"{len(gpus)} GPUs cannot host a job of {gpus_per_job}")
    return [g for g in groups for _ in range(jobs_per_group)]


def folder_jobs(folder: str) -> List[Tuple[str, str]]:
    """(name, command) of every `*.sh` of the folder that has no done-marker yet, in name order."""
    done = done_dir(folder)
    jobs = []
    for sh in sorted(glob.glob(os.path.join(folder, "*.sh"))):
        name = os.path.splitext(os.path.basename(sh))[0]
        if not os.path.exists(os.path.join(done, name)):
            jobs.append((name, f"bash {sh}"))
    return jobs


def done_dir(folder: str) -> str:
    return folder.rstrip("/") + "_done"


def run_queue(jobs: List[Tuple[str, str]], groups: List[List[int]], on_success: Optional[Callable[[str], None]] = None,
              more_jobs: Optional[Callable[[], List[Tuple[str, str]]]] = None, poll_s: float = 1.0) -> List[str]:
    """Run `jobs` over the GPU groups; returns the names of the jobs that failed.  `more_jobs()`, when given, is asked
    for new work whenever the queue is empty (the watch mode); it ends the run by raising KeyboardInterrupt."""
    queue = list(jobs)
    seen = {name for name, _ in queue}
    running: Dict[int, Tuple[subprocess.Popen, str]] = {}
    failed: List[str] = []
    while queue or running or more_jobs is not None:
        if not queue and more_jobs is not None:
            try:
                fresh = [j for j in more_jobs() if j[0] not in seen]
            except KeyboardInterrupt:
                more_jobs = None
                continue
            seen.update(name for name, _ in fresh)
            queue.extend(fresh)
        for slot, group in enumerate(groups):
            if slot not in running and queue:
                name, cmd = queue.pop(0)
                env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(map(str, group)))
                running[slot] = (subprocess.Popen(cmd, shell=True, env=env), name)
        for slot in list(running):
            proc, name = running[slot]
            if proc.poll() is None:
                continue
            del running[slot]
            if proc.returncode != 0:
                failed.append(name)
            elif on_success is not None:
                on_success(name)
        if queue or running or more_jobs is not None:
            time.sleep(poll_s)
    return failed


def main(argv: Optional[Sequence[str]] = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("folder", nargs="?", default=None, help="folder of *.sh job scripts")
    ap.add_argument("--commands", default=None, help="text file with one command per line")
    ap.add_argument("--gpus", default=None, help="comma-separated device ids (default: the first --max-gpus devices)")
    ap.add_argument("--max-gpus", "--max_gpus", type=int, default=0, help="0 = all visible GPUs")
    ap.add_argument("-s", "--start-gpu", "--start_gpu", type=int, default=0)
    ap.add_argument("-n", "--gpus-per-job", "--gpus_per_each_proc", type=int, default=1)
    ap.add_argument("-j", "--jobs-per-group", "--proc_num_for_each_gpu", type=int, default=1)
    ap.add_argument("--watch", "--inf", action="store_true", help="keep polling the folder for new scripts")
    args = ap.parse_args(argv)
    if (args.folder is None) == (args.commands is None):
        ap.error("give a folder of scripts or --commands, not both")
    if args.gpus:
        gpus = [int(g) for g in args.gpus.split(",")]
    else:
        n = args.max_gpus
        if not n:
            import torch

            n = torch.cuda.device_count()
        gpus = list(range(args.start_gpu, args.start_gpu + n))
    groups = gpu_groups(gpus, args.gpus_per_job, args.jobs_per_group)
    if args.commands:
        lines = [line.strip() for line in open(args.commands)]
        jobs = [(f"line{i}", c) for i, c in enumerate(lines) if c and not c.startswith("#")]
        failed = run_queue(jobs, groups)
    else:
        os.makedirs(done_dir(args.folder), exist_ok=True)

        def mark(name: str) -> None:
            open(os.path.join(done_dir(args.folder), name), "w").close()

        more = (lambda: folder_jobs(args.folder)) if args.watch else None
        failed = run_queue(folder_jobs(args.folder), groups, on_success=mark, more_jobs=more)
    if failed:
        raise SystemExit("failed jobs:\n" + "\n".join(failed))


if __name__ == "__main__":
    main()
