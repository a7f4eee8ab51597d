# SPDX-License-Identifier: Apache-2.0
"""Process launcher: one worker per GPU, torchrun-style environment, fail-fast supervision.

It accepts the launcher flags that recipes and docs of the reference pass through to its engine's
launcher (arctic_training_cli.py:24-48; projects/sequence-parallelism/README.md:77-111): ``--num_gpus``,
``--num_nodes``, ``--master_port``, ``--master_addr``, ``-H/--hostfile``, ``-q``.  On one node it spawns
the workers itself; with a hostfile it starts one copy of itself per node over ssh (``--node_rank`` is
filled in).  If any worker exits with an error the remaining workers of that node are terminated, so a
failed rank never leaves the others blocked in a collective.
"""

from __future__ import annotations

import argparse
import os
import shlex
import signal
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict
from typing import List
from typing import Optional
from typing import Tuple


def parse_hostfile(path: Path) -> List[Tuple[str, int]]:
    """Lines of ``hostname slots=N`` (comments with ``#``)."""
    hosts = []
    for line in Path(path).read_text().splitlines():
        line = line.split("#", 1)[0].strip()
        if not line:
            continue
        parts = line.split()
        slots = 0
        for p in parts[1:]:
            if p.startswith("slots="):
                slots = int(p.split("=", 1)[1])
        hosts.append((parts[0], slots))
    return hosts


def visible_gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="atb200-launch", add_help=True)
    p.add_argument("--num_gpus", "--nproc_per_node", type=int, default=-1)
    p.add_argument("--num_nodes", "--nnodes", type=int, default=1)
    p.add_argument("--node_rank", type=int, default=0)
    p.add_argument("--master_addr", type=str, default="127.0.0.1")
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("-H", "--hostfile", type=str, default=None)
    p.add_argument("-q", "--quiet", action="store_true")
    p.add_argument("--env", action="append", default=[], help="KEY=VALUE exported to every worker")
    p.add_argument("cmd", nargs=argparse.REMAINDER, help="module or script of the worker and its arguments")
    return p


def worker_env(base: Dict[str, str], rank: int, local_rank: int, world: int, addr: str, port: int) -> Dict[str, str]:
    env = dict(base)
    env.update(RANK=str(rank), LOCAL_RANK=str(local_rank), WORLD_SIZE=str(world), MASTER_ADDR=addr,
               MASTER_PORT=str(port), LOCAL_WORLD_SIZE=base.get("LOCAL_WORLD_SIZE", "1"))
    return env


def run_local(cmd: List[str], nproc: int, node_rank: int, num_nodes: int, addr: str, port: int,
              extra_env: Dict[str, str], quiet: bool = False, poll_s: float = 0.2) -> int:
    """Spawn ``nproc`` workers and supervise them; returns the first non-zero exit code (or 0)."""
    world = nproc * num_nodes
    base = dict(os.environ)
    base.update(extra_env)
    base["LOCAL_WORLD_SIZE"] = str(nproc)
    procs: List[subprocess.Popen] = []
    for lr in range(nproc):
        env = worker_env(base, node_rank * nproc + lr, lr, world, addr, port)
        out = subprocess.DEVNULL if (quiet and lr != 0) else None
        procs.append(subprocess.Popen(cmd + [f"--local_rank={lr}"], env=env, stdout=out, start_new_session=True))
    code = 0
    try:
        alive = set(range(nproc))
        while alive:
            for i in list(alive):
                rc = procs[i].poll()
                if rc is None:
                    continue
                alive.discard(i)
                if rc != 0 and code == 0:
                    code = rc
                    for j in alive:  # fail fast: do not leave peers waiting in a collective
                        _terminate(procs[j])
            time.sleep(poll_s)
    except KeyboardInterrupt:
        code = 130
        for p in procs:
            _terminate(p)
    return code


def _terminate(p: subprocess.Popen, grace_s: float = 5.0) -> None:
    if p.poll() is not None:
        return
    try:
        os.killpg(p.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    t0 = time.time()
    while p.poll() is None and time.time() - t0 < grace_s:
        time.sleep(0.05)
    if p.poll() is None:
        try:
            os.killpg(p.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    cmd = [c for c in args.cmd if c != "--"]
    if not cmd:
        raise SystemExit("no worker command given")
    if cmd[0].endswith(".py") or os.path.exists(cmd[0]) and not os.access(cmd[0], os.X_OK):
        cmd = [sys.executable, "-u"] + cmd
    extra_env = dict(kv.split("=", 1) for kv in args.env)
    nproc = args.num_gpus if args.num_gpus > 0 else max(1, visible_gpu_count())
    if args.hostfile and args.num_nodes >= 1 and os.getenv("ATB200_LAUNCH_CHILD") != "1":
        hosts = parse_hostfile(Path(args.hostfile))[: args.num_nodes if args.num_nodes > 1 else None]
        if len(hosts) > 1:
            return _run_multinode(hosts, args, cmd, nproc)
    return run_local(cmd, nproc, args.node_rank, args.num_nodes, args.master_addr, args.master_port, extra_env, args.quiet)


def _run_multinode(hosts, args, cmd: List[str], nproc: int) -> int:
    master = hosts[0][0] if args.master_addr in ("127.0.0.1", "localhost") else args.master_addr
    exports = " ".join(f"{k}={shlex.quote(v)}" for k, v in os.environ.items() if k.startswith(("WANDB", "NCCL", "ATB200", "AT_")))
    procs = []
    for node_rank, (host, slots) in enumerate(hosts):
        n = slots or nproc
        remote = (
            f"cd {shlex.quote(os.getcwd())} && ATB200_LAUNCH_CHILD=1 {exports} {shlex.quote(sys.executable)} -m "
            f"arctictraining_b200.launcher.local --num_gpus {n} --num_nodes {len(hosts)} --node_rank {node_rank} "
            f"--master_addr {master} --master_port {args.master_port} -- " + " ".join(shlex.quote(c) for c in cmd)
        )
        procs.append(subprocess.Popen(["ssh", "-o", "StrictHostKeyChecking=no", host, remote]))
    code = 0
    for p in procs:
        rc = p.wait()
        code = code or rc
    return code


if __name__ == "__main__":
    sys.exit(main())
