# SPDX-License-Identifier: Apache-2.0
"""Process launcher: one worker per GPU, torchrun-style environment, fail-fast supervision.

It accepts the launcher flags that recipes and docs of the reference pass through to its engine's
launcher (arctic_training_cli.py:24-48; projects/sequence-parallelism/README.md:77-111): ``--num_gpus``,
``--num_nodes``, ``--master_port``, ``--master_addr``, ``-H/--hostfile``, ``-i/--include``, ``-e/--exclude``,
``--no_local_rank``, ``-q``.  On one node it spawns the workers itself; with a hostfile it starts one copy of itself
per node over ssh (``--node_rank`` is filled in).  If any worker exits with an error the remaining workers of that
node are terminated - and, across nodes, the launchers of the other nodes - so a failed rank never leaves the others
blocked in a collective.  ``KEY=VALUE`` lines of an environment file (``.deepspeed_env`` in the working or the home
directory, or the file ``DS_ENV_FILE`` names) are exported to every worker on every node.
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


def parse_resource_filter(spec: str) -> Dict[str, Optional[List[int]]]:
    """``host1:0,1@host2`` -> ``{"host1": [0, 1], "host2": None}`` (``None``: every slot of that host)."""
    out: Dict[str, Optional[List[int]]] = {}
    for part in filter(None, (p.strip() for p in spec.split("@"))):
        host, _, slots = part.partition(":")
        out[host] = sorted({int(x) for x in slots.split(",") if x.strip()}) if slots else None
    return out


def select_resources(hosts: List[Tuple[str, int]], include: str = "", exclude: str = "",
                     default_slots: int = 0) -> List[Tuple[str, List[int]]]:
    """Apply ``--include`` / ``--exclude`` to the hosts of a hostfile (or to ``[("localhost", n)]``).  Returns
    ``[(host, [device ids])]`` without the hosts that are left with no device."""
    if include and exclude:
        raise ValueError("--include and --exclude are mutually exclusive")
    pool = [(h, list(range(n or default_slots))) for h, n in hosts]
    known = {h for h, _ in pool}
    wanted = parse_resource_filter(include or exclude)
    for h in wanted:
        if h not in known:
            raise ValueError(f"host {h!r} of the resource filter is not among the available hosts {sorted(known)}")
    out = []
    for host, slots in pool:
        if include:
            if host not in wanted:
                continue
            pick = wanted[host]
            bad = [] if pick is None else [d for d in pick if d not in slots]
            if bad:
                raise ValueError(f"{host} has no slot(s) {bad}")
            slots = slots if pick is None else pick
        elif exclude and host in wanted:
            drop = wanted[host]
            slots = [] if drop is None else [d for d in slots if d not in drop]
        if slots:
            out.append((host, slots))
    return out


def read_env_file(paths: Optional[List[Path]] = None) -> Dict[str, str]:
    """``KEY=VALUE`` lines (``#`` comments, optional ``export``) of the first environment file that exists."""
    if paths is None:
        named = os.getenv("DS_ENV_FILE")
        paths = [Path(named)] if named else [Path.cwd() / ".deepspeed_env", Path.home() / ".deepspeed_env"]
    for path in paths:
        if path.is_file():
            env: Dict[str, str] = {}
            for line in path.read_text().splitlines():
                line = line.strip()
                if not line or line.startswith("#") or "=" not in line:
                    continue
                key, value = line.removeprefix("export ").split("=", 1)
                env[key.strip()] = value.strip().strip("'\"")
            return env
    return {}


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
    p.add_argument("-i", "--include", type=str, default="", help="hosts / devices to use: host1:0,1@host2")
    p.add_argument("-e", "--exclude", type=str, default="", help="hosts / devices to leave out: host1:2,3")
    p.add_argument("--no_local_rank", action="store_true", help="do not append --local_rank=N to the worker command")
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
              extra_env: Dict[str, str], quiet: bool = False, poll_s: float = 0.2, devices: Optional[List[int]] = None,
              pass_local_rank: bool = True, world: Optional[int] = None, rank_offset: Optional[int] = None) -> int:
    """Spawn ``nproc`` workers and supervise them; returns the first non-zero exit code (or 0).  ``devices`` restricts
    the workers to those GPUs (``CUDA_VISIBLE_DEVICES``); ``world`` / ``rank_offset`` are given when the nodes of a
    job do not all run the same number of workers."""
    world = nproc * num_nodes if world is None else world
    rank_offset = node_rank * nproc if rank_offset is None else rank_offset
    base = dict(os.environ)
    base.update(extra_env)
    base["LOCAL_WORLD_SIZE"] = str(nproc)
    if devices is not None:
        base["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, devices))
    procs: List[subprocess.Popen] = []
    for lr in range(nproc):
        env = worker_env(base, rank_offset + lr, lr, world, addr, port)
        out = subprocess.DEVNULL if (quiet and lr != 0) else None
        argv = cmd + [f"--local_rank={lr}"] if pass_local_rank else list(cmd)
        procs.append(subprocess.Popen(argv, env=env, stdout=out, start_new_session=True))
    code = 0
    restore = _stop_on_signals()
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
    finally:
        restore()
    return code


def _stop_on_signals():
    """SIGTERM / SIGHUP (the parent launcher gave up, the ssh connection went away) end the supervision loop like
    Ctrl-C does, so the workers - which run in sessions of their own - are taken down with the launcher instead of
    being orphaned.  Returns a function that puts the previous handlers back."""
    def stop(signum, frame):
        raise KeyboardInterrupt

    previous = {}
    for sig in (signal.SIGTERM, signal.SIGHUP):
        try:
            previous[sig] = signal.signal(sig, stop)
        except ValueError:  # not the main thread: signals cannot be handled here
            pass

    def restore() -> None:
        for sig, handler in previous.items():
            signal.signal(sig, handler)

    return restore


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
    p = build_parser()
    p.add_argument("--world_size", type=int, default=0, help=argparse.SUPPRESS)     # set by the multi-node parent
    p.add_argument("--rank_offset", type=int, default=-1, help=argparse.SUPPRESS)
    p.add_argument("--devices", type=str, default="", help=argparse.SUPPRESS)
    args = p.parse_args(argv)
    cmd = [c for c in args.cmd if c != "--"]
    if not cmd:
        raise SystemExit("no worker command given")
    if cmd[0].endswith(".py") or os.path.exists(cmd[0]) and not os.access(cmd[0], os.X_OK):
        cmd = [sys.executable, "-u"] + cmd
    extra_env = {**read_env_file(), **dict(kv.split("=", 1) for kv in args.env)}
    nproc = args.num_gpus if args.num_gpus > 0 else max(1, visible_gpu_count())
    child = os.getenv("ATB200_LAUNCH_CHILD") == "1"
    devices = [int(d) for d in args.devices.split(",") if d] or None
    if not child:
        if args.hostfile:
            hosts = parse_hostfile(Path(args.hostfile))
            if args.num_nodes > 1:
                hosts = hosts[: args.num_nodes]
            picked = select_resources(hosts, args.include, args.exclude, default_slots=nproc)
            if args.num_gpus > 0:
                picked = [(h, d[: args.num_gpus]) for h, d in picked]
            if len(picked) > 1:
                return _run_multinode(picked, args, cmd, extra_env)
            if picked and (args.include or args.exclude):
                devices = picked[0][1]
        elif args.include or args.exclude:
            picked = select_resources([("localhost", nproc)], args.include, args.exclude)
            if not picked:
                raise SystemExit("the resource filter leaves no device")
            devices = picked[0][1]
            if args.num_gpus > 0:
                devices = devices[: args.num_gpus]
        if devices is not None:
            nproc = len(devices)
    return run_local(cmd, nproc, args.node_rank, args.num_nodes, args.master_addr, args.master_port, extra_env, args.quiet,
                     devices=devices, pass_local_rank=not args.no_local_rank, world=args.world_size or None,
                     rank_offset=args.rank_offset if args.rank_offset >= 0 else None)


def node_commands(picked: List[Tuple[str, List[int]]], args, cmd: List[str], extra_env: Dict[str, str]) -> List[Tuple[str, str]]:
    """(host, remote shell command) per node: a copy of this launcher with the node's rank range and devices."""
    master = picked[0][0] if args.master_addr in ("127.0.0.1", "localhost") else args.master_addr
    exported = {k: v for k, v in os.environ.items() if k.startswith(("WANDB", "NCCL", "ATB200", "AT_", "HF_", "PYTHONPATH"))}
    exported.update(extra_env)
    exports = " ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(exported.items()))
    world = sum(len(d) for _, d in picked)
    out, offset = [], 0
    for node_rank, (host, devices) in enumerate(picked):
        flags = f"--num_gpus {len(devices)} --num_nodes {len(picked)} --node_rank {node_rank} --master_addr {master} " \
                f"--master_port {args.master_port} --world_size {world} --rank_offset {offset} " \
                f"--devices {','.join(map(str, devices))}" + (" --no_local_rank" if args.no_local_rank else "") + \
                (" -q" if args.quiet else "")
        out.append((host, f"cd {shlex.quote(os.getcwd())} && ATB200_LAUNCH_CHILD=1 {exports} {shlex.quote(sys.executable)} -m "
                          f"arctictraining_b200.launcher.local {flags} -- " + " ".join(shlex.quote(c) for c in cmd)))
        offset += len(devices)
    return out


def _run_multinode(picked, args, cmd: List[str], extra_env: Dict[str, str], poll_s: float = 0.5,
                   remote_shell: Optional[List[str]] = None) -> int:
    remote_shell = remote_shell or ["ssh", "-o", "StrictHostKeyChecking=no"]
    procs = [subprocess.Popen(remote_shell + [host, remote], start_new_session=True)
             for host, remote in node_commands(picked, args, cmd, extra_env)]
    code = 0
    alive = set(range(len(procs)))
    try:
        while alive:
            for i in list(alive):
                rc = procs[i].poll()
                if rc is None:
                    continue
                alive.discard(i)
                if rc != 0 and code == 0:
                    code = rc
                    for j in alive:  # a node failed: the other nodes would wait in a collective for ever
                        _terminate(procs[j])
            time.sleep(poll_s)
    except KeyboardInterrupt:
        code = 130
        for p_ in procs:
            _terminate(p_)
    return code


if __name__ == "__main__":
    sys.exit(main())
