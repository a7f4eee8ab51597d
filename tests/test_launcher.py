# SPDX-License-Identifier: Apache-2.0
"""Process launcher: resource filters, environment file, worker environment, node fan-out through a stand-in remote
shell (both "nodes" are this machine) and fail-fast supervision across nodes."""
import os
import stat
import sys
import time
from pathlib import Path
from types import SimpleNamespace

import pytest

from arctictraining_b200.launcher import local as launcher

ROOT = Path(__file__).resolve().parent.parent


def test_resource_filters():
    hosts = [("a", 4), ("b", 4), ("c", 2)]
    assert launcher.parse_resource_filter("a:0,1@b") == {"a": [0, 1], "b": None}
    assert launcher.select_resources(hosts) == [("a", [0, 1, 2, 3]), ("b", [0, 1, 2, 3]), ("c", [0, 1])]
    assert launcher.select_resources(hosts, include="a:1,3@c") == [("a", [1, 3]), ("c", [0, 1])]
    assert launcher.select_resources(hosts, exclude="a@b:0,1,2") == [("b", [3]), ("c", [0, 1])]
    assert launcher.select_resources([("localhost", 0)], include="localhost:2", default_slots=4) == [("localhost", [2])]
    with pytest.raises(ValueError, match="mutually exclusive"):
        launcher.select_resources(hosts, include="a", exclude="b")
    with pytest.raises(ValueError, match="not among"):
        launcher.select_resources(hosts, include="z")
    with pytest.raises(ValueError, match="no slot"):
        launcher.select_resources(hosts, include="c:5")


def test_environment_file(tmp_path, monkeypatch):
    f = tmp_path / ".deepspeed_env"
    f.write_text("# comment\nNCCL_DEBUG=INFO\nexport HF_HOME='/data/hf'\nbroken line\n\nA=b=c\n")
    assert launcher.read_env_file([tmp_path / "missing", f]) == {"NCCL_DEBUG": "INFO", "HF_HOME": "/data/hf", "A": "b=c"}
    monkeypatch.setenv("DS_ENV_FILE", str(f))
    assert launcher.read_env_file()["NCCL_DEBUG"] == "INFO"
    monkeypatch.delenv("DS_ENV_FILE")
    monkeypatch.chdir(tmp_path)
    assert launcher.read_env_file()["A"] == "b=c"


_WORKER = ("import os, sys, pathlib; "
           "pathlib.Path(sys.argv[1], 'rank' + os.environ['RANK']).write_text(' '.join([os.environ['WORLD_SIZE'], "
           "os.environ['LOCAL_RANK'], os.environ.get('CUDA_VISIBLE_DEVICES', '-'), os.environ.get('FROM_FILE', '-'), "
           "str(len(sys.argv))]))")


def test_local_run_with_device_filter_and_env_file(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    (tmp_path / ".deepspeed_env").write_text("FROM_FILE=yes\n")
    worker = tmp_path / "w.py"
    worker.write_text(_WORKER.replace("; ", "\n"))
    rc = launcher.main(["--num_gpus", "4", "--include", "localhost:1,3", "--master_port", "29611", "--no_local_rank",
                        "--", str(worker), str(tmp_path)])
    assert rc == 0
    got = {p.name: p.read_text().split() for p in tmp_path.glob("rank*")}
    assert got == {"rank0": ["2", "0", "1,3", "yes", "2"], "rank1": ["2", "1", "1,3", "yes", "2"]}
    for p in tmp_path.glob("rank*"):
        p.unlink()
    rc = launcher.main(["--num_gpus", "1", "--master_port", "29612", "--", str(worker), str(tmp_path)])
    assert rc == 0 and (tmp_path / "rank0").read_text().split()[-1] == "3"  # --local_rank=0 was appended


def _fake_remote_shell(tmp_path):
    """Stands in for ssh: drops the host argument and runs the command here."""
    sh = tmp_path / "fake_ssh.sh"
    sh.write_text('#!/usr/bin/env bash\nshift\nexec bash -c "$1"\n')
    sh.chmod(sh.stat().st_mode | stat.S_IEXEC)
    return [str(sh)]


def _args(**kw):
    base = dict(master_addr="127.0.0.1", master_port=29613, no_local_rank=False, quiet=False)
    base.update(kw)
    return SimpleNamespace(**base)


def test_nodes_get_consecutive_rank_ranges_and_their_devices(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("PYTHONPATH", str(ROOT))
    worker = tmp_path / "w.py"
    worker.write_text(_WORKER.replace("; ", "\n"))
    picked = [("nodeA", [0, 1]), ("nodeB", [2])]
    cmds = launcher.node_commands(picked, _args(), [sys.executable, str(worker), str(tmp_path)], {"FROM_FILE": "multi"})
    assert [h for h, _ in cmds] == ["nodeA", "nodeB"]
    assert "--rank_offset 0" in cmds[0][1] and "--rank_offset 2" in cmds[1][1] and "--world_size 3" in cmds[1][1]
    assert "--master_addr nodeA" in cmds[1][1] and "FROM_FILE=multi" in cmds[0][1]
    rc = launcher._run_multinode(picked, _args(), [sys.executable, str(worker), str(tmp_path)], {"FROM_FILE": "multi"},
                                 poll_s=0.05, remote_shell=_fake_remote_shell(tmp_path))
    assert rc == 0
    got = {p.name: p.read_text().split() for p in tmp_path.glob("rank*")}
    assert got == {"rank0": ["3", "0", "0,1", "multi", "3"], "rank1": ["3", "1", "0,1", "multi", "3"],
                   "rank2": ["3", "0", "2", "multi", "3"]}


def test_a_failing_node_takes_the_other_nodes_down(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("PYTHONPATH", str(ROOT))
    worker = tmp_path / "w.py"
    worker.write_text("import os, sys, time, pathlib\nif os.environ['RANK'] == '1':\n    time.sleep(2)\n    sys.exit(7)\n"
                      "pathlib.Path(sys.argv[1]).write_text(str(os.getpid()))\ntime.sleep(120)\n")
    pid_file = tmp_path / "rank0.pid"
    t0 = time.time()
    rc = launcher._run_multinode([("nodeA", [0]), ("nodeB", [0])], _args(master_port=29614),
                                 [sys.executable, str(worker), str(pid_file)], {}, poll_s=0.05,
                                 remote_shell=_fake_remote_shell(tmp_path))
    assert rc == 7 and time.time() - t0 < 60
    # the surviving node's worker went down with its launcher (it runs in a session of its own)
    pid = int(pid_file.read_text())
    deadline = time.time() + 15
    while time.time() < deadline:
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            break
        time.sleep(0.1)
    else:
        os.kill(pid, 15)
        raise AssertionError("the worker of the other node outlived its launcher")
