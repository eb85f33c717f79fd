"""Replica mode (one process per GPU, no data-path collective) on CPU: two gloo ranks."""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

WORKER = r"""
import json, os, sys, time
from pathlib import Path
sys.path.insert(0, os.environ["AGI_ROOT"])
from aginfer_b200.replicas import ReplicaGroup

group = ReplicaGroup.from_env("gloo")
marker = Path(os.environ["AGI_MARKER"])

def build_once():
    # rank 0 must have finished before anyone else starts
    if group.rank == 0:
        time.sleep(0.3)
        marker.write_text("built")
        return "built-by-0"
    assert marker.read_text() == "built"
    return "seen-by-%d" % group.rank

first = group.rank0_first(build_once)
ms = group.max_over_ranks([10.0 + 5.0 * group.rank, 40.0 - 7.0 * group.rank])
rate = group.whole_job_rate(100, ms[0])
group.barrier()
print(json.dumps({"rank": group.rank, "world": group.world, "first": first, "ms": ms, "rate": rate}), flush=True)
group.close()
"""


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_agree_on_the_slowest_time(tmp_path):
    port = free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), AGI_ROOT=str(ROOT), AGI_MARKER=str(tmp_path / "marker"))
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    assert [o["first"] for o in outs] == ["built-by-0", "seen-by-1"]
    for o in outs:
        assert o["world"] == 2
        assert o["ms"] == [15.0, 40.0]                       # element-wise max over ranks
        assert abs(o["rate"] - 2 * 100 / 0.015) < 1e-6       # whole job: both replicas' units over the slowest time


def test_single_process_needs_no_group(monkeypatch):
    from aginfer_b200.replicas import ReplicaGroup
    for name in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        monkeypatch.delenv(name, raising=False)
    group = ReplicaGroup.from_env("gloo")
    assert (group.world, group.rank) == (1, 0)
    assert group.max_over_ranks([3, 4.5]) == [3.0, 4.5]
    assert group.rank0_first(lambda: 7) == 7
    assert group.whole_job_rate(10, 5.0) == 2000.0
    group.close()


def test_reference_arm_other_ranks_exit_quietly():
    """Under a multi-rank launch only rank 0 runs the reference arm; the others exit 0 without output."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                          env=env, capture_output=True, text=True, timeout=120)
    assert done.returncode == 0 and done.stdout.strip() == ""
