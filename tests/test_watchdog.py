"""Failure detection on the host: a rank that stops beating, a posted abort and a missed step deadline are all seen
by the survivors before their next step; no GPU is involved and nothing is made to fault."""

import os
import subprocess
import sys
import time

import pytest

from makani_b200.utils.watchdog import DictStore, RankFailure, Watchdog

HERE = os.path.dirname(os.path.abspath(__file__))


class FakeClock:
    def __init__(self):
        self.t = 1000.0

    def __call__(self):
        return self.t


def _pair(timeout=5.0, deadline=None):
    store, clock = DictStore(), FakeClock()
    a = Watchdog(store, 0, 2, interval=0.05, timeout=timeout, step_deadline=deadline, clock=clock)
    b = Watchdog(store, 1, 2, interval=0.05, timeout=timeout, step_deadline=deadline, clock=clock)
    return store, clock, a, b


def test_healthy_ranks_pass():
    _, clock, a, b = _pair()
    a.beat(); b.beat()
    clock.t += 1.0
    a.check(); b.check()


def test_silent_rank_is_detected_and_abort_propagates():
    _, clock, a, b = _pair(timeout=5.0)
    a.beat(); b.beat()
    clock.t += 10.0
    a.beat()                       # rank 1 never beats again
    with pytest.raises(RankFailure) as ei:
        a.check()
    assert ei.value.ranks == [1]
    # the abort reason is now in the store: any other rank leaves at its next check
    c = Watchdog(a.store, 1, 2, clock=clock)
    with pytest.raises(RankFailure, match="abort posted"):
        c.check()


def test_rank_that_never_started():
    _, clock, a, _ = _pair()
    a.beat()
    with pytest.raises(RankFailure):
        a.check(require_all_started=True)
    _, clock, a, _ = _pair()
    a.beat()
    a.check(require_all_started=False)


def test_step_deadline():
    _, clock, a, b = _pair(deadline=2.0)
    a.beat(); b.beat()
    a.begin_step()
    clock.t += 1.0
    a.check()
    clock.t += 5.0
    b.beat()
    with pytest.raises(RankFailure, match="deadline"):
        a.check()


def test_heartbeat_thread_and_pause():
    store = DictStore()
    a = Watchdog(store, 0, 2, interval=0.02, timeout=0.3).start()
    b = Watchdog(store, 1, 2, interval=0.02, timeout=0.3).start()
    try:
        time.sleep(0.1)
        a.check()
        b.pause()                  # rank 1 freezes (host-side stand-in for a hung process)
        time.sleep(0.6)
        with pytest.raises(RankFailure):
            a.check()
    finally:
        a.stop(); b.stop()


WORKER = r"""
import os, sys, time
sys.path.insert(0, sys.argv[1])
import torch.distributed as dist
from makani_b200.utils import watchdog
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
wd = watchdog.from_process_group(interval=0.1, timeout=1.0)
rank = dist.get_rank()
dist.barrier()
for step in range(1000):
    wd.begin_step(step)
    if rank == 1 and step == 3:
        os._exit(0)                # this rank dies between steps, with nothing in flight
    time.sleep(0.2)
    try:
        wd.check()
    except watchdog.RankFailure as e:
        print("DETECTED", e.ranks, flush=True)
        wd.stop()
        os._exit(0)
print("NOT DETECTED", flush=True)
"""


def test_process_exit_is_detected_by_survivor(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "wd_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    procs = [subprocess.Popen([sys.executable, str(script), os.path.dirname(HERE), str(port), str(r)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    out0, _ = procs[0].communicate(timeout=120)
    procs[1].communicate(timeout=120)
    assert "DETECTED [1]" in out0, out0
