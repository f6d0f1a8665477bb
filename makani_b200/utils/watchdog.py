"""Failure detection for multi-process jobs: heartbeats, step deadlines and a coordinated abort.

The reference has no such layer (it resumes from checkpoints at start-up, makani/train.py:130-136, and retries file
opens, makani/utils/dataloaders/dali_es_helper_2d.py:447-456); long jobs instead hang until the scheduler kills them
when one rank dies inside a collective.  This module makes a lost or stuck rank visible on the *host* before the
next collective is entered:

* every rank runs a daemon thread that writes `hb/<rank> = (step, wall time)` to a key-value store (the
  `torch.distributed` TCPStore / FileStore, or an in-process dict for tests) every `interval` seconds;
* `Watchdog.check()` (called by the training loop between steps, with nothing in flight) reads the peers' entries
  and raises `RankFailure` when one is older than `timeout` seconds, when a peer posted an abort reason, or when
  this rank's own step took longer than `step_deadline`;
* `Watchdog.abort(reason)` posts the reason so that every other rank leaves at its next check instead of entering a
  collective that can never complete; `Trainer` then writes an emergency checkpoint from the ranks that are alive.

Device side, every wait in the in-tree kernels (mbarriers, peer flags) is bounded and reports through an error word
that `makani_b200.ops._ext.check_device_errors` turns into an exception, which callers forward to `abort`.
Nothing here touches a GPU; failures in the tests are made on the host (a rank that stops beating, a posted abort).
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional


class RankFailure(RuntimeError):
    """A peer stopped responding, posted an abort, or the local step deadline ran out."""

    def __init__(self, message: str, ranks: Optional[List[int]] = None):
        super().__init__(message)
        self.ranks = ranks or []


class DictStore:
    """Minimal in-process stand-in for a c10d store (`set` / `get` / `check`), shared between threads in tests."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Watchdog:
    def __init__(self, store, rank: int, world_size: int, interval: float = 1.0, timeout: float = 30.0,
                 step_deadline: Optional[float] = None, clock: Callable[[], float] = time.time, prefix: str = "mkwd"):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.interval, self.timeout, self.step_deadline = interval, timeout, step_deadline
        self.clock, self.prefix = clock, prefix
        self.step = 0
        self._step_started = clock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._paused = False

    # ---- keys
    def _hb(self, r):
        return f"{self.prefix}/hb/{r}"

    def _abort_key(self):
        return f"{self.prefix}/abort"

    # ---- heartbeat
    def beat(self) -> None:
        self.store.set(self._hb(self.rank), f"{self.step}:{self.clock():.3f}")

    def _run(self):
        while not self._stop.wait(self.interval):
            if not self._paused:
                try:
                    self.beat()
                except Exception:
                    return      # the store is gone: the job is shutting down

    def start(self) -> "Watchdog":
        self.beat()
        self._thread = threading.Thread(target=self._run, name="makani-b200-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)

    def pause(self, flag: bool = True) -> None:
        """Stops beating without stopping the thread (used by tests to play a rank that froze)."""
        self._paused = flag

    # ---- step bookkeeping
    def begin_step(self, step: Optional[int] = None) -> None:
        self.step = self.step + 1 if step is None else step
        self._step_started = self.clock()

    # ---- checks
    def peers(self) -> Dict[int, Optional[tuple]]:
        out: Dict[int, Optional[tuple]] = {}
        for r in range(self.world_size):
            if r == self.rank:
                continue
            if not self.store.check([self._hb(r)]):
                out[r] = None
                continue
            raw = self.store.get(self._hb(r)).decode()
            s, t = raw.split(":")
            out[r] = (int(s), float(t))
        return out

    def aborted(self) -> Optional[str]:
        if self.store.check([self._abort_key()]):
            return self.store.get(self._abort_key()).decode()
        return None

    def check(self, require_all_started: bool = True) -> None:
        """Raises `RankFailure` if the job should stop.  Call it between steps, before entering a collective."""
        reason = self.aborted()
        if reason is not None:
            raise RankFailure(f"abort posted: {reason}")
        now = self.clock()
        if self.step_deadline is not None and now - self._step_started > self.step_deadline:
            self.abort(f"rank {self.rank}: step {self.step} exceeded its deadline of {self.step_deadline}s")
            raise RankFailure(f"step {self.step} exceeded its deadline", [self.rank])
        dead = []
        for r, hb in self.peers().items():
            if hb is None:
                if require_all_started:
                    dead.append(r)
                continue
            if now - hb[1] > self.timeout:
                dead.append(r)
        if dead:
            self.abort(f"rank {self.rank}: no heartbeat from ranks {dead} for more than {self.timeout}s")
            raise RankFailure(f"no heartbeat from ranks {dead}", dead)

    def abort(self, reason: str) -> None:
        if self.aborted() is None:
            self.store.set(self._abort_key(), reason)


def from_process_group(interval: float = 1.0, timeout: float = 60.0, step_deadline: Optional[float] = None) -> Optional[Watchdog]:
    """Watchdog on the default process group's store, or None when the job has a single process."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    store = dist.distributed_c10d._get_default_store()
    return Watchdog(store, dist.get_rank(), dist.get_world_size(), interval, timeout, step_deadline).start()
