"""Host-side failure detection: per-rank step heartbeats through the rendezvous store.

Every rank publishes ``(step, wall time)`` after each optimizer step; a daemon thread on every
rank reads all peers' entries and, when some rank has not advanced for ``timeout_s`` seconds
while this rank has, calls ``on_failure(stale_ranks)`` — by default it prints which ranks are
missing and exits the process with status 3 so the launcher can restart from the last complete
checkpoint. Nothing here touches the GPU: a hung or dead peer is noticed on the host before the
next collective is issued (the reference only has the 3-minute process-group timeout,
train.py:137-143).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, List, Optional

import torch.distributed as dist


class StepWatchdog:
    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 600.0, poll_s: float = 5.0,
                 on_failure: Optional[Callable[[List[int]], None]] = None, prefix: str = "pico_hb"):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix
        self.on_failure = on_failure or self._default_failure
        self._stop = threading.Event()
        self._thread = None
        self._my_step = -1
        self.failed_ranks: List[int] = []
        if store is not None and world_size > 1:
            self.beat(-1)
            self._thread = threading.Thread(target=self._run, daemon=True, name="pico-watchdog")
            self._thread.start()

    @classmethod
    def from_env(cls, rank: int, world_size: int):
        """Watchdog on the default process group's store; PICO_WATCHDOG_TIMEOUT=0 disables it."""
        timeout = float(os.environ.get("PICO_WATCHDOG_TIMEOUT", "600"))
        store = None
        if timeout > 0 and dist.is_initialized() and world_size > 1:
            store = dist.distributed_c10d._get_default_store()
        return cls(store, rank, world_size, timeout_s=timeout)

    def beat(self, step: int) -> None:
        self._my_step = step
        if self.store is not None:
            self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time()}")

    def _read(self, r: int):
        try:
            raw = self.store.get(f"{self.prefix}/{r}").decode()
            step, ts = raw.split(":")
            return int(step), float(ts)
        except Exception:
            return None

    def check_once(self, now: Optional[float] = None) -> List[int]:
        """Ranks whose heartbeat is older than the timeout and behind this rank's step."""
        now = time.time() if now is None else now
        stale = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            hb = self._read(r)
            if hb is None:
                continue
            step, ts = hb
            if step < self._my_step and now - ts > self.timeout_s:
                stale.append(r)
        return stale

    def _run(self):
        while not self._stop.wait(self.poll_s):
            stale = self.check_once()
            if stale:
                self.failed_ranks = stale
                self.on_failure(stale)
                return

    def _default_failure(self, stale):
        print(f"[watchdog] rank {self.rank}: no heartbeat from ranks {stale} for {self.timeout_s}s; aborting",
              flush=True)
        os._exit(3)

    def stop(self):
        self._stop.set()
