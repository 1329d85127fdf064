"""Host-side failure detection: per-rank step heartbeats through the rendezvous store.

Every rank publishes its step counter after each optimizer step; a daemon thread on every rank
reads all peers' entries and notes, on its own clock, when each entry last changed. A peer is
stale when its entry has not changed for ``timeout_s`` seconds and it is not ahead of this rank.
Two cases follow: the peer is behind (it died or hung between steps), or the whole job sits in
the same step because one rank hung inside it and the others block in its collectives — then
every rank sees every other rank stale and its own last step equally old. Either way
``on_failure(stale_ranks)`` is called — by default it prints which ranks are missing and exits
the process with status 3 so the launcher can restart from the last complete checkpoint. Ages are
measured with the reader's monotonic clock from the moment it saw the value change, so clock
differences between hosts do not matter. Nothing here touches the GPU: a hung or dead peer is noticed on the host before the
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
        self._my_beat_at = time.monotonic()
        self._seen = {}            # peer rank -> (last value read, local time it was first seen)
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
        self._my_beat_at = time.monotonic()
        if self.store is not None:
            self.store.set(f"{self.prefix}/{self.rank}", str(step))

    def _read(self, r: int):
        try:
            return int(self.store.get(f"{self.prefix}/{r}").decode().split(":")[0])
        except Exception:
            return None

    def check_once(self, now: Optional[float] = None) -> List[int]:
        """Ranks that have made no progress for ``timeout_s``: behind this rank, or in the same step
        while this rank has been stuck there for as long. ``now``: this rank's monotonic time."""
        now = time.monotonic() if now is None else now
        stale = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            step = self._read(r)
            if step is None:
                continue
            seen = self._seen.get(r)
            if seen is None or seen[0] != step:
                self._seen[r] = seen = (step, now)
            if now - seen[1] <= self.timeout_s:
                continue
            if step < self._my_step or (step == self._my_step and now - self._my_beat_at > self.timeout_s):
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
