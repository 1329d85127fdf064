"""Symmetric memory: buffers that every GPU of a process group can address directly.

``SymmGroup(group)`` allocates device buffers whose CUDA IPC handles are exchanged over the
process group, so a kernel on one rank can load from and store to the same buffer on any other
rank through NVLink peer pointers. It also owns the group's flag words: small epoch counters
that kernels raise (release, system scope) and wait on (acquire, bounded) to order their
accesses across GPUs. Nothing here calls NCCL on the data path; the process group is used once
per allocation to exchange 64-byte handles.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from .. import ops

FLAG_SLOTS = 256
MAX_PEERS = 8
FLAG_BYTES = (FLAG_SLOTS * MAX_PEERS + FLAG_SLOTS) * 4   # flag words, then one epoch-base word per slot
MAX_EPOCH_DELTAS = 256


class _Jitter:
    """Race-detection aid. ``PICO_RACE_JITTER=<seed>`` delays the launching stream by a random time
    (0 to ``PICO_RACE_JITTER_US``, default 200 microseconds, drawn separately on every rank) before each
    operation that takes a flag epoch, i.e. before every kernel that communicates. The delays move the
    ranks against each other without changing what is computed: a run with jitter must give the same
    bits as a run without, and any difference points at an ordering that the flags do not enforce.
    Delays are real launches, so the mode is meant for eager runs (``training.cuda_graph: false``)."""

    def __init__(self):
        import os
        import random
        seed = os.environ.get("PICO_RACE_JITTER", "")
        self.rng = None
        if seed not in ("", "0"):
            rank = dist.get_rank() if dist.is_initialized() else 0
            self.rng = random.Random(int(seed) * 1009 + rank)
            self.max_cycles = int(float(os.environ.get("PICO_RACE_JITTER_US", "200")) * 1900)

    def __call__(self):
        if self.rng is not None and torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            torch.cuda._sleep(self.rng.randrange(self.max_cycles))


GUARD_BYTES = 256        # canary zone on either side of a buffer (keeps the 256-byte alignment)
GUARD_PATTERN = 0xA5


class SymmBuffer:
    def __init__(self, nbytes: int, local_ptr: int, ptrs: List[int], device_index: int, guard: int = 0):
        """``guard`` > 0: the allocation is ``guard`` bytes larger on both sides than the ``nbytes`` the
        users see; ``local_ptr`` / ``ptrs`` point past the leading zone."""
        self.nbytes, self.local_ptr, self.ptrs, self.guard = nbytes, local_ptr, ptrs, guard
        self.local = ops.ext().tensor_from_ptr(local_ptr, nbytes, device_index)
        self.guards = None
        if guard:
            e = ops.ext()
            self.guards = (e.tensor_from_ptr(local_ptr - guard, guard, device_index),
                           e.tensor_from_ptr(local_ptr + nbytes, guard, device_index))
            for g in self.guards:
                g.fill_(GUARD_PATTERN)

    def guards_intact(self) -> bool:
        return self.guards is None or all(bool((g == GUARD_PATTERN).all()) for g in self.guards)

    def view(self, dtype: torch.dtype, shape, offset_bytes: int = 0) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.tensor([], dtype=dtype).element_size()
        assert offset_bytes + nb <= self.nbytes, "view exceeds the symmetric buffer"
        return self.local[offset_bytes:offset_bytes + nb].view(dtype).view(*shape)

    def peer_ptrs(self, offset_bytes: int = 0) -> List[int]:
        return [p + offset_bytes for p in self.ptrs]


class GraphEpochs:
    """What a captured graph assumed about a group's epochs: ``used[slot]`` epochs per replay,
    starting ``rel0[slot]`` above the slot's base word."""

    def __init__(self, group: "SymmGroup", used, rel0):
        self.group, self.used, self.rel0 = group, used, rel0

    def before_replay(self) -> None:
        """Eager kernels that used one of the graph's slots since the last replay moved the epoch
        without moving the base: re-align the base (one tiny launch, only when that happened)."""
        g = self.group
        slots = [s for s in self.used if g._epochs[s] - g._base[s] != self.rel0[s]]
        if slots:
            g._add_base(slots, [g._epochs[s] - g._base[s] - self.rel0[s] for s in slots])

    def after_replay(self) -> None:
        g = self.group
        for s, n in self.used.items():
            g._epochs[s] += n
            g._base[s] += n


_LIVE_GROUPS = None      # weak set of the process's open groups (for ``check_all_canaries``)


def check_all_canaries() -> None:
    """``check_canaries`` on every open group of this process (tests call it after their last kernel)."""
    for g in list(_LIVE_GROUPS or ()):
        if not g._closed:
            g.check_canaries()


class SymmGroup:
    _jitter = None           # race-detection delays (``_Jitter``), set per instance

    def __init__(self, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert self.world <= MAX_PEERS, f"at most {MAX_PEERS} GPUs per symmetric group"
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._buffers: List[SymmBuffer] = []
        import os
        self._guard = GUARD_BYTES if os.environ.get("PICO_SYMM_CANARY", "0") == "1" else 0
        self.flags = self.alloc(FLAG_BYTES)
        self._jitter = _Jitter()
        self._epochs = [0] * FLAG_SLOTS          # absolute epoch last used per slot
        self._base = [0] * FLAG_SLOTS            # host mirror of the device's epoch-base words
        self._recording = None                   # slot -> epochs used, while a graph is being captured
        self._closed = False
        global _LIVE_GROUPS
        if _LIVE_GROUPS is None:
            import weakref
            _LIVE_GROUPS = weakref.WeakSet()
        _LIVE_GROUPS.add(self)

    def alloc(self, nbytes: int) -> SymmBuffer:
        """Collective over the group: every rank must call it with the same size."""
        e = ops.ext()
        nbytes = (nbytes + 255) // 256 * 256
        g = self._guard
        with torch.cuda.device(self.device):
            ptr, handle = e.symm_alloc(nbytes + 2 * g)
            if self.world == 1:
                ptrs = [ptr]
            else:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=self.group)
                ptrs = [ptr if r == self.rank else e.symm_open(handles[r]) for r in range(self.world)]
                dist.barrier(group=self.group)
        buf = SymmBuffer(nbytes, ptr + g, [p + g for p in ptrs], self.device.index, guard=g)
        self._buffers.append(buf)
        return buf

    def check_canaries(self) -> None:
        """With ``PICO_SYMM_CANARY=1`` every symmetric buffer sits between two 256-byte zones of a fixed
        pattern; a kernel of any rank that stores past either end of a buffer of this rank changes them.
        Synchronises and raises when a zone was touched. No-op without the switch."""
        if not self._guard:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            bad = [i for i, buf in enumerate(self._buffers) if not buf.guards_intact()]
        if bad:
            raise RuntimeError(f"symmetric buffers {bad} of rank {self.rank}: guard words overwritten "
                               f"(sizes {[self._buffers[i].nbytes for i in bad]})")

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's. Collective in effect: every rank must stop
        using the group's buffers before any rank closes (callers synchronise and barrier first)."""
        if self._closed:
            return
        self._closed = True
        e = ops.ext()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1 and dist.is_initialized() and self._guard:
                dist.barrier(group=self.group)       # every rank's kernels are done before zones are read
            damaged = [i for i, buf in enumerate(self._buffers) if not buf.guards_intact()]
            for buf in self._buffers:
                for r, p in enumerate(buf.ptrs):
                    if r != self.rank and p != buf.local_ptr:
                        e.symm_close(p - buf.guard)
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)       # nobody frees memory a peer still has mapped
            for buf in self._buffers:
                e.symm_free(buf.local_ptr - buf.guard)
        if damaged:
            self._buffers.clear()
            raise RuntimeError(f"symmetric buffers {damaged} of rank {self.rank}: guard words overwritten")
        self._buffers.clear()

    def next_epoch(self, slot: int) -> int:
        """The next epoch of ``slot`` as kernels take it: relative to the slot's device-side base
        word (zero until a CUDA graph over this group has been replayed)."""
        if self._jitter is not None:
            self._jitter()
        self._epochs[slot] += 1
        if self._recording is not None:
            self._recording[slot] = self._recording.get(slot, 0) + 1
        return self._epochs[slot] - self._base[slot]

    # -- CUDA graph support ---------------------------------------------------------------------
    def begin_graph(self) -> None:
        """Call right after stream capture starts: epochs handed out from now on belong to the graph."""
        assert self._recording is None, "nested graph capture over one symmetric group"
        self._recording = {}
        self._rel0 = {}

    def end_graph(self) -> "GraphEpochs":
        """Call at the end of the captured region (still capturing): appends the node that moves the
        device-side bases past the epochs the graph used, and returns the record ``replay`` needs."""
        used = dict(self._recording)
        self._recording = None
        slots = sorted(used)
        assert len(slots) <= MAX_EPOCH_DELTAS, "too many flag slots in one graph"
        rel0 = {s: self._epochs[s] - used[s] - self._base[s] for s in slots}
        if slots:
            ops.ext().epoch_base_add(self.flags.local_ptr, slots, [used[s] for s in slots])
            ops.count_launch()
        # the capture itself executed nothing: take the epochs back until the first replay
        for s in slots:
            self._epochs[s] -= used[s]
        return GraphEpochs(self, used, rel0)

    def _add_base(self, slots, deltas) -> None:
        ops.ext().epoch_base_add(self.flags.local_ptr, list(slots), list(deltas))
        ops.count_launch()
        for s, d in zip(slots, deltas):
            self._base[s] += d

    def signal(self, slot: int, epoch: int) -> None:
        ops.ext().signal_peers(self.flags.ptrs, self.world, self.rank, slot, epoch)
        ops.count_launch()

    def wait(self, slot: int, epoch: int, timeout_ms: int = 20000) -> None:
        ops.ext().wait_flags(self.flags.local_ptr, self.world, slot, epoch, timeout_ms)
        ops.count_launch()

    def barrier(self, slot: int = FLAG_SLOTS - 1, timeout_ms: int = 20000) -> None:
        """Device-side barrier over the group on the current stream (no host blocking)."""
        e = self.next_epoch(slot)
        self.signal(slot, e)
        self.wait(slot, e, timeout_ms)
