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


class SymmBuffer:
    def __init__(self, nbytes: int, local_ptr: int, ptrs: List[int], device_index: int):
        self.nbytes, self.local_ptr, self.ptrs = nbytes, local_ptr, ptrs
        self.local = ops.ext().tensor_from_ptr(local_ptr, nbytes, device_index)

    def view(self, dtype: torch.dtype, shape, offset_bytes: int = 0) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.tensor([], dtype=dtype).element_size()
        assert offset_bytes + nb <= self.nbytes, "view exceeds the symmetric buffer"
        return self.local[offset_bytes:offset_bytes + nb].view(dtype).view(*shape)

    def peer_ptrs(self, offset_bytes: int = 0) -> List[int]:
        return [p + offset_bytes for p in self.ptrs]


class SymmGroup:
    def __init__(self, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert self.world <= MAX_PEERS, f"at most {MAX_PEERS} GPUs per symmetric group"
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._buffers: List[SymmBuffer] = []
        self.flags = self.alloc(FLAG_SLOTS * MAX_PEERS * 4)
        self._epochs = [0] * FLAG_SLOTS

    def alloc(self, nbytes: int) -> SymmBuffer:
        """Collective over the group: every rank must call it with the same size."""
        e = ops.ext()
        nbytes = (nbytes + 255) // 256 * 256
        with torch.cuda.device(self.device):
            ptr, handle = e.symm_alloc(nbytes)
            if self.world == 1:
                ptrs = [ptr]
            else:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=self.group)
                ptrs = [ptr if r == self.rank else e.symm_open(handles[r]) for r in range(self.world)]
                dist.barrier(group=self.group)
        buf = SymmBuffer(nbytes, ptr, ptrs, self.device.index)
        self._buffers.append(buf)
        return buf

    def next_epoch(self, slot: int) -> int:
        self._epochs[slot] += 1
        return self._epochs[slot]

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
