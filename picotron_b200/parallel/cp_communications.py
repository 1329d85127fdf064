"""Ring exchange for context parallelism.

``ContextCommunicate`` batches the isend/irecv pairs of one ring step and lets the caller
overlap them with a block of attention: ``send_recv`` queues a transfer to the next rank and
from the previous one, ``commit`` posts the batch, ``wait`` completes it. Unlike
picotron/context_parallel/cp_communications.py:63-79 ``wait`` only waits for the requests (on
GPUs that is a stream dependency) instead of synchronising the whole device, so the ring also
runs on CPU/gloo.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm

VERBOSE = os.environ.get("VERBOSE", "0") == "1"


class ContextCommunicate:
    def __init__(self, msg: str = "", group=None, send_rank: Optional[int] = None, recv_rank: Optional[int] = None):
        m = pgm.get_pgm()
        self.msg = msg
        self.group = group if group is not None else m.cp_group
        self.send_rank = m.cp_send_rank if send_rank is None else send_rank
        self.recv_rank = m.cp_recv_rank if recv_rank is None else recv_rank
        self._ops: List[dist.P2POp] = []
        self._reqs = None
        self._keepalive: List[torch.Tensor] = []

    def send_recv(self, tensor_to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty_like(tensor_to_send) if recv_tensor is None else recv_tensor
        t = tensor_to_send.contiguous()
        self._keepalive.append(t)
        self._ops.append(dist.P2POp(dist.isend, t, self.send_rank))
        self._ops.append(dist.P2POp(dist.irecv, out, self.recv_rank))
        if VERBOSE:
            print(f"[cp {self.msg}] rank {dist.get_rank()} -> {self.send_rank}, <- {self.recv_rank}: "
                  f"{tuple(t.shape)} {t.dtype}", flush=True)
        return out

    def commit(self) -> None:
        assert self._reqs is None, "commit called twice without wait"
        self._reqs = dist.batch_isend_irecv(self._ops) if self._ops else []

    def wait(self) -> None:
        assert self._reqs is not None, "wait called before commit"
        for r in self._reqs:
            r.wait()
        self._reqs = None
        self._ops = []
        self._keepalive = []
