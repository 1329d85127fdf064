"""Point-to-point communication between pipeline stages (NCCL on GPUs, gloo on CPU).

``RoundCommunicator`` serves the schedule executor: all transfers of one schedule round are
posted as a single ``batch_isend_irecv`` group per rank (ops sorted by peer and message key so
both ends agree on the order); nothing blocks the host and nothing synchronises the device —
the consumer waits on the request of the message it needs right before using it, so transfers
overlap with the compute of other micro-batches. (The reference waits for each transfer and then
calls ``torch.cuda.synchronize()``, picotron/pipeline_parallel/pp_communications.py:40-47.)

``pipeline_communicate`` / ``bidirectional_pipeline_communicate`` keep the reference's blocking
helpers for callers that drive stages by hand (pp_communications.py:17-149).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm

VERBOSE = os.environ.get("VERBOSE", "0") == "1"
_STEP = 0


class RoundCommunicator:
    def __init__(self, device, dtype):
        self.device, self.dtype = device, dtype
        self.inbox: Dict[tuple, torch.Tensor] = {}
        self.requests: Dict[tuple, object] = {}
        self._send_keepalive: List = []
        self._pending_sends: List = []

    def post_round(self, messages, my_rank_in_pp: int, pp_group_ids: List[int], outgoing: Dict[tuple, torch.Tensor],
                   shape) -> None:
        """messages: the cross-rank messages produced in the current schedule round (``pp_schedules.Message``)."""
        ops, recv_keys = [], []
        mine = [m for m in messages if m.src_rank == my_rank_in_pp or m.dst_rank == my_rank_in_pp]
        mine.sort(key=lambda m: (m.dst_rank if m.src_rank == my_rank_in_pp else m.src_rank, m.kind, m.dst_stage, m.mb))
        for m in mine:
            if m.src_rank == my_rank_in_pp:
                t = outgoing.pop(m.key).contiguous()
                ops.append(dist.P2POp(dist.isend, t, pp_group_ids[m.dst_rank]))
                self._send_keepalive.append(t)
                recv_keys.append(None)
            else:
                buf = torch.empty(shape, device=self.device, dtype=self.dtype)
                self.inbox[m.key] = buf
                ops.append(dist.P2POp(dist.irecv, buf, pp_group_ids[m.src_rank]))
                recv_keys.append(m.key)
        if not ops:
            return
        if VERBOSE:
            global _STEP
            _STEP += 1
            print(f"[pp step {_STEP}] rank {dist.get_rank()}: " +
                  ", ".join(("send" if k is None else "recv") for k in recv_keys), flush=True)
        reqs = dist.batch_isend_irecv(ops)
        # NCCL returns one request for the whole group, gloo one per op
        per_op = len(reqs) == len(ops)
        for i, key in enumerate(recv_keys):
            if key is not None:
                self.requests[key] = reqs[i] if per_op else reqs[-1]
            elif per_op:
                self._pending_sends.append(reqs[i])
        if not per_op:
            self._pending_sends.extend(reqs)

    def take(self, key) -> torch.Tensor:
        req = self.requests.pop(key, None)
        if req is not None:
            req.wait()
        return self.inbox.pop(key)

    def finish(self) -> None:
        for r in self._pending_sends:
            r.wait()
        self._pending_sends = []
        self._send_keepalive.clear()
        assert not self.inbox, f"unconsumed pipeline messages: {list(self.inbox)}"


# ------------------------------------------------------------------------------------------
# blocking helpers with the reference's names
# ------------------------------------------------------------------------------------------
def _sync(device):
    if torch.device(device).type == "cuda":
        torch.cuda.current_stream().synchronize()


def pipeline_communicate(operation: str, device, dtype, tensor: Optional[torch.Tensor] = None, shapes=None):
    """``recv_forward`` / ``send_forward`` / ``recv_backward`` / ``send_backward`` between
    neighbouring stages; returns the received tensor (requires_grad) or None."""
    m = pgm.get_pgm()
    if operation == "recv_forward":
        if m.pp_is_first_stage:
            return None
        tensor = torch.empty(shapes, requires_grad=True, device=device, dtype=dtype)
        peer, fn = m.pp_prev_rank, dist.irecv
    elif operation == "send_forward":
        if m.pp_is_last_stage:
            return None
        peer, fn = m.pp_next_rank, dist.isend
    elif operation == "recv_backward":
        if m.pp_is_last_stage:
            return None
        tensor = torch.empty(shapes, requires_grad=True, device=device, dtype=dtype)
        peer, fn = m.pp_next_rank, dist.irecv
    elif operation == "send_backward":
        if m.pp_is_first_stage:
            return None
        peer, fn = m.pp_prev_rank, dist.isend
    else:
        raise ValueError(f"unknown operation {operation}")
    for req in dist.batch_isend_irecv([dist.P2POp(fn, tensor, peer)]):
        req.wait()
    _sync(device)
    return tensor if operation.startswith("recv") else None


def bidirectional_pipeline_communicate(operation: str, send_tensor: torch.Tensor, recv_shapes, device, dtype):
    """``send_fwd_recv_bwd`` / ``send_bwd_recv_fwd``: one batched send+recv with the same peer."""
    m = pgm.get_pgm()
    is_fwd = operation == "send_fwd_recv_bwd"
    if (is_fwd and m.pp_is_last_stage) or (not is_fwd and m.pp_is_first_stage):
        return None
    peer = m.pp_next_rank if is_fwd else m.pp_prev_rank
    recv = torch.empty(recv_shapes, requires_grad=True, device=device, dtype=dtype)
    for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, send_tensor, peer),
                                       dist.P2POp(dist.irecv, recv, peer)]):
        req.wait()
    _sync(device)
    return recv


def _post_and_wait(ops, device) -> None:
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        _sync(device)


def interleaved_pipeline_communicate(device, dtype, shapes, send_forward_tensor=None, send_backward_tensor=None,
                                     recv_forward=False, recv_backward=False):
    """Blocking ring exchange of the interleaved schedule as one batched group (the reference's helper of
    this name, pp_communications.py:53-94): activations go to the next rank of the pipeline ring, gradients
    to the previous one; returns ``(received activation or None, received gradient or None)``. Every rank
    posts its sends before its receives and forward before backward, so the two ends of a pair agree on
    the order even when next and previous rank are the same process (two stages)."""
    m = pgm.get_pgm()
    ring = m.pp_group_ids
    nxt, prv = ring[(m.pp_rank + 1) % len(ring)], ring[(m.pp_rank - 1) % len(ring)]
    got = {"forward": None, "backward": None}
    ops = [dist.P2POp(dist.isend, t, peer) for t, peer in ((send_forward_tensor, nxt), (send_backward_tensor, prv))
           if t is not None]
    for name, wanted, peer in (("forward", recv_forward, prv), ("backward", recv_backward, nxt)):
        if wanted:
            got[name] = torch.empty(shapes, requires_grad=True, device=device, dtype=dtype)
            ops.append(dist.P2POp(dist.irecv, got[name], peer))
    _post_and_wait(ops, device)
    return got["forward"], got["backward"]


def vshape_pipeline_communicate(device, dtype, shape, sends, recvs):
    """Blocking exchange with arbitrary pipeline peers in one batched group (the reference's helper for
    the V-shaped zero-bubble schedule, pp_communications.py:97-122). ``sends``: ``(key, tensor, peer
    pipeline rank)``; ``recvs``: ``(key, peer pipeline rank)``; returns ``{key: received tensor}``. Both lists
    are posted in (peer, key) order, which both ends of a pair derive identically."""
    ring = pgm.get_pgm().pp_group_ids
    ops = [dist.P2POp(dist.isend, t, ring[peer]) for _, t, peer in sorted(sends, key=lambda e: (e[2], e[0]))]
    received = {}
    for key, peer in sorted(recvs, key=lambda e: (e[1], e[0])):
        received[key] = torch.empty(shape, requires_grad=True, device=device, dtype=dtype)
        ops.append(dist.P2POp(dist.irecv, received[key], ring[peer]))
    _post_and_wait(ops, device)
    return received

