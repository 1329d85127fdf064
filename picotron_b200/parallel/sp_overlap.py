"""Chunked communication/compute overlap for sequence parallelism (MegaScale-style).

``ring_all_gather_linear``: instead of gathering the whole sequence and then multiplying, the
local shard is multiplied while the next shard travels around a ring of point-to-point
transfers; after ``tp`` steps every rank has produced the rows of all shards
(picotron/sequence_parallel/overlap.py:40-76).

``linear_pipelined_reduce_scatter``: the output is produced one destination chunk at a time and
each chunk's reduction towards its owner starts while the next chunk is being multiplied
(overlap.py:79-118); an optional ``addend`` (the MLP partial sum of a parallel block) is folded
into the same reduction.

Backward passes use the plain collectives, like the reference (overlap.py:121-183).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..ops import gemm as gemm_ops
from .dist_utils import group_rank, group_size
from .sequence_parallel import all_gather_along_seq, reduce_scatter_along_seq


def ring_all_gather_matmul(x_shard: torch.Tensor, weight, group=None) -> torch.Tensor:
    """[b, s/tp, in] -> [b, s, sum(out)] with the ring transfer of shard i+1 overlapping the
    matmul of shard i. ``weight``: one ``[out, in]`` tensor (the reference's call, overlap.py:40 there)
    or a list of them sharing the input."""
    weights = [weight] if torch.is_tensor(weight) else list(weight)
    group = group if group is not None else pgm.get_pgm().tp_group
    n = group_size(group)
    rank = group_rank(group)
    b, s_loc, _ = x_shard.shape
    out_dim = sum(w.shape[0] for w in weights)
    out = torch.empty((b, s_loc * n, out_dim), device=x_shard.device, dtype=x_shard.dtype)
    cur = x_shard.contiguous()
    nxt = torch.empty_like(cur)
    send_to = dist.get_global_rank(group, (rank + 1) % n)
    recv_from = dist.get_global_rank(group, (rank - 1) % n)
    for step in range(n):
        reqs = []
        if step < n - 1:
            ops = [dist.P2POp(dist.isend, cur, send_to, group), dist.P2POp(dist.irecv, nxt, recv_from, group)]
            reqs = dist.batch_isend_irecv(ops)
        owner = (rank - step) % n  # whose shard is in hand
        col = 0
        with torch.no_grad():
            for w in weights:
                out[:, owner * s_loc:(owner + 1) * s_loc, col:col + w.shape[0]] = \
                    gemm_ops.linear(cur.detach(), w.detach())
                col += w.shape[0]
        for r in reqs:
            r.wait()
        if step < n - 1:
            cur, nxt = nxt, cur
    return out


def pipelined_matmul_reduce_scatter(x_full: torch.Tensor, weight: torch.Tensor, addend_full=None, group=None):
    """x_full [b, s, in/tp] @ weight.T summed over ranks, sequence-scattered: chunk i is reduced to
    rank i while chunk i+1 is being multiplied. Returns this rank's [b, s/tp, out]."""
    group = group if group is not None else pgm.get_pgm().tp_group
    n = group_size(group)
    rank = group_rank(group)
    b, s, _ = x_full.shape
    s_loc = s // n
    handles, partials = [], []
    with torch.no_grad():
        for i in range(n):
            chunk = gemm_ops.linear(x_full[:, i * s_loc:(i + 1) * s_loc].detach(), weight.detach())
            if addend_full is not None:
                chunk = chunk + addend_full[:, i * s_loc:(i + 1) * s_loc].detach()
            chunk = chunk.contiguous()
            partials.append(chunk)
            handles.append(dist.reduce(chunk, dst=dist.get_global_rank(group, i), group=group, async_op=True))
        for h in handles:
            h.wait()
    return partials[rank]


class _RingAllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, n_w, *weights):
        ctx.group = group
        ctx.save_for_backward(x, *weights)
        return ring_all_gather_matmul(x, list(weights), group)

    @staticmethod
    def backward(ctx, dy):
        x, *weights = ctx.saved_tensors
        xg = all_gather_along_seq(x, ctx.group)
        x2 = xg.reshape(-1, xg.shape[-1])
        dy2 = dy.reshape(-1, dy.shape[-1])
        wcat = torch.cat(list(weights), dim=0)
        dx = reduce_scatter_along_seq(dy2.matmul(wcat).view(xg.shape), ctx.group)
        dws = dy2.t().matmul(x2).split([w.shape[0] for w in weights], dim=0)
        return (dx, None, None, *dws)


class _LinearPipelinedReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, addend):
        ctx.group = group
        ctx.has_addend = addend is not None
        ctx.save_for_backward(x, weight)
        return pipelined_matmul_reduce_scatter(x, weight, addend, group)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dyg = all_gather_along_seq(dy.contiguous(), ctx.group)
        dy2 = dyg.reshape(-1, dyg.shape[-1])
        dx = dy2.matmul(weight).view(x.shape)
        dw = dy2.t().matmul(x.reshape(-1, x.shape[-1]))
        return dx, dw, None, (dyg if ctx.has_addend else None)


def ring_all_gather_linear(x, mods, group) -> torch.Tensor:
    """Sequence-parallel column projections with the gather overlapped; returns [b, s, sum(out_i)]."""
    weights = [m.weight for m in mods]
    return _RingAllGatherLinear.apply(x, group, len(weights), *weights)


def linear_pipelined_reduce_scatter(x, weight, group, addend=None):
    return _LinearPipelinedReduceScatter.apply(x, weight, group, addend)


# ------------------------------------------------------------------------------------------
# the reference's functional names (picotron/sequence_parallel/overlap.py:121-183)
# ------------------------------------------------------------------------------------------
def overlapped_column_parallel_linear_sp(x, weight, bias=None, group=None):
    """Column-parallel projection of a sequence shard with the all-gather overlapped chunk by chunk."""
    assert bias is None, "bias is not supported"
    group = group if group is not None else pgm.get_pgm().tp_group
    return _RingAllGatherLinear.apply(x, group, 1, weight)


def overlapped_row_parallel_linear_sp(x, weight, addend=None, group=None):
    """Row-parallel projection whose reduce-scatter is pipelined over sequence chunks; ``addend`` is a
    second full-sequence partial sum folded into the same reduction (parallel transformer block)."""
    group = group if group is not None else pgm.get_pgm().tp_group
    return _LinearPipelinedReduceScatter.apply(x, weight, group, addend)


class OverlappedColumnParallelLinearSP:
    """``.apply(x_shard, weight, bias)`` like the reference's autograd function of this name."""
    apply = staticmethod(overlapped_column_parallel_linear_sp)


class OverlappedRowParallelLinearSP:
    """``.apply(x_full, weight, addend)`` like the reference's autograd function of this name."""
    apply = staticmethod(overlapped_row_parallel_linear_sp)

