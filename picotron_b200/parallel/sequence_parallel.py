"""Megatron sequence parallelism over the tensor-parallel group.

Between tensor-parallel blocks the activations ``[b, s, h]`` are sharded along the sequence
(dim 1). A column-parallel linear all-gathers its input, a row-parallel linear reduce-scatters
its output; the backward passes are the conjugates. The column linear keeps only the *sharded*
input for the backward and gathers it again there, like
picotron/sequence_parallel/sequence_parallel.py:20-55, so activation memory shrinks by the TP
degree.

Operators: ``GatherFromSequenceParallelRegion`` (AG fwd / RS bwd),
``ReduceScatterToSequenceParallelRegion`` (RS fwd / AG bwd),
``column_linear_sequence_parallel`` (one gather feeding several weight matrices — q/k/v or
gate/up — where the reference gathers once per projection).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..ops import gemm as gemm_ops
from .dist_utils import all_gather_cat, group_size, reduce_scatter_dim

SEQ_DIM = 1


def _tp_group(group=None):
    return group if group is not None else pgm.get_pgm().tp_group


def all_gather_along_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """[b, s/tp, h] -> [b, s, h] (picotron/sequence_parallel/sp_communications.py:27-35)."""
    return all_gather_cat(x, SEQ_DIM, _tp_group(group))


def reduce_scatter_along_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """[b, s, h] summed over ranks -> this rank's [b, s/tp, h] (sp_communications.py:38-47)."""
    return reduce_scatter_dim(x, SEQ_DIM, _tp_group(group))


class GatherFromSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = _tp_group(group)
        return all_gather_along_seq(x, ctx.group)

    @staticmethod
    def backward(ctx, grad):
        return reduce_scatter_along_seq(grad, ctx.group), None


class ReduceScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = _tp_group(group)
        return reduce_scatter_along_seq(x, ctx.group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather_along_seq(grad, ctx.group), None


class ScatterToSequenceParallelRegion(torch.autograd.Function):
    """Keep this rank's sequence chunk of a replicated tensor; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = _tp_group(group)
        n = group_size(ctx.group)
        if n == 1:
            return x
        return x.chunk(n, dim=SEQ_DIM)[dist.get_rank(ctx.group)].contiguous()

    @staticmethod
    def backward(ctx, grad):
        return all_gather_along_seq(grad, ctx.group), None


class _ColumnLinearSP(torch.autograd.Function):
    """y = gather(x) @ cat(weights).T; saves the sharded x, re-gathers it in backward and
    reduce-scatters the input gradient."""

    @staticmethod
    def forward(ctx, x, group, ws, *params):
        ctx.group, ctx.ws = group, ws
        ctx.save_for_backward(x)
        xg = all_gather_along_seq(x, group)
        ctx.use_k = gemm_ops.use_kernels(xg, params[0])
        if ctx.use_k:
            x2 = xg.reshape(-1, xg.shape[-1])
            return gemm_ops.project_all(x2, ws).view(*xg.shape[:-1], ws.out_features)
        return torch.cat([torch.nn.functional.linear(xg, w) for w in params], dim=-1)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        ws = ctx.ws
        xg = all_gather_along_seq(x, ctx.group)
        x2 = xg.reshape(-1, xg.shape[-1])
        dy2 = dy.reshape(-1, dy.shape[-1])
        if ctx.use_k:
            if dy2.stride(-1) != 1:
                dy2 = dy2.contiguous()
            dx, grads = gemm_ops.backward_all(dy2, x2, ws)
        else:
            wcat = torch.cat(list(ws.params), dim=0)
            dx = dy2.matmul(wcat)
            grads = list(dy2.t().matmul(x2).split(ws.splits, dim=0))
        dx = reduce_scatter_along_seq(dx.view(xg.shape), ctx.group)
        return (dx, None, None, *grads)


def column_linear_sequence_parallel(x: torch.Tensor, mods, group=None) -> torch.Tensor:
    """One sequence gather feeding every projection in ``mods``; returns the concatenated
    outputs ``[b, s, sum(out_i)]``."""
    ws = gemm_ops.WeightSet.of(mods)
    return _ColumnLinearSP.apply(x, _tp_group(group), ws, *ws.params)


def column_parallel_linear_sp(x: torch.Tensor, weight: torch.Tensor, bias=None, group=None) -> torch.Tensor:
    """The reference's functional entry point (picotron/sequence_parallel/sequence_parallel.py:54-55):
    one column-parallel projection of a sequence shard, ``gather(x) @ weight.T``. Bias is not supported
    by any layer of the model (the reference's layers pass None as well)."""
    assert bias is None, "bias is not supported"
    ws = gemm_ops.WeightSet([weight])
    return _ColumnLinearSP.apply(x, _tp_group(group), ws, weight)
