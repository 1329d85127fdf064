"""Autograd-aware collectives of Megatron-style tensor parallelism.

Same operators as picotron/tensor_parallel/tp_communications.py:23-192 — the conjugate pair
``f`` (identity forward / all-reduce backward) and ``g`` (all-reduce forward / identity
backward), the last-dim gather, a linear whose input-gradient all-reduce overlaps the weight
gradient, and the vocabulary-parallel cross entropy — but every op takes its process group as an
argument (default: the TP group of the global manager) instead of reading a global in
``forward``, and the gathers use the single-buffer collectives.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..ops import cross_entropy as ce_ops
from ..ops import gemm as gemm_ops
from .dist_utils import all_gather_cat, group_rank, group_size


def merge_first_two_dims(grad_output: torch.Tensor, input_: torch.Tensor):
    """Both tensors as 2-D ``[b*s, ...]`` views (tp_communications.py:8-10 of the reference)."""
    return grad_output.contiguous().flatten(0, 1), input_.contiguous().flatten(0, 1)


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int):
    """``num_partitions`` equal slices of the last dimension (tp_communications.py:13-20 of the reference)."""
    width = tensor.shape[-1]
    assert width % num_partitions == 0, f"{width} is not divisible by {num_partitions}"
    return tensor.split(width // num_partitions, dim=-1)


def _tp_group(group=None):
    return group if group is not None else pgm.get_pgm().tp_group


class CopyToModelParallelRegion(torch.autograd.Function):
    """f: identity in forward, all-reduce of the gradient in backward."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = _tp_group(group)
        return x

    @staticmethod
    def backward(ctx, grad):
        if group_size(ctx.group) > 1:
            grad = grad.contiguous()
            dist.all_reduce(grad, group=ctx.group)
        return grad, None


class ReduceFromModelParallelRegion(torch.autograd.Function):
    """g: all-reduce in forward, identity in backward."""

    @staticmethod
    def forward(ctx, x, group=None):
        group = _tp_group(group)
        if group_size(group) > 1:
            x = x.contiguous()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class GatherFromModelParallelRegion(torch.autograd.Function):
    """All-gather along the last dimension; backward keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = _tp_group(group)
        return all_gather_cat(x, x.dim() - 1, ctx.group)

    @staticmethod
    def backward(ctx, grad):
        n = group_size(ctx.group)
        if n == 1:
            return grad, None
        return grad.chunk(n, dim=-1)[group_rank(ctx.group)].contiguous(), None


class LinearWithAsyncAllReduce(torch.autograd.Function):
    """y = x @ w.T whose backward starts the all-reduce of dX, computes dW while it is in
    flight, and only then waits (picotron/tensor_parallel/tp_communications.py:84-115)."""

    @staticmethod
    def forward(ctx, x, w, group=None):
        ctx.group = _tp_group(group)
        ctx.save_for_backward(x, w)
        if gemm_ops.use_kernels(x, w):
            return gemm_ops.gemm_nt(x.reshape(-1, x.shape[-1]).contiguous(), w).view(*x.shape[:-1], w.shape[0])
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        if gemm_ops.use_kernels(dy2, w):
            dx = gemm_ops.gemm_nn(dy2.contiguous(), w).view(x.shape)
        else:
            dx = dy.matmul(w)
        handle = None
        if group_size(ctx.group) > 1:
            handle = dist.all_reduce(dx, group=ctx.group, async_op=True)
        if gemm_ops.use_kernels(dy2, w):
            dw = gemm_ops.wgrad_into(w, dy2.contiguous(), x2.contiguous())
        else:
            dw = dy2.t().matmul(x2)
        if handle is not None:
            handle.wait()
        return dx, dw, None


def linear_with_all_reduce(x, weight, bias=None, group=None):
    """Plain tensor-parallel column linear: f(x) @ weight.T (``bias`` must be None, as in every layer)."""
    assert bias is None, "bias is not supported"
    return gemm_ops.linear(CopyToModelParallelRegion.apply(x, group), weight)


def linear_with_async_all_reduce(x, weight, bias=None, group=None):
    assert bias is None, "bias is not supported"
    return LinearWithAsyncAllReduce.apply(x, weight, group)


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor, target: torch.Tensor, group=None) -> torch.Tensor:
    """Per-token loss from vocabulary-sharded logits ``[..., V/tp]``; rank r owns columns
    ``[r*V/tp, (r+1)*V/tp)``. Callers take the mean. (tp_communications.py:137-192)"""
    logits, targets = vocab_parallel_logits, target
    group = _tp_group(group)
    v_local = logits.shape[-1]
    start = group_rank(group) * v_local
    return ce_ops.cross_entropy(logits, targets, vocab_start=start, group=group)
