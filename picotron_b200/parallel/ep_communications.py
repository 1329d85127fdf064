"""All-to-all primitives of expert parallelism (variable splits, autograd-aware).

* ``all_to_all(x, out_splits, in_splits, group)`` — rows exchange whose backward is the reverse
  exchange (picotron/expert_parallel/ep_communications.py:22-43)
* ``all_to_all_fp8`` — the same with the payload quantised to E4M3 (1x128 block scales by
  default, per-row scales for parity with ep_communications.py:59-118); the backward is a
  straight-through bf16 exchange of the gradients
* ``all_to_all_no_grad`` / ``*_async`` — metadata and pipelined variants
* ``exchange_counts`` — the ``[ep, L]`` table of rows per (destination rank, local expert); one
  small exchange replaces the reference's split-size exchange plus per-row expert-id exchange
  (ep_communications.py:55,177)
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..ops import quant
from .dist_utils import group_size


def _a2a(x: torch.Tensor, out_splits: List[int], in_splits: List[int], group, async_op: bool = False):
    out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    work = dist.all_to_all_single(out, x.contiguous(), output_split_sizes=list(out_splits),
                                  input_split_sizes=list(in_splits), group=group, async_op=async_op)
    return out, work


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        return _a2a(x, out_splits, in_splits, group)[0]

    @staticmethod
    def backward(ctx, grad):
        return _a2a(grad, ctx.in_splits, ctx.out_splits, ctx.group)[0], None, None, None


def all_to_all(x, output_split_sizes, input_split_sizes, group):
    if group_size(group) == 1:
        return x
    return _AllToAll.apply(x, output_split_sizes, input_split_sizes, group)


class _AllToAllAsync(torch.autograd.Function):
    """Variable-size all-to-all whose forward returns before the transfer has finished; the caller waits
    on the work handle that is put into ``box``. The backward pass is the opposite exchange, blocking."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group, box):
        ctx.group, ctx.out_splits, ctx.in_splits = group, list(out_splits), list(in_splits)
        out, work = _a2a(x, out_splits, in_splits, group, async_op=True)
        box.append(work)
        return out

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.in_splits, ctx.out_splits, ctx.group)[0], None, None, None, None


def all_to_all_async(x, output_split_sizes, input_split_sizes, group):
    """Differentiable all-to-all launched asynchronously: returns ``(output, work)``; ``work.wait()`` before
    the output is used (picotron/expert_parallel/ep_communications.py:155-159)."""
    box = []
    out = _AllToAllAsync.apply(x, output_split_sizes, input_split_sizes, group, box)
    return out, box[0]


def all_to_all_no_grad(x, output_split_sizes, input_split_sizes, group):
    if group_size(group) == 1:
        return x
    return _a2a(x, output_split_sizes, input_split_sizes, group)[0]


def all_to_all_no_grad_async(x, output_split_sizes, input_split_sizes, group):
    """Returns (output, work); the output is valid after ``work.wait()``."""
    return _a2a(x, output_split_sizes, input_split_sizes, group, async_op=True)


class _AllToAllFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group, granularity):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        payload, scales = quant.quantize_fp8(x, granularity)
        recv_payload = _a2a(payload, out_splits, in_splits, group)[0]
        recv_scales = _a2a(scales, out_splits, in_splits, group)[0]
        return quant.dequantize_fp8(recv_payload, recv_scales, x.dtype, granularity)

    @staticmethod
    def backward(ctx, grad):
        return _a2a(grad, ctx.in_splits, ctx.out_splits, ctx.group)[0], None, None, None, None


def all_to_all_fp8(x, output_split_sizes, input_split_sizes, group, granularity: str = "block"):
    """Dispatch with an FP8 payload; wire bytes per row: d + 4*ceil(d/128) (block) or d + 4 (row)."""
    if group_size(group) == 1:
        return x
    return _AllToAllFP8.apply(x, output_split_sizes, input_split_sizes, group, granularity)


def exchange_counts(send_counts: torch.Tensor, group) -> torch.Tensor:
    """send_counts[r, l] = rows this rank sends to local expert l of rank r. Returns
    recv_counts[s, l] = rows arriving from rank s for this rank's local expert l."""
    if group_size(group) == 1:
        return send_counts
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts.contiguous(), group=group)
    return recv


def exchange_split_sizes(input_split_sizes: torch.Tensor, group) -> torch.Tensor:
    """Per-rank row counts: what each peer will send me (ep_communications.py:170-178)."""
    return exchange_counts(input_split_sizes.view(-1, 1), group).view(-1)
