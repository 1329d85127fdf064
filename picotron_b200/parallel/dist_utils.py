"""Small helpers over ``torch.distributed`` that treat "no group" as a group of one."""
from __future__ import annotations

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


def all_reduce_(t: torch.Tensor, group, op=None, async_op: bool = False):
    if group_size(group) == 1:
        return None
    return dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group, async_op=async_op)


def all_gather_cat(t: torch.Tensor, dim: int, group) -> torch.Tensor:
    """Concatenate every rank's ``t`` along ``dim`` (rank order)."""
    n = group_size(group)
    if n == 1:
        return t
    t = t.contiguous()
    if t.dim() == 0:
        t = t.view(1)
    flat = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype)
    dist.all_gather_into_tensor(flat, t, group=group)
    if dim == 0:
        return flat
    out = flat.view((n,) + tuple(t.shape))
    # [n, d0, .., dim, ..] -> [d0, .., n*dim, ..]
    out = out.movedim(0, dim)  # [d0, .., n, dim, ..]
    shape = list(t.shape)
    shape[dim] = n * t.shape[dim]
    return out.reshape(shape)


def reduce_scatter_dim(t: torch.Tensor, dim: int, group) -> torch.Tensor:
    """Sum over ranks and keep this rank's chunk of ``dim``."""
    n = group_size(group)
    if n == 1:
        return t
    assert t.shape[dim] % n == 0
    if dim != 0:
        chunk = t.shape[dim] // n
        shape = list(t.shape)
        # [.., n*chunk, ..] -> [n, .., chunk, ..]
        t = t.reshape(shape[:dim] + [n, chunk] + shape[dim + 1:]).movedim(dim, 0)
    t = t.contiguous()
    if dim == 0:
        out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype)
        dist.reduce_scatter_tensor(out, t, group=group)
        return out
    out = torch.empty(tuple(t.shape[1:]), device=t.device, dtype=t.dtype)
    dist.reduce_scatter_tensor(out, t.view((n * t.shape[1],) + tuple(t.shape[2:])), group=group)
    return out
