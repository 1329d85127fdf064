"""Mixture-of-experts routing ops: router (softmax + bias + top-k + renormalisation + counts), slot
assignment inside the experts' queues, and the router-weighted combine of the experts' outputs.

Each op has the kernel form (``csrc/elementwise/moe_route.cu``; bf16 CUDA tensors) and a plain PyTorch
restatement (any device; the oracle of the kernel tests). On the kernel path nothing is read back to
the host and every tensor has a static shape, so a layer built from these ops can be captured in a
CUDA graph.

Reference: picotron/expert_parallel/expert_parallel.py:168-187 (router), :189-212 (counts for the
balancing terms), :219-224 (weight x sum over k); capacity_moe.py:44-57 (slot assignment).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import count_launch, ext, use_kernels


# ------------------------------------------------------------------------------------------ router
def route_ref(logits: torch.Tensor, bias, top_k: int, renorm: bool):
    """(probs fp32 [T, E], idx int64 [T, k], weights fp32 [T, k], counts int64 [E])."""
    probs = F.softmax(logits.float(), dim=-1)
    scores = probs + bias.to(probs.dtype) if bias is not None else probs
    idx = torch.topk(scores, top_k, dim=-1).indices
    w = probs.gather(-1, idx)
    if renorm and top_k > 1:
        w = w / w.sum(dim=-1, keepdim=True)
    counts = torch.zeros(logits.shape[-1], dtype=torch.int64, device=logits.device).scatter_add_(
        0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.int64, device=logits.device))
    return probs, idx, w, counts


class _RouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, renorm):
        T, E = logits.shape
        probs = torch.empty((T, E), device=logits.device, dtype=torch.float32)
        idx = torch.empty((T, top_k), device=logits.device, dtype=torch.int32)
        w = torch.empty((T, top_k), device=logits.device, dtype=torch.float32)
        counts = torch.zeros(E, device=logits.device, dtype=torch.int32)
        ext().moe_route(logits, bias, probs, idx, w, counts, top_k, renorm)
        count_launch()
        ctx.save_for_backward(probs, idx, w)
        ctx.top_k, ctx.renorm, ctx.dtype = top_k, renorm, logits.dtype
        ctx.mark_non_differentiable(idx, counts)
        return probs, idx, w, counts

    @staticmethod
    def backward(ctx, dprobs, _didx, dw, _dcounts):
        probs, idx, w = ctx.saved_tensors
        T, E = probs.shape
        if dw is None:
            dw = torch.zeros_like(w)
        dlogits = torch.empty((T, E), device=probs.device, dtype=torch.float32)
        dp = dprobs.contiguous().float() if dprobs is not None else None
        ext().moe_route_bwd(probs, idx, w, dw.contiguous().float(), dp, dlogits, ctx.top_k, ctx.renorm)
        count_launch()
        return dlogits.to(ctx.dtype), None, None, None


def route(logits: torch.Tensor, bias, top_k: int, renorm: bool):
    """Router of a mixture-of-experts layer on ``logits`` [T, E]: returns (probs fp32 [T, E], expert
    indices [T, k], weights fp32 [T, k], rows per expert [E]). The probabilities and the weights are
    differentiable w.r.t. the logits; the selection uses ``probs + bias`` (loss-free balancing), the
    weights the un-biased probabilities."""
    if use_kernels(logits) and logits.dim() == 2 and logits.shape[1] <= 256 and top_k <= 8 and logits.stride(1) == 1:
        b = bias.float().contiguous() if bias is not None else None
        return _RouteFn.apply(logits, b, top_k, bool(renorm))
    return route_ref(logits, bias, top_k, renorm)


# ------------------------------------------------------------------------------------ slot assignment
def slots_ref(expert_idx: torch.Tensor, num_experts: int, capacity: int = 0):
    """(pos [R], row_of_slot [E*C] or None): position of each routed row in its expert's queue (row
    order) and, for ``capacity`` > 0, the row that occupies every (expert, slot) pair (-1 = empty)."""
    flat = expert_idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.zeros(num_experts, dtype=torch.int64, device=flat.device).scatter_add_(
        0, flat, torch.ones_like(flat))
    starts = torch.cumsum(counts, 0) - counts
    pos_sorted = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
    pos = torch.empty_like(pos_sorted)
    pos[order] = pos_sorted
    table = None
    if capacity > 0:
        table = torch.full((num_experts * capacity + 1,), -1, dtype=torch.int32, device=flat.device)
        where = torch.where(pos < capacity, flat * capacity + pos, torch.full_like(pos, num_experts * capacity))
        table.scatter_(0, where, torch.arange(flat.numel(), device=flat.device, dtype=torch.int32))
        table = table[:num_experts * capacity]
    return pos, table


def slots(expert_idx: torch.Tensor, num_experts: int, capacity: int = 0):
    if expert_idx.is_cuda and expert_idx.dtype == torch.int32 and expert_idx.is_contiguous():
        flat = expert_idx.reshape(-1)
        pos = torch.empty_like(flat)
        table = torch.full((num_experts * capacity,), -1, dtype=torch.int32, device=flat.device) if capacity > 0 \
            else None
        ext().moe_slots(flat, num_experts, capacity, pos, table)
        count_launch()
        return pos, table
    return slots_ref(expert_idx, num_experts, capacity)


# -------------------------------------------------------------------------------------------- combine
def combine_ref(out: torch.Tensor, idx: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, capacity: int):
    """y [T, d] = sum_j [pos < C] w[t, j] * out[idx[t, j] * C + pos[t, j]]."""
    T, k = idx.shape
    fits = pos.view(T, k) < capacity
    rows = (idx.long() * capacity + pos.view(T, k).long()).clamp(max=out.shape[0] - 1)
    picked = out[rows.reshape(-1)].view(T, k, -1).float() * w.view(T, k, 1).float()
    return torch.where(fits.unsqueeze(-1), picked, torch.zeros_like(picked)).sum(dim=1).to(out.dtype)


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, out, idx, pos, w, row_of_slot, capacity):
        T, k = idx.shape
        d = out.shape[-1]
        y = torch.empty((T, d), device=out.device, dtype=out.dtype)
        ext().moe_combine(out, idx, pos, w, y, k, capacity)
        count_launch()
        ctx.save_for_backward(out, row_of_slot, w)
        ctx.k = k
        return y

    @staticmethod
    def backward(ctx, dy):
        out, row_of_slot, w = ctx.saved_tensors
        dout = torch.empty_like(out)
        dw = torch.zeros_like(w)
        ext().moe_combine_bwd(dy.contiguous(), out, row_of_slot, w, dout, dw, ctx.k)
        count_launch()
        return dout, None, None, dw, None, None


def combine(out: torch.Tensor, idx: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, row_of_slot: torch.Tensor,
            capacity: int) -> torch.Tensor:
    """Router-weighted sum of the experts' outputs per token. ``out`` [E*C, d] is indexed by (expert,
    slot); ``row_of_slot`` is the table ``slots`` built for the same routing (used by the backward
    pass: every slot has exactly one reader)."""
    if use_kernels(out) and out.is_contiguous() and out.shape[-1] % 8 == 0 and idx.dtype == torch.int32 \
            and pos.dtype == torch.int32 and w.dtype == torch.float32 and idx.shape[1] <= 8:
        return _CombineFn.apply(out, idx.contiguous(), pos.contiguous(), w.contiguous(), row_of_slot, capacity)
    return combine_ref(out, idx, pos, w, capacity)
