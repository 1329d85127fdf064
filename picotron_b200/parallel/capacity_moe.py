"""Fixed-capacity expert dispatch: every (rank, expert) pair handles exactly ``C`` rows per
round, so every buffer of the MoE layer has a static shape whatever the router does
(GShard / Switch style; behaviour of picotron/expert_parallel/capacity_moe.py:33-173).

* ``C = max(1, int(factor * T * k / E + 0.999))``
* a routed row's slot is its position in its expert's queue (row order); rows with slot >= C
  are dropped (``dropless=False``) or handled in later rounds (``dropless=True``): the number of
  rounds is ``ceil(max_count / C)`` capped by ``max_rounds`` and maximised over the EP group so all
  ranks issue the same collectives, empty rounds included
* the exchange is an equal-split all-to-all of ``L*C`` rows per peer; received rows are viewed
  ``[L, ep*C, d]`` and each expert runs on its fixed batch (padding rows are zero and a bias-free
  SwiGLU maps zero to zero)
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ep_communications as epc


def compute_capacity(num_tokens: int, top_k: int, num_experts: int, capacity_factor: float) -> int:
    return max(1, int(capacity_factor * num_tokens * top_k / num_experts + 0.999))


def expert_counts(expert_idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Rows per expert (int64). ``scatter_add`` instead of ``bincount``: the latter reads the maximum
    back to the host on CUDA, which stalls the stream and cannot be captured in a CUDA graph."""
    return torch.zeros(num_experts, dtype=torch.int64, device=expert_idx.device).scatter_add_(
        0, expert_idx, torch.ones_like(expert_idx, dtype=torch.int64))


def slot_assignment(expert_idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """slot[i] = number of earlier rows routed to the same expert as row i."""
    order = torch.argsort(expert_idx, stable=True)
    counts = expert_counts(expert_idx, num_experts)
    starts = torch.cumsum(counts, 0) - counts
    sorted_expert = expert_idx[order]
    pos = torch.arange(order.numel(), device=expert_idx.device) - starts[sorted_expert]
    slot = torch.empty_like(pos)
    slot[order] = pos
    return slot


def _capacity_moe_fused(layer, epf, tokens, expert_idx, weights, token_idx, num_tokens, slot, rounds):
    """Same computation with the exchanges done by the peer-memory kernels of ``ops.fused_ep``: rows
    are gathered from the tokens and (optionally) quantised while they are being sent, and arrive
    grouped by local expert; the outputs come back indexed by (expert, slot)."""
    from ..ops import fused_ep
    E, L, ep, C, d = layer.num_experts, layer.num_local_experts, layer.ep_world_size, epf.C, epf.d
    R = expert_idx.numel()
    y = torch.zeros((num_tokens, d), device=tokens.device, dtype=torch.float32)
    rows = torch.arange(R, device=tokens.device, dtype=torch.int32)
    for r in range(rounds):
        # no boolean-mask indexing or nonzero(): those read sizes back to the host. Rows outside this
        # round are routed to a spare table entry (index E*C) on the way out and weighted by zero on
        # the way back, so every tensor keeps a static shape.
        in_round = (slot >= r * C) & (slot < (r + 1) * C)
        idx = torch.where(in_round, expert_idx * C + (slot - r * C), torch.full_like(slot, E * C))
        row_of_slot = torch.full((E * C + 1,), -1, device=tokens.device, dtype=torch.int32)
        row_of_slot.scatter_(0, idx, rows)
        x = fused_ep.dispatch(tokens, row_of_slot[:E * C], layer.top_k, epf, bool(layer.ep_fp8_dispatch))  # [L, ep*C, d]
        out = layer.experts_uniform(x)
        back = fused_ep.combine(out, epf)                                                           # [E*C, d]
        contrib = back[idx.clamp(max=E * C - 1)].float() * weights.float().unsqueeze(-1)
        y = y.index_add(0, token_idx, torch.where(in_round.unsqueeze(-1), contrib, torch.zeros_like(contrib)))
    dropped = (slot >= rounds * C).float().mean()
    return y.to(tokens.dtype), dropped


def capacity_moe(layer, routed, expert_idx, weights, token_idx, num_tokens: int, capacity: int, dropless: bool,
                 max_rounds: int, tokens=None):
    """Returns (y [T, d] gate-weighted and summed per token, fraction of routed rows dropped)."""
    E, L, ep, d = layer.num_experts, layer.num_local_experts, layer.ep_world_size, routed.shape[1]
    C = capacity
    slot = slot_assignment(expert_idx, E)
    rounds = 1
    if dropless:
        max_count = expert_counts(expert_idx, E).max()
        need = torch.clamp((max_count + C - 1) // C, min=1, max=max_rounds).to(torch.int64)
        if ep > 1:
            dist.all_reduce(need, op=dist.ReduceOp.MAX, group=layer.ep_group)
        rounds = int(need.item())
    y = torch.zeros((num_tokens, d), device=routed.device, dtype=routed.dtype)
    equal = [L * C] * ep
    epf = getattr(layer, "fused_ep", None)
    if epf is not None and routed.is_cuda and routed.dtype == torch.bfloat16 and ep > 1 and tokens is not None \
            and epf.C == C:
        return _capacity_moe_fused(layer, epf, tokens, expert_idx, weights, token_idx, num_tokens, slot, rounds)
    for r in range(rounds):
        sel = torch.nonzero((slot >= r * C) & (slot < (r + 1) * C)).squeeze(1)
        idx = expert_idx[sel] * C + (slot[sel] - r * C)
        buf = torch.zeros((E * C, d), device=routed.device, dtype=routed.dtype).index_add(0, idx, routed[sel])
        if ep > 1:
            if layer.ep_fp8_dispatch:
                recv = epc.all_to_all_fp8(buf, equal, equal, layer.ep_group, layer.ep_fp8_granularity)
            else:
                recv = epc.all_to_all(buf, equal, equal, layer.ep_group)
        else:
            recv = buf
        x = recv.view(ep, L, C, d).transpose(0, 1).reshape(L, ep * C, d)
        out = layer.experts_uniform(x)
        back = out.view(L, ep, C, d).transpose(0, 1).reshape(ep * L * C, d)
        if ep > 1:
            back = epc.all_to_all(back, equal, equal, layer.ep_group)
        y = y.index_add(0, token_idx[sel], back[idx] * weights[sel].unsqueeze(-1))
    dropped = (slot >= rounds * C).float().mean()
    return y, dropped
