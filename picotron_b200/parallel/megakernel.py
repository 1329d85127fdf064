"""Functional entry points of the reference's grouped-expert module
(picotron/expert_parallel/megakernel.py:294-410) for scripts that call them directly.

``x_sorted`` is ``[N, H]`` with rows grouped by expert, ``counts`` ``[E]`` rows per expert, ``gate_w`` /
``up_w`` ``[E, I, H]``, ``down_w`` ``[E, H, I]``; the result is ``down(silu(gate(x)) * up(x))`` per expert,
optionally scaled per row. ``MoELayer`` itself does not come through here: it keeps its experts'
weights stacked and runs them as two grouped tcgen05 GEMM launches around one SwiGLU kernel
(``MoELayer._experts_on_layout``, ``ops/grouped_gemm.py``). These functions serve the same arithmetic on
loose weight tensors as one small matmul chain per expert (the library GEMM of PyTorch), which is enough for
the scripts and tests that call them; the fast path is the layer's.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F


def cuda_available() -> bool:
    """True on a CUDA device with this library's extension built (the reference's callers use the answer to
    choose their GPU path)."""
    if not torch.cuda.is_available():
        return False
    try:
        from ..ops import ext
        ext()
        return True
    except Exception:  # noqa: BLE001  extension missing: the torch path serves the call
        return False


def _counts_list(counts) -> List[int]:
    return [int(c) for c in (counts.tolist() if torch.is_tensor(counts) else counts)]


def torch_fused_ffn(x_sorted, counts, gate_w, up_w, down_w, row_weight):
    """Plain PyTorch restatement, differentiable: one SwiGLU feed-forward per expert segment."""
    pieces, lo = [], 0
    for e, n in enumerate(_counts_list(counts)):
        seg = x_sorted[lo:lo + n]
        pieces.append(F.linear(F.silu(F.linear(seg, gate_w[e])) * F.linear(seg, up_w[e]), down_w[e]))
        lo += n
    y = torch.cat(pieces, dim=0) if pieces else x_sorted.new_empty((0, x_sorted.shape[1]))
    return y if row_weight is None else y * row_weight.unsqueeze(-1)


def fused_moe(x_sorted, counts, gate_w, up_w, down_w, row_weight=None):
    """Differentiable grouped SwiGLU feed-forward (the reference's ``fused_moe``, megakernel.py:403-405)."""
    return torch_fused_ffn(x_sorted, counts, gate_w, up_w, down_w, row_weight)


def fused_moe_forward(x_sorted, counts, gate_w, up_w, down_w, row_weight=None):
    """Forward only (no autograd graph), like megakernel.py:294-305 of the reference."""
    with torch.no_grad():
        return fused_moe(x_sorted, counts, gate_w, up_w, down_w, row_weight)


def torch_moe_backward(x_sorted, counts, gate_w, up_w, down_w, dy):
    """``(dx, dgate_w, dup_w, ddown_w)`` by autograd over the PyTorch restatement."""
    with torch.enable_grad():
        leaves = [t.detach().requires_grad_(True) for t in (x_sorted, gate_w, up_w, down_w)]
        y = torch_fused_ffn(leaves[0], counts, leaves[1], leaves[2], leaves[3], None)
        return torch.autograd.grad(y, leaves, dy)


def fused_moe_backward(x_sorted, counts, gate_w, up_w, down_w, dy):
    """``(dx, dgate_w, dup_w, ddown_w)`` of the un-weighted feed-forward for the output gradient ``dy``."""
    with torch.enable_grad():
        leaves = [t.detach().requires_grad_(True) for t in (x_sorted, gate_w, up_w, down_w)]
        y = fused_moe(leaves[0], counts, leaves[1], leaves[2], leaves[3], None)
        return torch.autograd.grad(y, leaves, dy)


def fused_moe_dgrad(x_sorted, counts, gate_w, up_w, down_w, dy):
    """Input gradient with the intermediates the weight gradients need: ``(dx, a, d_inter13)`` where
    ``a = silu(gate(x)) * up(x)`` and ``d_inter13 = [d gate(x) | d up(x)]`` (megakernel.py:332-347)."""
    dxs, acts, dinters, lo = [], [], [], 0
    for e, n in enumerate(_counts_list(counts)):
        seg, dseg = x_sorted[lo:lo + n], dy[lo:lo + n]
        g, u = F.linear(seg, gate_w[e]), F.linear(seg, up_w[e])
        sig = torch.sigmoid(g)
        acts.append(g * sig * u)
        da = dseg @ down_w[e]                                   # [n, I]
        dg = da * u * sig * (1 + g * (1 - sig))                 # d silu(g) = sig * (1 + g * (1 - sig))
        du = da * g * sig
        dinters.append(torch.cat([dg, du], dim=-1))
        dxs.append(dg @ gate_w[e] + du @ up_w[e])
        lo += n
    cat = lambda parts, width: torch.cat(parts) if parts else x_sorted.new_empty((0, width))    # noqa: E731
    inter = gate_w.shape[1]
    return cat(dxs, x_sorted.shape[1]), cat(acts, inter), cat(dinters, 2 * inter)


def fused_moe_wgrad(x_sorted, counts, a, d_inter13, dy):
    """Weight gradients ``(dgate_w, dup_w, ddown_w)`` from the intermediates of ``fused_moe_dgrad``
    (megakernel.py:350-357)."""
    inter = a.shape[1]
    dg, du, dd, lo = [], [], [], 0
    for n in _counts_list(counts):
        seg = slice(lo, lo + n)
        dd.append(dy[seg].T @ a[seg])                            # [H, I]
        d13 = d_inter13[seg].T @ x_sorted[seg]                   # [2I, H]
        dg.append(d13[:inter])
        du.append(d13[inter:])
        lo += n
    return torch.stack(dg), torch.stack(du), torch.stack(dd)
