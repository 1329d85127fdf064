"""Grouped linear layers for the local experts of a mixture-of-experts layer.

The rows of the activation matrix are expert-contiguous, every expert's segment padded with zero
rows to a multiple of 128 (``GroupLayout``), so a 128-row output tile never mixes experts. One
launch of the tcgen05 GEMM (``csrc/gemm/gemm_bf16_sm100.cu``, grouped modes) then covers all local
experts:

* forward ``y[rows_e] = x[rows_e] @ W[e].T`` and input gradient ``dx[rows_e] = dy[rows_e] @ W[e]``
  pick the expert's matrix per row tile from a device array (no host synchronisation, no
  per-expert launches);
* weight gradient ``dW[e] (+)= dy[rows_e].T @ x[rows_e]`` reduces every expert's own row range and
  accumulates into the fp32 ``main_grad`` of the stacked weights.

The expert weights are one ``[E_local * out, in]`` block: the views of the per-expert parameters
stored back to back (``param_store``), so state dicts keep the reference's per-expert names.

Reference: picotron/expert_parallel/megakernel.py:40-102 (grouped GEMM over 64-row blocks),
:209-291 (grouped weight gradient), :294-357 (forward / dgrad / wgrad composition); the block
schedule there is built on the host from ``counts.tolist()`` (:116-129).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import count_launch, ext, use_kernels

TILE = 128


@dataclass
class GroupLayout:
    """Padded expert-major row layout: expert e owns rows [seg_start[e], seg_start[e+1])."""
    num_groups: int
    rows: int                         # total padded rows (multiple of 128)
    seg_start: torch.Tensor           # [G+1] int32, multiples of 128
    tile_group: torch.Tensor          # [rows/128] int32
    pad_index: Optional[torch.Tensor]  # [n] int64: padded row of every unpadded (expert-sorted) row; None = no padding

    @staticmethod
    def from_counts(counts: List[int], device) -> "GroupLayout":
        """Layout for expert-sorted rows with ``counts[e]`` rows of expert e (host integers)."""
        padded = [(c + TILE - 1) // TILE * TILE for c in counts]
        starts = [0]
        for p in padded:
            starts.append(starts[-1] + p)
        tiles = []
        for e, p in enumerate(padded):
            tiles += [e] * (p // TILE)
        seg = torch.tensor(starts, dtype=torch.int32, device=device)
        tg = torch.tensor(tiles if tiles else [0], dtype=torch.int32, device=device)
        pad_index = None
        if any(c != p for c, p in zip(counts, padded)):
            idx = [torch.arange(c, dtype=torch.int64) + starts[e] for e, c in enumerate(counts)]
            pad_index = torch.cat(idx).to(device) if idx else torch.zeros(0, dtype=torch.int64, device=device)
        return GroupLayout(len(counts), starts[-1], seg, tg, pad_index)

    @staticmethod
    def uniform(num_groups: int, rows_per_group: int, device) -> "GroupLayout":
        """Every expert has the same number of rows (fixed-capacity dispatch)."""
        return GroupLayout.from_counts([rows_per_group] * num_groups, device)

    def pad(self, x: torch.Tensor) -> torch.Tensor:
        if self.pad_index is None:
            return x
        out = x.new_zeros((self.rows, x.shape[1]))
        return out.index_copy(0, self.pad_index, x)

    def unpad(self, y: torch.Tensor) -> torch.Tensor:
        if self.pad_index is None:
            return y
        return y.index_select(0, self.pad_index)


def grouped_gemm_nt(x, w, layout: GroupLayout, out_rows: int):
    """y[P, out] with y[rows_e] = x[rows_e] @ w[e*out:(e+1)*out].T"""
    P, K = x.shape
    y = torch.empty((P, out_rows), device=x.device, dtype=torch.bfloat16)
    ext().gemm_grouped(x, w, y, P, out_rows, K, x.stride(0), w.stride(0), y.stride(0), False, False, 0,
                       0, layout.tile_group, layout.num_groups, out_rows)
    count_launch()
    return y


def grouped_gemm_nn(dy, w, layout: GroupLayout, out_rows: int):
    """dx[P, in] with dx[rows_e] = dy[rows_e] @ w[e*out:(e+1)*out]"""
    P = dy.shape[0]
    n_in = w.shape[1]
    dx = torch.empty((P, n_in), device=dy.device, dtype=torch.bfloat16)
    ext().gemm_grouped(dy, w, dx, P, n_in, out_rows, dy.stride(0), w.stride(0), dx.stride(0), False, True, 0,
                       0, layout.tile_group, layout.num_groups, out_rows)
    count_launch()
    return dx


def grouped_gemm_tn(dy, x, layout: GroupLayout, out: torch.Tensor, accumulate: bool):
    """out[e*M:(e+1)*M] (+)= dy[rows_e].T @ x[rows_e]; blocks of experts without rows are untouched."""
    P, M = dy.shape
    N = x.shape[1]
    if accumulate:
        assert out.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if out.dtype == torch.bfloat16 else 1
    ext().gemm_grouped(dy, x, out, M, N, P, dy.stride(0), x.stride(0), out.stride(0), True, True, mode,
                       1, layout.seg_start, layout.num_groups, 0)
    count_launch()
    return out


class _GroupedLinearFn(torch.autograd.Function):
    """``w`` is the stacked ``[G * out_rows, in]`` weight block. When it is the fused view of
    parameters that carry ``main_grad`` buffers, the weight gradient accumulates there and autograd
    sees none; the parameters are passed so the backward runs even if ``x`` needs no gradient."""

    @staticmethod
    def forward(ctx, x, w, layout, out_rows, main_grad, *params):
        ctx.save_for_backward(x, w)
        ctx.layout, ctx.out_rows, ctx.main_grad, ctx.params = layout, out_rows, main_grad, params
        return grouped_gemm_nt(x, w, layout, out_rows)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        layout, out_rows = ctx.layout, ctx.out_rows
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = grouped_gemm_nn(dy, w, layout, out_rows)
        if ctx.main_grad is not None:
            grouped_gemm_tn(dy, x, layout, ctx.main_grad, accumulate=True)
            for p in ctx.params:
                hook = getattr(p, "grad_ready_hook", None)
                if hook is not None:
                    hook()
            return (dx, None, None, None, None) + (None,) * len(ctx.params)
        pgrads = (None,) * len(ctx.params)
        if ctx.needs_input_grad[1] or any(ctx.needs_input_grad[5:]):
            full = torch.zeros_like(w)
            grouped_gemm_tn(dy, x, layout, full, accumulate=False)
            if ctx.needs_input_grad[1]:
                dw = full
            else:       # fused view of parameters without main_grad buffers: hand each its rows
                pgrads = tuple(full.split([p.shape[0] for p in ctx.params], dim=0))
        return (dx, dw, None, None, None) + pgrads


def grouped_linear(x: torch.Tensor, mods, layout: GroupLayout, out_rows: int) -> torch.Tensor:
    """``y[rows_e] = x[rows_e] @ W_e.T`` for the padded expert-major ``x``; ``mods`` are the bias-free
    linears whose weights, stacked in order, form expert e's ``[out_rows, in]`` matrix (several per
    expert when projections are fused, e.g. gate and up)."""
    from .gemm import WeightSet
    ws = WeightSet.of(mods)
    if ws.fused_weight is not None:
        return _GroupedLinearFn.apply(x, ws.fused_weight, layout, out_rows, ws.fused_main_grad, *ws.params)
    w = torch.cat(list(ws.params), dim=0)      # separate parameters: stack (differentiable)
    return _GroupedLinearFn.apply(x, w, layout, out_rows, None)


def grouped_linear_ref(x, weights: List[torch.Tensor], layout: GroupLayout):
    """Plain PyTorch restatement (test oracle): per-expert ``F.linear`` on the padded layout."""
    seg = layout.seg_start.tolist()
    outs = [F.linear(x[seg[e]:seg[e + 1]], weights[e]) for e in range(layout.num_groups)]
    return torch.cat(outs, dim=0)


def kernel_ok(x: torch.Tensor, *dims: int) -> bool:
    return use_kernels(x) and x.dtype == torch.bfloat16 and all(d % 64 == 0 for d in dims)
