"""SwiGLU activation on the fused gate|up projection.

``swiglu(gu)`` takes ``gu[..., 2*I]`` (gate in the first half, up in the second, as the fused
gate/up GEMM writes them) and returns ``silu(gate) * up``. Reference math:
picotron/model.py:258 (``down(silu(gate(x)) * up(x))``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import count_launch, ext, use_kernels


def swiglu_ref(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, rows_dev=None):
        I = gu.shape[-1] // 2
        gu2 = gu.reshape(-1, 2 * I)
        if gu2.stride(1) != 1:
            gu2 = gu2.contiguous()
        rows = gu2.shape[0]
        y = torch.empty((rows, I), device=gu.device, dtype=gu.dtype)
        ext().swiglu_fwd(gu2, gu2.stride(0), y, rows, I, rows_dev)
        count_launch()
        ctx.save_for_backward(gu2)
        ctx.shape, ctx.rows_dev = gu.shape, rows_dev
        return y.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        rows, two_i = gu2.shape
        I = two_i // 2
        dy2 = dy.reshape(rows, I)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dgu = torch.empty((rows, two_i), device=dy.device, dtype=dy.dtype)
        ext().swiglu_bwd(dy2, gu2, gu2.stride(0), dgu, two_i, rows, I, ctx.rows_dev)
        count_launch()
        return dgu.view(ctx.shape), None


def swiglu(gu: torch.Tensor, rows_in_use: torch.Tensor | None = None) -> torch.Tensor:
    """``rows_in_use``: optional int32 device scalar; rows at or past it are skipped (their outputs are
    unspecified) — for buffers whose fill level is known only on the device."""
    if use_kernels(gu) and gu.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(gu, rows_in_use)
    return swiglu_ref(gu)
