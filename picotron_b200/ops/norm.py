"""RMSNorm with the residual add folded in.

``rmsnorm(x, w, eps)`` is the plain norm; ``add_rmsnorm(x, residual, w, eps)`` returns
``(norm(x + residual), x + residual)`` from one pass over memory. fp32 statistics, as
picotron/model.py:96-115 (LlamaRMSNorm) computes them.
"""
from __future__ import annotations

import torch

from . import count_launch, ext, use_kernels

_scratch: dict = {}


def _partials(device, H: int) -> torch.Tensor:
    key = (device, H)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(ext().rmsnorm_bwd_num_partials() * H, device=device, dtype=torch.float32)
        _scratch[key] = buf
    return buf


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    dtype = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (w.float() * (xf * torch.rsqrt(var + eps))).to(dtype)


def add_rmsnorm_ref(x, residual, w, eps):
    h = x + residual
    return rmsnorm_ref(h, w, eps), h


def _c2d(t: torch.Tensor, H: int) -> torch.Tensor:
    t2 = t.reshape(-1, H)
    return t2 if t2.is_contiguous() else t2.contiguous()


def _backward(ctx, dy, dh_in):
    h, w, rstd = ctx.saved_tensors
    rows, H = h.shape
    dy2 = _c2d(dy, H)
    dres = _c2d(dh_in, H) if dh_in is not None else None
    dh = torch.empty_like(h)
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        ext().rmsnorm_bwd(dy2, h, w, rstd, dres, dh, _partials(h.device, H), main_grad, None, True, rows, H)
        dw = None
        hook = getattr(w, "grad_ready_hook", None)
        if hook is not None:
            hook()
    else:
        dw = torch.empty_like(w)
        ext().rmsnorm_bwd(dy2, h, w, rstd, dres, dh, _partials(h.device, H), None, dw, False, rows, H)
    count_launch(2)
    return dh.view(ctx.shape), dw


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        H = x.shape[-1]
        x2 = _c2d(x, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        ext().rmsnorm_fwd(x2, None, w, y, None, rstd, rows, H, eps)
        count_launch()
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        dh, dw = _backward(ctx, dy, None)
        return dh, dw, None


class _AddRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps):
        H = x.shape[-1]
        x2 = _c2d(x, H)
        r2 = _c2d(residual, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        h = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        ext().rmsnorm_fwd(x2, r2, w, y, h, rstd, rows, H, eps)
        count_launch()
        ctx.save_for_backward(h, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh_in):
        dh, dw = _backward(ctx, dy, dh_in)
        return dh, dh, dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if use_kernels(x, w) and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, w, eps)
    return rmsnorm_ref(x, w, eps)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, w: torch.Tensor, eps: float):
    """Returns (norm(x + residual), x + residual); residual=None means the stream is x itself."""
    if residual is None:
        return rmsnorm(x, w, eps), x
    if use_kernels(x, w) and x.shape[-1] % 8 == 0:
        return _AddRMSNormFn.apply(x, residual, w, eps)
    return add_rmsnorm_ref(x, residual, w, eps)
