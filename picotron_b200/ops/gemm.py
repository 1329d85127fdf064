"""Bias-free linear layers on the tcgen05 GEMM.

``linear(x, w)`` computes ``x @ w.T`` like ``F.linear``. On bf16 CUDA tensors forward, dgrad
and wgrad all run on ``csrc/gemm/gemm_bf16_sm100.cu`` without transposed copies (the kernel
reads K-major and MN-major operands). When the weight carries an fp32 ``main_grad`` buffer the
wgrad GEMM accumulates straight into it (TMA reduce-add epilogue) — the bucket accumulation the
reference does with a separate ``main_grad.add_(grad)`` per parameter
(picotron/data_parallel/data_parallel.py:143) — and autograd sees no weight gradient.

Reference: picotron/model.py:160-162,232,258,285 (F.linear call sites).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import count_launch, ext, use_kernels


def linear_ref(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w)


def _rows(x: torch.Tensor) -> int:
    return x.numel() // x.shape[-1]


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, max_ctas: int = 0,
            out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out[M,N] = a[M,K] @ b[N,K].T  (both K-contiguous; row strides may exceed K)."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    mode = 0 if out.dtype == torch.bfloat16 else 1
    ext().gemm(a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), False, False, mode, max_ctas)
    count_launch()
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
    """out[M,N] = a[M,K] @ b[K,N]  (b is N-contiguous)."""
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.bfloat16)
    mode = 0 if out.dtype == torch.bfloat16 else 1
    ext().gemm(a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), False, True, mode, max_ctas)
    count_launch()
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
            max_ctas: int = 0) -> torch.Tensor:
    """out[M,N] (+)= a[K,M].T @ b[K,N]. ``accumulate`` needs an fp32 ``out``."""
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.bfloat16)
    if accumulate:
        assert out.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if out.dtype == torch.bfloat16 else 1
    ext().gemm(a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), True, True, mode, max_ctas)
    count_launch()
    return out


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0:
        x2 = x2.contiguous()
    return x2


def _gemm_ok(*dims: int) -> bool:
    # TMA needs 16-byte aligned pitches: every contiguous extent a multiple of 8 bf16
    return all(d % 8 == 0 for d in dims)


def wgrad_into(weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor):
    """Weight gradient of y = x @ w.T. Accumulates into ``weight.main_grad`` (fp32) when the
    parameter has one and returns None; otherwise returns the bf16 gradient."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        gemm_tn(dy2, x2, out=main_grad, accumulate=True)
        hook = getattr(weight, "grad_ready_hook", None)
        if hook is not None:
            hook()
        return None
    return gemm_tn(dy2, x2)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = _as_2d(x)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        y = gemm_nt(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = wgrad_into(w, dy2, x2)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if use_kernels(x, w) and _gemm_ok(x.shape[-1], w.shape[0]):
        return _LinearFn.apply(x, w)
    if _ZB_MODE and torch.is_grad_enabled():
        return _LinearRefFn.apply(x, w)
    return linear_ref(x, w)


# ---------------------------------------------------------------------------------------------
# several projections of one input
# ---------------------------------------------------------------------------------------------
class WeightSet:
    """The weights of projections that share an input: either separate parameters or one fused
    ``[sum(out_i), in]`` view over parameters stored back to back (see ``param_store``)."""

    def __init__(self, params, fused_weight=None, fused_main_grad=None):
        self.params = list(params)
        self.fused_weight = fused_weight
        self.fused_main_grad = fused_main_grad
        self.splits = [p.shape[0] for p in self.params]

    @staticmethod
    def of(mods) -> "WeightSet":
        fused = getattr(mods[0], "_fused_group", None)
        if fused is not None and len(fused.mods) == len(mods) and all(a is b for a, b in zip(fused.mods, mods)):
            return WeightSet([m.weight for m in mods], fused.weight, fused.main_grad)
        return WeightSet([m.weight for m in mods])

    @property
    def out_features(self) -> int:
        return sum(self.splits)


def project_all(x2: torch.Tensor, ws: WeightSet) -> torch.Tensor:
    """x2[M,K] -> [M, sum(out_i)]; one GEMM when fused, else one per weight into column slices."""
    M = x2.shape[0]
    if ws.fused_weight is not None:
        return gemm_nt(x2, ws.fused_weight)
    out = torch.empty((M, ws.out_features), device=x2.device, dtype=x2.dtype)
    col = 0
    for w in ws.params:
        gemm_nt(x2, w, out=out[:, col:col + w.shape[0]])
        col += w.shape[0]
    return out


def backward_all(dy2: torch.Tensor, x2: torch.Tensor, ws: WeightSet, need_dx: bool = True):
    """Returns (dx2 or None, [grad per param or None when accumulated into main_grad])."""
    dx = None
    if ws.fused_weight is not None:
        if need_dx:
            dx = gemm_nn(dy2, ws.fused_weight)
        if ws.fused_main_grad is not None:
            gemm_tn(dy2, x2, out=ws.fused_main_grad, accumulate=True)
            for p in ws.params:
                hook = getattr(p, "grad_ready_hook", None)
                if hook is not None:
                    hook()
            return dx, [None] * len(ws.params)
        dw = gemm_tn(dy2, x2)
        return dx, list(dw.split(ws.splits, dim=0))
    grads = []
    col = 0
    for w in ws.params:
        dyi = dy2[:, col:col + w.shape[0]]
        col += w.shape[0]
        if need_dx:
            part = gemm_nn(dyi, w)
            dx = part if dx is None else dx.add_(part)
        grads.append(wgrad_into(w, dyi, x2))
    return dx, grads


class _MultiLinearFn(torch.autograd.Function):
    """y = x @ cat(weights).T as one output tensor; parameters are passed so that autograd runs
    the backward (and with it the main_grad accumulation) even when x needs no gradient."""

    @staticmethod
    def forward(ctx, x, ws, *params):
        x2 = _as_2d(x)
        ctx.ws = ws
        ctx.x_shape = x.shape
        ctx.save_for_backward(x2)
        return project_all(x2, ws).view(*x.shape[:-1], ws.out_features)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx, grads = backward_all(dy2, x2, ctx.ws, need_dx=ctx.needs_input_grad[0])
        return (dx.view(ctx.x_shape) if dx is not None else None, None, *grads)


def multi_linear_cat(x: torch.Tensor, mods) -> torch.Tensor:
    """Concatenated outputs ``[..., sum(out_i)]`` of bias-free projections sharing the input x."""
    ws = WeightSet.of(mods)
    if use_kernels(x, ws.params[0]) and _gemm_ok(x.shape[-1], *ws.splits):
        return _MultiLinearFn.apply(x, ws, *ws.params)
    return torch.cat([linear(x, w) for w in ws.params], dim=-1)


# ---------------------------------------------------------------------------------------------
# zero-bubble support: weight gradients split off from the backward pass
# ---------------------------------------------------------------------------------------------
_ZB_MODE = False          # linears use the deferrable autograd functions also on the torch path
_DEFER_QUEUE = None       # list collecting weight-gradient closures while a "B" action runs


def set_zero_bubble(enabled: bool) -> None:
    """While enabled, every bias-free linear routes its backward through code that can postpone
    the weight gradient (the role of the globally patched ``nn.Linear.forward`` and
    ``_DeferredLinear`` in picotron/pipeline_parallel/pipeline_parallel.py:21-54)."""
    global _ZB_MODE
    _ZB_MODE = enabled


class defer_wgrad:
    """Context manager: weight gradients of linears whose backward runs inside are not computed
    but queued; ``run_deferred(queue)`` computes them later (the W action of a zero-bubble
    schedule)."""

    def __enter__(self):
        global _DEFER_QUEUE
        self.prev = _DEFER_QUEUE
        self.queue = []
        _DEFER_QUEUE = self.queue
        return self.queue

    def __exit__(self, *exc):
        global _DEFER_QUEUE
        _DEFER_QUEUE = self.prev
        return False


def run_deferred(queue) -> None:
    for fn in queue:
        fn()
    queue.clear()


def _accumulate_grad(p: torch.Tensor, g: torch.Tensor) -> None:
    main_grad = getattr(p, "main_grad", None)
    if main_grad is not None and p.is_cuda:
        main_grad.add_(g)
    elif p.grad is None:
        p.grad = g.to(p.dtype)
    else:
        p.grad = p.grad + g.to(p.dtype)


class _LinearRefFn(torch.autograd.Function):
    """Torch-path linear (any device / dtype) with a deferrable weight gradient."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return F.linear(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dy.matmul(w) if ctx.needs_input_grad[0] else None
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        if _DEFER_QUEUE is not None:
            _DEFER_QUEUE.append(lambda: _accumulate_grad(w, dy2.t().matmul(x2)))
            return dx, None
        return dx, dy2.t().matmul(x2)


_plain_wgrad_into = wgrad_into
_plain_backward_all = backward_all


def wgrad_into(weight, dy2, x2):  # noqa: F811  (deferral-aware wrapper)
    if _DEFER_QUEUE is not None:
        def later():
            g = _plain_wgrad_into(weight, dy2, x2)
            if g is not None:
                _accumulate_grad(weight, g)
        _DEFER_QUEUE.append(later)
        return None
    return _plain_wgrad_into(weight, dy2, x2)


def backward_all(dy2, x2, ws, need_dx=True):  # noqa: F811  (deferral-aware wrapper)
    if _DEFER_QUEUE is None:
        return _plain_backward_all(dy2, x2, ws, need_dx)
    dx = None
    if need_dx:
        if ws.fused_weight is not None:
            dx = gemm_nn(dy2, ws.fused_weight)
        else:
            col = 0
            for w in ws.params:
                part = gemm_nn(dy2[:, col:col + w.shape[0]], w)
                col += w.shape[0]
                dx = part if dx is None else dx.add_(part)

    def later():
        _, grads = _plain_backward_all(dy2, x2, ws, need_dx=False)
        for p, g in zip(ws.params, grads):
            if g is not None:
                _accumulate_grad(p, g)
    _DEFER_QUEUE.append(later)
    return dx, [None] * len(ws.params)
