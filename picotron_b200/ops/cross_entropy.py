"""Cross entropy that never keeps a softmax tensor, dense or vocabulary-parallel.

The loss of a row is ``log(sum_j exp(l_j - m)) + m - l_target``. On a vocabulary shard each
rank computes ``(m, sum, l_target)`` for its columns, the triples are combined over the
tensor-parallel group (one packed all-gather instead of the three all-reduces of
picotron/tensor_parallel/tp_communications.py:150,160,166), and the gradient
``(softmax - onehot) * g`` overwrites the logits in place during the same pass that evaluates
the loss. The reference keeps a full ``[N, V/tp]`` softmax for the backward
(tp_communications.py:139-174); here the logits buffer itself becomes the gradient.

``cross_entropy(logits, targets)`` returns the per-token loss (fp32) like
``vocab_parallel_cross_entropy`` in the reference; callers take the mean.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import count_launch, ext, use_kernels


def cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Per-token loss, dense vocabulary."""
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.view(-1), reduction="none")


#: process group -> object with ``stats_loss_grad(l2, targets, loss, dlogits, scale, vocab_start)`` that
#: exchanges the per-shard triples through NVLink peer memory inside the two loss kernels
#: (``ops.fused_tp.PeerStatsExchange``); installed by the engine for its tensor-parallel group
_PEER_EXCHANGE = {}


def install_peer_exchange(group, exchange) -> None:
    if exchange is None:
        _PEER_EXCHANGE.pop(group, None)
    else:
        _PEER_EXCHANGE[group] = exchange


def _stats_loss_grad(l2, t, loss, dlogits, scale, vocab_start, group):
    """The two kernel passes of the fused loss: statistics, then loss + gradient over the logits."""
    rows, V = l2.shape
    ex = _PEER_EXCHANGE.get(group) if group is not None else None
    if ex is not None and ex.fits(rows):
        ex.stats_loss_grad(l2, t, loss, dlogits, scale, vocab_start)
        return
    stats = torch.empty((rows, 3), device=l2.device, dtype=torch.float32)
    ext().ce_stats(l2, l2.stride(0), t, stats, rows, V, vocab_start)
    stats = combine_stats(stats, group)
    ext().ce_loss_grad(l2, l2.stride(0), t, stats, loss, dlogits, dlogits.stride(0), scale, rows, V, vocab_start)
    count_launch(2)


def combine_stats(stats: torch.Tensor, group) -> torch.Tensor:
    """Merge per-shard (max, sumexp, target_logit) triples over ``group``. stats: [N, 3] fp32."""
    if group is None or dist.get_world_size(group) == 1:
        return stats
    world = dist.get_world_size(group)
    flat = torch.empty((world * stats.shape[0],) + tuple(stats.shape[1:]), device=stats.device, dtype=stats.dtype)
    dist.all_gather_into_tensor(flat, stats.contiguous(), group=group)
    gathered = flat.view((world,) + tuple(stats.shape))
    m = gathered[..., 0].max(dim=0).values
    s = (gathered[..., 1] * torch.exp(gathered[..., 0] - m)).sum(dim=0)
    t = gathered[..., 2].sum(dim=0)
    return torch.stack([m, s, t], dim=-1)


def vocab_parallel_cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int,
                                     group) -> torch.Tensor:
    """Pure-torch vocabulary-parallel loss with autograd through the local shard."""
    lf = logits.float().view(-1, logits.shape[-1])
    t = targets.view(-1)
    V = lf.shape[-1]
    local_max = lf.max(dim=-1).values
    gmax = local_max.detach().clone()
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    shifted = lf - gmax[:, None]
    sumexp = _AllReduceSum.apply(shifted.exp().sum(dim=-1), group)
    local_t = t - vocab_start
    in_shard = (local_t >= 0) & (local_t < V)
    safe = local_t.clamp(0, V - 1)
    tl = shifted.gather(1, safe[:, None]).squeeze(1) * in_shard.to(lf.dtype)
    tl = _AllReduceSum.apply(tl, group)
    return sumexp.log() - tl


class _AllReduceSum(torch.autograd.Function):
    """Sum over the group in forward; identity gradient (every rank holds the same loss)."""

    @staticmethod
    def forward(ctx, x, group):
        if group is None or dist.get_world_size(group) == 1:
            return x
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _FusedCEFn(torch.autograd.Function):
    """Per-token loss; the gradient w.r.t. the logits is produced in the forward pass, scaled by
    ``grad_scale`` and written over the logits. The incoming gradient of the loss must therefore
    be uniform (``loss.sum() * c`` or ``loss.mean()``): it is applied as a scalar in backward."""

    @staticmethod
    def forward(ctx, logits, targets, vocab_start, group, inplace):
        V = logits.shape[-1]
        l2 = logits.view(-1, V)
        assert l2.stride(1) == 1
        rows = l2.shape[0]
        t = targets.reshape(-1)
        if not t.is_contiguous():
            t = t.contiguous()
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        dlogits = l2 if inplace else torch.empty_like(l2)
        _stats_loss_grad(l2, t, loss, dlogits, 1.0, vocab_start, group)
        ctx.save_for_backward(dlogits)
        ctx.shape = logits.shape
        return loss.view(targets.shape)

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        # uniform upstream gradient: read one element (stays on device, no sync)
        scale = dloss.reshape(-1)[:1].to(dlogits.dtype)
        dlogits.mul_(scale)
        return dlogits.view(ctx.shape), None, None, None, None


class _FusedMeanCEFn(torch.autograd.Function):
    """Scalar ``mean(loss) / divisor``. The gradient of that scalar w.r.t. the logits,
    ``(softmax - onehot) / (rows * divisor)``, is written over the logits during the forward pass.
    When the result is what ``backward()`` is called on (incoming gradient 1, the training loop's
    case) backward hands that buffer out untouched; any other incoming gradient is applied by a
    kernel that first reads the scalar on the device and returns at once when it is 1, so the
    common case costs no pass over ``[rows, V]`` and no host synchronisation."""

    @staticmethod
    def forward(ctx, logits, targets, vocab_start, group, divisor):
        V = logits.shape[-1]
        l2 = logits.view(-1, V)
        assert l2.stride(1) == 1
        rows = l2.shape[0]
        t = targets.reshape(-1)
        if not t.is_contiguous():
            t = t.contiguous()
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        scale = 1.0 / (rows * divisor)
        _stats_loss_grad(l2, t, loss, l2, scale, vocab_start, group)
        ctx.save_for_backward(l2)
        ctx.shape = logits.shape
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        if dlogits.is_contiguous():
            ext().scale_unless_one(dlogits, dloss.reshape(1).float())
            count_launch()
        else:
            dlogits.mul_(dloss.to(dlogits.dtype))
        return dlogits.view(ctx.shape), None, None, None, None


def mean_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0, group=None,
                       divisor: float = 1.0) -> torch.Tensor:
    """``cross_entropy(...).mean() / divisor`` as a scalar; on the kernel path the logits are consumed
    and the result must be what ``backward()`` is called on (see ``_FusedMeanCEFn``)."""
    if use_kernels(logits) and logits.shape[-1] % 8 == 0 and logits.is_contiguous() and torch.is_grad_enabled() \
            and logits.requires_grad:
        return _FusedMeanCEFn.apply(logits, targets, vocab_start, group, float(divisor))
    return cross_entropy(logits, targets, vocab_start, group).mean() / divisor


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0, group=None,
                  inplace: bool = True) -> torch.Tensor:
    """Per-token loss over (a shard of) the vocabulary. With ``inplace`` the logits are consumed."""
    if use_kernels(logits) and logits.shape[-1] % 8 == 0 and logits.is_contiguous():
        return _FusedCEFn.apply(logits, targets, vocab_start, group, inplace)
    if group is None or dist.get_world_size(group) == 1:
        return cross_entropy_ref(logits, targets).view(targets.shape)
    return vocab_parallel_cross_entropy_ref(logits, targets, vocab_start, group).view(targets.shape)
