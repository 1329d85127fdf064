"""Token embedding lookup, optionally on a vocabulary shard.

Ids outside ``[vocab_start, vocab_start + V_local)`` produce zero rows, which is what a
vocabulary-parallel embedding sums over the tensor-parallel group
(picotron/tensor_parallel/tensor_parallel.py:365-381). The backward scatters into the fp32
``main_grad`` of the table when it has one.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import count_launch, ext, use_kernels


def embedding_ref(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    V = weight.shape[0]
    local = ids - vocab_start
    mask = (local < 0) | (local >= V)
    safe = local.clamp(0, V - 1)
    out = F.embedding(safe, weight)
    return out.masked_fill(mask.unsqueeze(-1), 0.0)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start):
        V, H = weight.shape
        flat = ids.reshape(-1).contiguous()
        out = torch.empty((flat.numel(), H), device=weight.device, dtype=weight.dtype)
        ext().embedding_fwd(weight, flat, out, flat.numel(), H, V, vocab_start)
        count_launch()
        ctx.save_for_backward(flat, weight)
        ctx.vocab_start = vocab_start
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        flat, weight = ctx.saved_tensors
        V, H = weight.shape
        d2 = dout.reshape(-1, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            ext().embedding_bwd(d2, flat, main_grad, flat.numel(), H, V, ctx.vocab_start)
            count_launch()
            hook = getattr(weight, "grad_ready_hook", None)
            if hook is not None:
                hook()
            return None, None, None
        acc = torch.zeros((V, H), device=weight.device, dtype=torch.float32)
        ext().embedding_bwd(d2, flat, acc, flat.numel(), H, V, ctx.vocab_start)
        count_launch()
        return None, acc.to(weight.dtype), None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    if use_kernels(weight) and weight.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, weight, vocab_start)
    return embedding_ref(ids, weight, vocab_start)
