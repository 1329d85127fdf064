"""DeepSpeed-Ulysses context parallelism: trade the sequence shard for a head shard with an
all-to-all, run ordinary attention over the full sequence on ``heads / cp`` heads, and trade
back (picotron/context_parallel/ulysses.py:39-111).

The all-to-all uses the single-buffer collective, which also exists on gloo, and K/V are sent
with their own head count whenever it divides by the CP size (the reference always sends the
GQA-expanded heads).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import process_group_manager as pgm
from ..ops import attention as attn_ops
from .dist_utils import group_size


def _all_to_all(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    """Split ``x`` along ``scatter_dim`` into one piece per rank, exchange, concatenate the
    received pieces along ``gather_dim``."""
    n = group_size(group)
    if n == 1:
        return x
    assert x.shape[scatter_dim] % n == 0
    # bring the scatter dim to the front as [n, chunk, ...] so the exchange is one flat buffer
    parts = x.reshape(*x.shape[:scatter_dim], n, x.shape[scatter_dim] // n, *x.shape[scatter_dim + 1:])
    send = parts.movedim(scatter_dim, 0).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv.view(n, -1), send.view(n, -1), group=group)
    # recv[j] is rank j's piece: concatenate along gather_dim (positions shifted by the moved dim)
    pieces = recv.unbind(0)
    return torch.cat(pieces, dim=gather_dim)


class _SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group):
        ctx.scatter_dim, ctx.gather_dim, ctx.group = scatter_dim, gather_dim, group
        return _all_to_all(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, grad):
        return _all_to_all(grad.contiguous(), ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None, None


#: optional ``ops.fused_ulysses.UlyssesFused``: the all-to-alls as peer-memory store kernels
_FUSED = None


def install_fused_ulysses(u) -> None:
    global _FUSED
    _FUSED = u


def ulysses_attention_bshd(q, k, v, causal: bool = True, sm_scale=None, group=None):
    """q: [b, s/cp, H, d]; k, v: [b, s/cp, Hkv, d] -> [b, s/cp, H, d]."""
    group = group if group is not None else pgm.get_pgm().cp_group
    n = group_size(group)
    if n == 1:
        return attn_ops.attention(q, k, v, causal, sm_scale)
    H, kvh = q.shape[2], k.shape[2]
    assert H % n == 0, f"Ulysses needs the local head count ({H}) divisible by the CP size ({n})"
    if kvh % n != 0:
        k, v = attn_ops._expand_kv(k, H), attn_ops._expand_kv(v, H)
    u = _FUSED
    if u is not None and u.sg.group is group and q.is_cuda and q.dtype == torch.bfloat16 \
            and u.matches(q, True) and u.matches(k, True) and not attn_ops.reference_ops_forced_():
        from ..ops import fused_ulysses as fu
        out = attn_ops.attention(fu.heads_to_seq(q, u), fu.heads_to_seq(k, u), fu.heads_to_seq(v, u), causal, sm_scale)
        return fu.seq_to_heads(out, u)
    # [b, s/cp, H, d] -> scatter heads (dim 2), gather sequence (dim 1) -> [b, s, H/cp, d]
    qg = _SeqAllToAll.apply(q, 2, 1, group)
    kg = _SeqAllToAll.apply(k, 2, 1, group)
    vg = _SeqAllToAll.apply(v, 2, 1, group)
    out = attn_ops.attention(qg, kg, vg, causal, sm_scale)
    return _SeqAllToAll.apply(out, 1, 2, group)


def ulysses_attention(q, k, v, causal=None, group=None, is_causal=None):
    """Reference-layout entry point on ``[b, heads, s_local, d]`` tensors (``causal`` is the reference's
    parameter name, ulysses.py:86 there; ``is_causal`` the name its ring counterpart uses)."""
    causal = is_causal if causal is None else causal
    assert causal is not None, "pass causal=True/False"
    out = ulysses_attention_bshd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), bool(causal), None, group)
    return out.transpose(1, 2)
