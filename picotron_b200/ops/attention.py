"""Scaled dot-product attention in the ``[batch, seq, heads, head_dim]`` layout.

``attention(q, k, v, causal)`` accepts grouped-query inputs (fewer K/V heads than Q heads)
without materialising the repeated heads that picotron/model.py:197-202 creates.
``attention_block(q, k, v, causal)`` additionally returns the log-sum-exp per (batch, head,
query) so partial results over different key blocks can be merged exactly — the building
block of ring attention (picotron/context_parallel/context_parallel.py:240-290).
``merge_attention_blocks`` is that merge (context_parallel.py:293-323), written with
``logaddexp`` instead of the sigmoid/logsigmoid pair.

Everything here is differentiable through ordinary autograd (the block form uses explicit
matmuls so it runs on CPU/gloo); the CUDA fast path for whole-sequence attention is selected
in ``attention``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _expand_kv(k: torch.Tensor, n_heads: int) -> torch.Tensor:
    """[b, s, kvh, d] -> [b, s, n_heads, d] by repeating each KV head for its query group."""
    kvh = k.shape[2]
    if kvh == n_heads:
        return k
    rep = n_heads // kvh
    return k[:, :, :, None, :].expand(-1, -1, -1, rep, -1).reshape(k.shape[0], k.shape[1], n_heads, k.shape[3])


def attention_ref(q, k, v, causal: bool, sm_scale: float | None = None) -> torch.Tensor:
    """fp32-accumulating reference. q: [b, sq, H, d], k/v: [b, sk, Hkv, d] -> [b, sq, H, d]."""
    out, _ = attention_block(q, k, v, causal, sm_scale)
    return out


def attention_block(q, k, v, causal: bool, sm_scale: float | None = None, q_offset: int = 0,
                    k_offset: int = 0):
    """Attention of q against one block of keys, returning (out, lse).

    ``q_offset`` / ``k_offset`` are the global positions of the first query / key; with
    ``causal`` a query at global position i sees keys at global positions <= i. Rows that see
    no key get out = 0 and lse = -inf. lse has shape [b, H, sq] (fp32).
    """
    b, sq, H, d = q.shape
    sk = k.shape[1]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d)
    kf = _expand_kv(k, H)
    vf = _expand_kv(v, H)
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf.float()) * scale
    if causal:
        qi = torch.arange(sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(sk, device=q.device)[None, :] + k_offset
        scores = scores.masked_fill(ki > qi, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)  # [b, H, sq]
    safe_lse = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(scores - safe_lse[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    out = torch.einsum("bhqk,bkhd->bqhd", p, vf.float())
    return out.to(q.dtype), lse


def merge_attention_blocks(out, lse, blk_out, blk_lse):
    """Exact merge of two partial attention results over disjoint key sets.

    out/blk_out: [b, s, H, d]; lse/blk_lse: [b, H, s] fp32. Returns (out, lse) with out fp32.
    """
    if out is None:
        return blk_out.float(), blk_lse
    if blk_out.is_cuda and blk_out.dtype == torch.bfloat16 and out.dtype in (torch.float32, torch.bfloat16) \
            and out.is_contiguous() and blk_out.is_contiguous() and lse.is_contiguous() and blk_lse.is_contiguous() \
            and not reference_ops_forced_() and not torch.is_grad_enabled():
        # one kernel instead of six eager ones (the ring forward runs under no_grad: its autograd
        # function owns the backward); fp32 accumulators are updated in place
        from . import count_launch, ext
        merged = out if out.dtype == torch.float32 else torch.empty(out.shape, device=out.device, dtype=torch.float32)
        new_lse = torch.empty_like(lse)
        ext().attn_merge(out, lse, blk_out, blk_lse, merged, new_lse)
        count_launch()
        return merged, new_lse
    new_lse = torch.logaddexp(lse, blk_lse)
    safe = torch.where(torch.isinf(new_lse), torch.zeros_like(new_lse), new_lse)
    w_old = torch.exp(lse - safe).transpose(1, 2).unsqueeze(-1)      # [b, s, H, 1]
    w_new = torch.exp(blk_lse - safe).transpose(1, 2).unsqueeze(-1)
    return out.float() * w_old + blk_out.float() * w_new, new_lse


def _packed_heads(t: torch.Tensor) -> bool:
    return t.stride(3) == 1 and t.stride(2) == t.shape[3] and (t.stride(1) * 2) % 16 == 0 \
        and (t.stride(0) * 2) % 16 == 0 and t.data_ptr() % 16 == 0


def flash_attention_forward(q, k, v, causal, sm_scale=None, q_pos0: int = 0, k_pos0: int = 0):
    """tcgen05 kernel: returns (out [b, sq, H, d] bf16, lse [b, H, sq] fp32)."""
    from . import count_launch, ext
    b, sq, H, d = q.shape
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d)
    q, k, v = (t if _packed_heads(t) else t.contiguous() for t in (q, k, v))
    out = torch.empty((b, sq, H, d), device=q.device, dtype=q.dtype)
    lse = torch.empty((b, H, sq), device=q.device, dtype=torch.float32)
    ext().attention_fwd(q, k, v, out, lse, scale, causal, q_pos0, k_pos0, None)
    count_launch()
    return out, lse


def flash_attention_backward(dout, q, k, v, out, lse, causal, sm_scale=None, q_pos0: int = 0, k_pos0: int = 0):
    """tcgen05 kernel: returns (dq, dk, dv) as column slices of one ``[b, s, (H + 2*Hkv)*d]`` buffer when
    the sequence lengths match (so a fused QKV projection can consume them without a copy)."""
    from . import count_launch, ext
    b, sq, H, d = q.shape
    sk, kvh = k.shape[1], k.shape[2]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d)
    q, k, v, dout, out = (t if _packed_heads(t) else t.contiguous() for t in (q, k, v, dout, out))
    if sq == sk:
        fused = torch.empty((b, sq, (H + 2 * kvh) * d), device=q.device, dtype=q.dtype)
        dq = fused[..., :H * d].view(b, sq, H, d)
        dk = fused[..., H * d:(H + kvh) * d].view(b, sk, kvh, d)
        dv = fused[..., (H + kvh) * d:].view(b, sk, kvh, d)
    else:
        dq = torch.empty((b, sq, H, d), device=q.device, dtype=q.dtype)
        dk = torch.empty((b, sk, kvh, d), device=q.device, dtype=q.dtype)
        dv = torch.empty((b, sk, kvh, d), device=q.device, dtype=q.dtype)
    delta = torch.empty((b, H, sq), device=q.device, dtype=torch.float32)
    dq_accum = torch.empty((b, sq, H, d), device=q.device, dtype=torch.float32)
    ext().attention_bwd(q, k, v, out, dout, lse, dq, dk, dv, delta, dq_accum, scale, causal, q_pos0, k_pos0)
    count_launch(4)
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale):
        out, lse = flash_attention_forward(q, k, v, causal, sm_scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.sm_scale = causal, sm_scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attention_backward(dout, q, k, v, out, lse, ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None


class _RopeAttentionFn(torch.autograd.Function):
    """Rotary embedding + causal attention on the fused QKV projection output.

    ``qkv``: [b, s, (H + 2*Hkv)*d] as the fused GEMM wrote it. q and k are rotated in place (the
    projection output is not needed by any other backward), attention runs on strided views, and
    the backward writes dq/dk/dv straight into one ``[b, s, (H + 2*Hkv)*d]`` buffer, un-rotates
    dq/dk in place and hands that buffer to the projection's backward: no split / cat / clone copies.
    """

    @staticmethod
    def forward(ctx, qkv, H, Hkv, d, cos_half, sin_half, pos_offset, causal, sm_scale):
        from .rope import rope_inplace_
        b, s, _ = qkv.shape
        raw = qkv.detach()
        q = raw[..., :H * d].view(b, s, H, d)
        k = raw[..., H * d:(H + Hkv) * d].view(b, s, Hkv, d)
        v = raw[..., (H + Hkv) * d:].view(b, s, Hkv, d)
        # q and k lie side by side in the fused buffer: one launch rotates the H + Hkv heads of both
        rope_inplace_(raw[..., :(H + Hkv) * d].view(b, s, H + Hkv, d), cos_half, sin_half, pos_offset, 1)
        out, lse = flash_attention_forward(q, k, v, causal, sm_scale)
        ctx.save_for_backward(raw, out, lse, cos_half, sin_half)
        ctx.dims = (H, Hkv, d, pos_offset, causal, sm_scale)
        return out.view(b, s, H * d)

    @staticmethod
    def backward(ctx, dout):
        from .rope import rope_inplace_
        raw, out, lse, cos_half, sin_half = ctx.saved_tensors
        H, Hkv, d, pos_offset, causal, sm_scale = ctx.dims
        b, s, _ = raw.shape
        q = raw[..., :H * d].view(b, s, H, d)
        k = raw[..., H * d:(H + Hkv) * d].view(b, s, Hkv, d)
        v = raw[..., (H + Hkv) * d:].view(b, s, Hkv, d)
        dq, dk, dv = flash_attention_backward(dout.reshape(b, s, H, d), q, k, v, out, lse, causal, sm_scale)
        fused = dq._base
        if fused is not None and fused.shape == raw.shape and fused.is_contiguous():
            # dq | dk | dv of one buffer: un-rotate dq and dk in one launch
            rope_inplace_(fused[..., :(H + Hkv) * d].view(b, s, H + Hkv, d), cos_half, sin_half, pos_offset, -1)
            return fused, None, None, None, None, None, None, None, None
        rope_inplace_(dq, cos_half, sin_half, pos_offset, -1)
        rope_inplace_(dk, cos_half, sin_half, pos_offset, -1)
        dqkv = torch.cat([dq.reshape(b, s, -1), dk.reshape(b, s, -1), dv.reshape(b, s, -1)], dim=-1)
        return dqkv, None, None, None, None, None, None, None, None


def rope_attention_fused(qkv, H, Hkv, d, cos_half, sin_half, pos_offset, causal=True, sm_scale=None):
    return _RopeAttentionFn.apply(qkv, H, Hkv, d, cos_half, sin_half, pos_offset, causal, sm_scale)


def reference_ops_forced_() -> bool:
    from . import reference_ops_forced
    return reference_ops_forced()


def kernel_supports(q, k) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and q.shape[2] % k.shape[2] == 0


def attention(q, k, v, causal: bool = True, sm_scale: float | None = None) -> torch.Tensor:
    """Whole-sequence attention. q: [b, s, H, d]; k, v: [b, s, Hkv, d] -> [b, s, H, d]. bf16 CUDA
    tensors with head_dim 64 or 128 run on the tcgen05 flash-attention kernels of this library;
    everything else uses the torch restatement."""
    from . import reference_ops_forced
    if kernel_supports(q, k) and not reference_ops_forced():
        return _FlashAttnFn.apply(q, k, v, causal, sm_scale)
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        H, kvh = q.shape[2], k.shape[2]
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=causal, scale=sm_scale, enable_gqa=(H != kvh))
        return o.transpose(1, 2)
    return attention_ref(q, k, v, causal, sm_scale)


def attention_block_backward(dout, q, k, v, out, lse, causal: bool, sm_scale: float | None = None,
                             q_offset: int = 0, k_offset: int = 0):
    """Gradients of one key block's contribution given the *final* (merged) ``out`` and ``lse``.

    With P = exp(S - lse) the probabilities under the global normaliser, dV = P^T dO,
    dS = P * (dO V^T - rowsum(dO * O)), dQ = dS K * scale, dK = dS^T Q * scale
    (picotron/context_parallel/context_parallel.py:262-290). Returns fp32 (dq, dk, dv) with dk/dv
    in the un-expanded K/V head layout.
    """
    b, sq, H, d = q.shape
    sk, kvh = k.shape[1], k.shape[2]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(d)
    kf, vf = _expand_kv(k, H).float(), _expand_kv(v, H).float()
    qf, dof = q.float(), dout.float()
    scores = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    if causal:
        qi = torch.arange(sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(sk, device=q.device)[None, :] + k_offset
        scores = scores.masked_fill(ki > qi, float("-inf"))
    safe_lse = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(scores - safe_lse[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    dv = torch.einsum("bhqk,bqhd->bkhd", p, dof)
    dp = torch.einsum("bqhd,bkhd->bhqk", dof, vf)
    delta = (dof * out.float()).sum(-1).transpose(1, 2)  # [b, H, sq]
    ds = p * (dp - delta[..., None])
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf) * scale
    dk = torch.einsum("bhqk,bqhd->bkhd", ds, qf) * scale
    if kvh != H:
        rep = H // kvh
        dk = dk.view(b, sk, kvh, rep, d).sum(3)
        dv = dv.view(b, sk, kvh, rep, d).sum(3)
    return dq, dk, dv
