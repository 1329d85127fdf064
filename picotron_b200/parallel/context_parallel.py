"""Context parallelism: ring attention over sequence shards.

Every CP rank holds a contiguous slice of the sequence (rank r: positions
``[r*s/cp, (r+1)*s/cp)``). ``ring_attention`` rotates the K/V blocks around the ring while
each rank attends its queries to the block in hand and merges the partial results with their
log-sum-exps; the backward pass runs a second K/V ring together with a ring that carries the
fp32 dK/dV accumulators back to their owners (picotron/context_parallel/context_parallel.py:
150-237). Differences from the reference:

* K and V travel with their own (un-expanded) head count; grouped-query expansion happens
  inside the block attention, which cuts ring traffic by ``heads / kv_heads``
* the causal structure is expressed with global positions (a block is skipped when all its keys
  lie in the future, masked only on the diagonal), so any shard layout could be plugged in
* transfers never synchronise the device
* ``apply_context_parallel(model, attention=...)`` installs the attention backend and the RoPE
  position offset on the model instead of setting environment variables

The public ``ring_attention(q, k, v, sm_scale, is_causal)`` takes ``[b, heads, s_local, d]``
tensors like the reference; the model calls the ``[b, s, heads, d]`` form directly.
"""
from __future__ import annotations

import torch

from .. import process_group_manager as pgm
from ..ops import attention as attn_ops
from .cp_communications import ContextCommunicate
from .dist_utils import group_rank, group_size


def shard_pieces(rank: int, n: int, s_loc: int, zigzag: bool):
    """How rank ``rank`` of ``n`` holds its ``s_loc`` tokens: a list of (local start, length, global
    position of the first token). Contiguous sharding is one piece at ``rank * s_loc``. Zigzag sharding
    cuts the sequence into ``2n`` chunks and gives rank r chunks r and 2n-1-r, which balances causal
    attention: every rank owns one early (cheap) and one late (expensive) chunk."""
    if not zigzag:
        return [(0, s_loc, rank * s_loc)]
    assert s_loc % 2 == 0, "zigzag sharding needs an even number of tokens per rank"
    h = s_loc // 2
    return [(0, h, rank * h), (h, h, (2 * n - 1 - rank) * h)]


class _RingAttention(torch.autograd.Function):
    """q: [b, s_loc, H, d]; k, v: [b, s_loc, Hkv, d] (this rank's shard, contiguous or zigzag pieces)."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale, causal, group, zigzag):
        n, rank = group_size(group), group_rank(group)
        s_loc = q.shape[1]
        comm = ContextCommunicate("fwd", group=group, send_rank=_ring_peer(group, +1),
                                  recv_rank=_ring_peer(group, -1))
        q_pieces = shard_pieces(rank, n, s_loc, zigzag)
        acc = [(None, None) for _ in q_pieces]           # (out, lse) per query piece
        cur_k, cur_v = k.contiguous(), v.contiguous()
        use_kernel = attn_ops.kernel_supports(q, k) and not attn_ops.reference_ops_forced_()
        for step in range(n):
            if step + 1 < n:
                next_k = comm.send_recv(cur_k)
                next_v = comm.send_recv(cur_v)
                comm.commit()
            src = (rank - step) % n          # owner of the block in hand
            for qi, (q0, qlen, qpos) in enumerate(q_pieces):
                for k0, klen, kpos in shard_pieces(src, n, s_loc, zigzag):
                    if causal and kpos > qpos + qlen - 1:
                        continue             # every key of this piece lies in the future of every query
                    qq, kk, vv = q[:, q0:q0 + qlen], cur_k[:, k0:k0 + klen], cur_v[:, k0:k0 + klen]
                    if use_kernel:
                        # tcgen05 flash attention on this key piece; global positions give the mask
                        blk_out, blk_lse = attn_ops.flash_attention_forward(qq, kk, vv, causal, sm_scale,
                                                                            q_pos0=qpos, k_pos0=kpos)
                    else:
                        blk_out, blk_lse = attn_ops.attention_block(qq, kk, vv, causal, sm_scale,
                                                                    q_offset=qpos, k_offset=kpos)
                    acc[qi] = attn_ops.merge_attention_blocks(acc[qi][0], acc[qi][1], blk_out, blk_lse)
            if step + 1 < n:
                comm.wait()
                cur_k, cur_v = next_k, next_v
        out = torch.cat([o for o, _ in acc], dim=1).to(q.dtype) if len(acc) > 1 else acc[0][0].to(q.dtype)
        lse = torch.cat([l for _, l in acc], dim=2) if len(acc) > 1 else acc[0][1]
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.sm_scale, ctx.causal, ctx.group, ctx.use_kernel, ctx.zigzag = sm_scale, causal, group, use_kernel, zigzag
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, causal, zigzag = ctx.group, ctx.causal, ctx.zigzag
        n, rank = group_size(group), group_rank(group)
        kv_comm = ContextCommunicate("bwd-kv", group=group, send_rank=_ring_peer(group, +1),
                                     recv_rank=_ring_peer(group, -1))
        grad_comm = ContextCommunicate("bwd-dkv", group=group, send_rank=_ring_peer(group, +1),
                                       recv_rank=_ring_peer(group, -1))
        dq = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
        dk_acc = dv_acc = None   # fp32 accumulators travelling with the K/V block they belong to
        cur_k, cur_v = k.contiguous(), v.contiguous()
        s_loc = q.shape[1]
        dout = dout.contiguous()
        q_pieces = shard_pieces(rank, n, s_loc, zigzag)
        for step in range(n):
            if step + 1 < n:
                next_k = kv_comm.send_recv(cur_k)
                next_v = kv_comm.send_recv(cur_v)
                kv_comm.commit()
            src = (rank - step) % n
            bdk = torch.zeros(cur_k.shape, device=q.device, dtype=torch.float32)
            bdv = torch.zeros(cur_v.shape, device=q.device, dtype=torch.float32)
            for q0, qlen, qpos in q_pieces:
                for k0, klen, kpos in shard_pieces(src, n, s_loc, zigzag):
                    if causal and kpos > qpos + qlen - 1:
                        continue
                    qs, ks = slice(q0, q0 + qlen), slice(k0, k0 + klen)
                    args = (dout[:, qs], q[:, qs], cur_k[:, ks], cur_v[:, ks], out[:, qs], lse[:, :, qs].contiguous(),
                            causal, ctx.sm_scale)
                    if ctx.use_kernel:
                        pdq, pdk, pdv = attn_ops.flash_attention_backward(*args, q_pos0=qpos, k_pos0=kpos)
                    else:
                        pdq, pdk, pdv = attn_ops.attention_block_backward(*args, q_offset=qpos, k_offset=kpos)
                    dq[:, qs] += pdq
                    bdk[:, ks] += pdk
                    bdv[:, ks] += pdv
            if step > 0:
                grad_comm.wait()          # accumulators of the block now in hand have arrived
                dk_acc, dv_acc = recv_dk + bdk, recv_dv + bdv
            else:
                dk_acc, dv_acc = bdk, bdv
            # pass the accumulators on with their block; after the last step one more hop brings
            # every block's sum home to its owner
            recv_dk = grad_comm.send_recv(dk_acc)
            recv_dv = grad_comm.send_recv(dv_acc)
            grad_comm.commit()
            if step + 1 < n:
                kv_comm.wait()
                cur_k, cur_v = next_k, next_v
        grad_comm.wait()
        return dq.to(q.dtype), recv_dk.to(k.dtype), recv_dv.to(v.dtype), None, None, None, None


def _ring_peer(group, delta: int) -> int:
    """Global rank of the ring neighbour at distance ``delta`` inside ``group``."""
    import torch.distributed as dist
    n, r = group_size(group), group_rank(group)
    return dist.get_global_rank(group, (r + delta) % n)


#: optional ``ops.fused_cp.CPFused``: K/V exchange and dK/dV reduction through NVLink peer memory
_FUSED_CP = None


def install_fused_cp(cp) -> None:
    """Route causal ring attention of matching shapes through the peer-memory gather (``ops.fused_cp``)."""
    global _FUSED_CP
    _FUSED_CP = cp


def ring_attention_bshd(q, k, v, causal: bool = True, sm_scale=None, group=None, zigzag: bool = False):
    """``zigzag``: the local tokens are chunks r and 2n-1-r of the sequence (see ``shard_pieces``)
    instead of one contiguous slice."""
    group = group if group is not None else pgm.get_pgm().cp_group
    if group_size(group) == 1:
        return attn_ops.attention(q, k, v, causal, sm_scale)
    cp = _FUSED_CP
    if cp is not None and causal and not zigzag and cp.sg.group is group and cp.matches(k) \
            and attn_ops.kernel_supports(q, k) and not attn_ops.reference_ops_forced_():
        from ..ops.fused_cp import gathered_causal_attention
        return gathered_causal_attention(q, k, v, sm_scale, cp)
    return _RingAttention.apply(q, k, v, sm_scale, causal, group, zigzag)


def ring_attention(q, k, v, sm_scale, is_causal, group=None):
    """Reference-layout entry point: q, k, v are ``[b, heads, s_local, d]``; returns the same."""
    out = ring_attention_bshd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, sm_scale, group)
    return out.transpose(1, 2)


# ------------------------------------------------------------------------------------------
# the reference's block-level names (picotron/context_parallel/context_parallel.py:37-323), all in its
# [b, heads, s, d] layout
# ------------------------------------------------------------------------------------------
def ring_attention_forward(q, k, v, sm_scale, is_causal):
    """Attention of the local queries against ONE key/value block: ``(out [b, heads, s, d], log-sum-exp
    [b, heads, s])``; the causal mask, if any, is the diagonal block's."""
    out, lse = attn_ops.attention_block(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, sm_scale)
    return out.transpose(1, 2), lse


def ring_attention_backward(dout, q, k, v, out, softmax_lse, sm_scale, is_causal):
    """Gradients ``(dq, dk, dv)`` of one block's contribution, given the merged output and log-sum-exp."""
    dq, dk, dv = attn_ops.attention_block_backward(dout.transpose(1, 2), q.transpose(1, 2), k.transpose(1, 2),
                                                   v.transpose(1, 2), out.transpose(1, 2), softmax_lse, is_causal,
                                                   sm_scale)
    return tuple(g.transpose(1, 2).to(q.dtype) for g in (dq, dk, dv))


def update_out_and_lse(out, lse, block_out, block_lse, slice_=None):
    """Exact merge of a new block's result into the running ``(out fp32 [b, heads, s, d], lse [b, heads, s,
    1])``; the first call (``out is None``) returns the block itself. ``slice_`` restricts the update to
    a part of the running tensors."""
    block_out = block_out.float()
    block_lse = block_lse.unsqueeze(-1)
    if out is None:
        if slice_ is not None:
            raise RuntimeError("the first block cannot be merged into a slice")
        return block_out, block_lse

    def merged(cur_out, cur_lse):
        new_lse = torch.logaddexp(cur_lse, block_lse)
        return torch.exp(cur_lse - new_lse) * cur_out + torch.exp(block_lse - new_lse) * block_out, new_lse

    if slice_ is None:
        return merged(out, lse)
    out[slice_], lse[slice_] = merged(out[slice_], lse[slice_])
    return out, lse


class RingAttentionFunc:
    """``.apply(q, k, v, sm_scale, is_causal)`` like the reference's autograd function of this name."""

    @staticmethod
    def apply(q, k, v, sm_scale, is_causal):
        return ring_attention(q, k, v, sm_scale, is_causal)


#: the reference keeps a second function for its flash-attention blocks; here the blocks run on the
#: flash kernels of this library whenever the tensors allow, so both names are the same entry point
RingFlashAttentionFunc = RingAttentionFunc


def update_rope_for_context_parallel(cos, sin, cp_rank=None, cp_world_size=None):
    """Slice full-sequence RoPE tables to this rank's positions (context_parallel.py:326-334)."""
    m = pgm.get_pgm()
    cp_rank = m.cp_rank if cp_rank is None else cp_rank
    n = m.cp_world_size if cp_world_size is None else cp_world_size
    s = cos.shape[0]
    assert s % n == 0
    per = s // n
    return cos[cp_rank * per:(cp_rank + 1) * per], sin[cp_rank * per:(cp_rank + 1) * per]


def apply_context_parallel(model, attention: str = None, group=None, seq_length: int = None,
                           zigzag: bool = False):
    """Install ring or Ulysses attention on every layer and offset RoPE positions to this rank's
    slice of the sequence: rank r holds positions ``[r * s_local, (r + 1) * s_local)`` with
    ``s_local = seq_length / cp``. ``seq_length`` is the training sequence length; it defaults to
    the model's ``max_position_embeddings`` (the reference slices its tables by that,
    context_parallel.py:326-334), which is only right when the two are equal. ``zigzag`` (ring
    attention only; the data loader must slice the same way, ``MicroBatchDataLoader(cp_zigzag=True)``)
    gives rank r chunks r and 2n-1-r of the sequence instead, so that causal attention costs every
    rank the same (with contiguous shards rank r computes r+1 blocks and the last rank paces the ring,
    as the reference's README notes, context_parallel/README.md:146-148). Returns the model.

    ``attention`` = None takes the strategy from the ``CP_ATTENTION`` environment variable (the reference's
    switch, read by its model in every forward pass; here it is read once, by this call), default ring.
    The reference's one-argument call ``apply_context_parallel(model)`` therefore does the same job."""
    if attention is None:
        import os
        attention = os.environ.get("CP_ATTENTION", "ring")
    assert attention in ("ring", "ulysses"), f"unknown context-parallel attention {attention!r}"
    m = pgm.get_pgm()
    group = group if group is not None else m.cp_group
    n, rank = group_size(group), group_rank(group)
    if n == 1:
        return model
    if attention == "ulysses":
        from .ulysses import ulysses_attention_bshd

        def core(q, k, v, causal, sm_scale=None):
            return ulysses_attention_bshd(q, k, v, causal, sm_scale, group)
    else:
        def core(q, k, v, causal, sm_scale=None):
            return ring_attention_bshd(q, k, v, causal, sm_scale, group, zigzag=zigzag)
    for layer in model.decoder_layers_iter():
        layer.attention.core = core
    s_total = model.rope.max_positions if seq_length is None else int(seq_length)
    assert s_total <= model.rope.max_positions, \
        f"sequence length {s_total} exceeds max_position_embeddings {model.rope.max_positions}"
    assert s_total % n == 0, "sequence length must be divisible by the context-parallel size"
    assert not (zigzag and attention == "ulysses"), "zigzag sharding applies to ring attention only"
    model.rope.pos_offset = rank * (s_total // n)
    model.rope.pos_pieces = shard_pieces(rank, n, s_total // n, True) if zigzag else None
    model.cp_group = group
    model.cp_attention = attention
    return model
