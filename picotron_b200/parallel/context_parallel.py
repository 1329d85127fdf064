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


class _RingAttention(torch.autograd.Function):
    """q: [b, s_loc, H, d]; k, v: [b, s_loc, Hkv, d] (this rank's shard)."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale, causal, group):
        n, rank = group_size(group), group_rank(group)
        s_loc = q.shape[1]
        comm = ContextCommunicate("fwd", group=group, send_rank=_ring_peer(group, +1),
                                  recv_rank=_ring_peer(group, -1))
        out, lse = None, None
        cur_k, cur_v = k.contiguous(), v.contiguous()
        use_kernel = attn_ops.kernel_supports(q, k) and not attn_ops.reference_ops_forced_()
        for step in range(n):
            if step + 1 < n:
                next_k = comm.send_recv(cur_k)
                next_v = comm.send_recv(cur_v)
                comm.commit()
            src = (rank - step) % n          # owner of the block in hand
            if not causal or src <= rank:
                if use_kernel:
                    # tcgen05 flash attention on this key block; global positions give the mask
                    blk_out, blk_lse = attn_ops.flash_attention_forward(q, cur_k, cur_v, causal, sm_scale,
                                                                        q_pos0=rank * s_loc, k_pos0=src * s_loc)
                else:
                    blk_out, blk_lse = attn_ops.attention_block(q, cur_k, cur_v, causal and src == rank, sm_scale,
                                                                q_offset=0, k_offset=0)
                out, lse = attn_ops.merge_attention_blocks(out, lse, blk_out, blk_lse)
            if step + 1 < n:
                comm.wait()
                cur_k, cur_v = next_k, next_v
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.sm_scale, ctx.causal, ctx.group, ctx.use_kernel = sm_scale, causal, group, use_kernel
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, causal = ctx.group, ctx.causal
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
        for step in range(n):
            if step + 1 < n:
                next_k = kv_comm.send_recv(cur_k)
                next_v = kv_comm.send_recv(cur_v)
                kv_comm.commit()
            src = (rank - step) % n
            if not causal or src <= rank:
                if ctx.use_kernel:
                    bdq, bdk, bdv = attn_ops.flash_attention_backward(dout, q, cur_k, cur_v, out, lse, causal,
                                                                      ctx.sm_scale, q_pos0=rank * s_loc,
                                                                      k_pos0=src * s_loc)
                    bdk, bdv = bdk.float(), bdv.float()
                else:
                    bdq, bdk, bdv = attn_ops.attention_block_backward(dout, q, cur_k, cur_v, out, lse,
                                                                      causal and src == rank, ctx.sm_scale)
                dq += bdq
            else:
                bdk = torch.zeros(cur_k.shape, device=q.device, dtype=torch.float32)
                bdv = torch.zeros(cur_v.shape, device=q.device, dtype=torch.float32)
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
        return dq.to(q.dtype), recv_dk.to(k.dtype), recv_dv.to(v.dtype), None, None, None


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


def ring_attention_bshd(q, k, v, causal: bool = True, sm_scale=None, group=None):
    group = group if group is not None else pgm.get_pgm().cp_group
    if group_size(group) == 1:
        return attn_ops.attention(q, k, v, causal, sm_scale)
    cp = _FUSED_CP
    if cp is not None and causal and cp.sg.group is group and cp.matches(k) and attn_ops.kernel_supports(q, k) \
            and not attn_ops.reference_ops_forced_():
        from ..ops.fused_cp import gathered_causal_attention
        return gathered_causal_attention(q, k, v, sm_scale, cp)
    return _RingAttention.apply(q, k, v, sm_scale, causal, group)


def ring_attention(q, k, v, sm_scale, is_causal, group=None):
    """Reference-layout entry point: q, k, v are ``[b, heads, s_local, d]``; returns the same."""
    out = ring_attention_bshd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, sm_scale, group)
    return out.transpose(1, 2)


def update_rope_for_context_parallel(cos, sin, cp_rank=None, cp_world_size=None):
    """Slice full-sequence RoPE tables to this rank's positions (context_parallel.py:326-334)."""
    m = pgm.get_pgm()
    cp_rank = m.cp_rank if cp_rank is None else cp_rank
    n = m.cp_world_size if cp_world_size is None else cp_world_size
    s = cos.shape[0]
    assert s % n == 0
    per = s // n
    return cos[cp_rank * per:(cp_rank + 1) * per], sin[cp_rank * per:(cp_rank + 1) * per]


def apply_context_parallel(model, attention: str = "ring", group=None, seq_length: int = None):
    """Install ring or Ulysses attention on every layer and offset RoPE positions to this rank's
    slice of the sequence: rank r holds positions ``[r * s_local, (r + 1) * s_local)`` with
    ``s_local = seq_length / cp``. ``seq_length`` is the training sequence length; it defaults to
    the model's ``max_position_embeddings`` (the reference slices its tables by that,
    context_parallel.py:326-334), which is only right when the two are equal. Returns the model."""
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
            return ring_attention_bshd(q, k, v, causal, sm_scale, group)
    for layer in model.decoder_layers_iter():
        layer.attention.core = core
    s_total = model.rope.max_positions if seq_length is None else int(seq_length)
    assert s_total <= model.rope.max_positions, \
        f"sequence length {s_total} exceeds max_position_embeddings {model.rope.max_positions}"
    assert s_total % n == 0, "sequence length must be divisible by the context-parallel size"
    model.rope.pos_offset = rank * (s_total // n)
    model.cp_group = group
    model.cp_attention = attention
    return model
