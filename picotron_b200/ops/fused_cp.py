"""Context-parallel causal attention whose K/V exchange and dK/dV reduction go through NVLink peer
memory instead of a ring of point-to-point messages.

Every rank holds a contiguous sequence shard (picotron/data.py:115-118). Under a causal mask rank r
needs the keys and values of ranks 0..r. Instead of rotating blocks around a ring for ``cp`` steps
(picotron/context_parallel/context_parallel.py:37-68, one attention launch and one merge per step),

* forward: each rank pushes its K and V rows into every peer's gather buffer (one store kernel,
  flags raised when it is done) and meanwhile runs the flash kernel on its own (diagonal) block;
  when the flags of the earlier ranks have arrived, ONE more launch covers all earlier blocks at
  once, and the two partial results are merged by log-sum-exp. Two attention launches per layer
  regardless of ``cp``.
* backward: K/V are gathered again the same way (the buffers are shared by all layers); the flash
  backward runs on the local block and once on all earlier blocks; the dK/dV it produces for
  earlier ranks are stored into those ranks' staging slots (one scatter kernel per tensor) and every
  owner sums its slots in rank order, so the reduction is deterministic.

Buffers are double-buffered by operation count and all ranks wait for all flags of an operation, so
no acknowledgements are needed (a rank cannot start operation n+2 before everyone finished n).
The fp32 dK/dV accumulators of the reference's ring travel as bf16 partial sums here (at most
``cp - 1`` addends per element, summed in fp32).
"""
from __future__ import annotations

import os
from typing import List

import torch

from . import attention as attn_ops
from . import count_launch, ext

GATHER_SLOTS = (30, 31)
SCATTER_SLOTS = (32, 33)


class CPFused:
    def __init__(self, symm_group, batch: int, s_local: int, kv_cols: int):
        """``kv_cols`` = kv_heads * head_dim (width of one K or V row)."""
        self.sg = symm_group
        self.world, self.rank = symm_group.world, symm_group.rank
        self.batch, self.s_local, self.kv_cols = batch, s_local, kv_cols
        self.block_bytes = s_local * kv_cols * 2                       # one rank's rows of one batch element
        self.region_bytes = self.world * self.block_bytes               # all ranks' rows of one batch element
        nbytes = 2 * batch * self.region_bytes                          # K and V
        self.gather = [symm_group.alloc(nbytes) for _ in range(2)]
        self.staging = [symm_group.alloc(nbytes) for _ in range(2)]
        self.n_gather = 0
        self.n_scatter = 0
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))

    def matches(self, k: torch.Tensor) -> bool:
        b, s, h, d = k.shape
        return b == self.batch and s == self.s_local and h * d == self.kv_cols

    def _region(self, which: int, bi: int) -> int:
        return (which * self.batch + bi) * self.region_bytes

    # -- all-gather of K and V by pushing --------------------------------------------------------
    def gather_kv(self, k: torch.Tensor, v: torch.Tensor):
        """Push this rank's rows to every peer. Returns (copy index, slot, epoch of the last push)."""
        c = self.n_gather % 2
        self.n_gather += 1
        slot = GATHER_SLOTS[c]
        epoch = 0
        for which, t in enumerate((k, v)):
            for bi in range(self.batch):
                rows = t[bi].reshape(self.s_local, self.kv_cols)
                if not rows.is_contiguous():
                    rows = rows.contiguous()
                epoch = self.sg.next_epoch(slot)
                ext().push_rows(rows, self.gather[c].peer_ptrs(self._region(which, bi)), self.sg.flags.ptrs,
                                self.world, self.rank, self.s_local, self.kv_cols, slot, epoch, 0, 0)
                count_launch()
        return c, slot, epoch

    def gathered(self, c: int, which: int, num_blocks: int, kv_heads: int, head_dim: int) -> torch.Tensor:
        """View [batch, num_blocks * s_local, kv_heads, head_dim] of the first ``num_blocks`` ranks' rows."""
        full = self.gather[c].view(torch.bfloat16, (self.batch, self.world * self.s_local, kv_heads, head_dim),
                                   self._region(which, 0))
        return full[:, :num_blocks * self.s_local]

    def wait(self, slot: int, epoch: int) -> None:
        self.sg.wait(slot, epoch, self.timeout_ms)

    # -- reduce-scatter of dK and dV ---------------------------------------------------------------
    def reduce_dkv(self, d_earlier: List[torch.Tensor], d_local: List[torch.Tensor]) -> List[torch.Tensor]:
        """``d_earlier[w]``: [batch, rank * s_local, kv_heads, d] gradients this rank computed for the
        blocks of ranks 0..rank-1 (None on rank 0); ``d_local[w]``: its gradient for its own block.
        Returns the complete gradients of the own block (sum over ranks >= own)."""
        c = self.n_scatter % 2
        self.n_scatter += 1
        slot = SCATTER_SLOTS[c]
        epoch = 0
        for which in range(2):
            for bi in range(self.batch):
                epoch = self.sg.next_epoch(slot)
                if self.rank > 0:
                    src = d_earlier[which][bi].reshape(self.rank * self.s_local, self.kv_cols)
                    if not src.is_contiguous():
                        src = src.contiguous()
                else:
                    src = d_local[which][bi].reshape(self.s_local, self.kv_cols)    # not read (no destination)
                    if not src.is_contiguous():
                        src = src.contiguous()
                ext().scatter_rows(src, self.staging[c].peer_ptrs(self._region(which, bi)), self.sg.flags.ptrs,
                                   self.world, self.rank, self.rank, self.s_local, self.kv_cols, slot, epoch, 0)
                count_launch()
        outs = []
        for which in range(2):
            local = d_local[which]
            out = torch.empty_like(local, memory_format=torch.contiguous_format)
            for bi in range(self.batch):
                stg = self.staging[c].view(torch.bfloat16, (self.world, self.s_local, self.kv_cols),
                                           self._region(which, bi))
                add = local[bi].reshape(self.s_local, self.kv_cols)
                if not add.is_contiguous():
                    add = add.contiguous()
                ext().slot_sum_from(stg, self.world, self.rank + 1, self.s_local, self.kv_cols, add,
                                    out[bi].view(self.s_local, self.kv_cols), self.sg.flags.local_ptr, slot, epoch,
                                    self.timeout_ms)
                count_launch()
            outs.append(out)
        return outs


class _GatheredCausalAttention(torch.autograd.Function):
    """q: [b, s_loc, H, d]; k, v: [b, s_loc, Hkv, d] (this rank's shard, positions rank*s_loc ...)."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale, cp: CPFused):
        r, s_loc = cp.rank, cp.s_local
        kvh, d = k.shape[2], k.shape[3]
        c, slot, epoch = cp.gather_kv(k, v)
        # own block while the other ranks' rows are still arriving
        out, lse = attn_ops.flash_attention_forward(q, k, v, True, sm_scale, q_pos0=r * s_loc, k_pos0=r * s_loc)
        cp.wait(slot, epoch)
        if r > 0:
            ke, ve = cp.gathered(c, 0, r, kvh, d), cp.gathered(c, 1, r, kvh, d)
            out2, lse2 = attn_ops.flash_attention_forward(q, ke, ve, False, sm_scale)
            out, lse = attn_ops.merge_attention_blocks(out, lse, out2, lse2)
            out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.sm_scale, ctx.cp = sm_scale, cp
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        cp: CPFused = ctx.cp
        r, s_loc = cp.rank, cp.s_local
        kvh, d = k.shape[2], k.shape[3]
        dout = dout.contiguous()
        c, slot, epoch = cp.gather_kv(k, v)
        dq, dk_l, dv_l = attn_ops.flash_attention_backward(dout, q, k, v, out, lse, True, ctx.sm_scale,
                                                           q_pos0=r * s_loc, k_pos0=r * s_loc)
        cp.wait(slot, epoch)
        d_earlier = [None, None]
        if r > 0:
            ke, ve = cp.gathered(c, 0, r, kvh, d), cp.gathered(c, 1, r, kvh, d)
            dq2, dk_e, dv_e = attn_ops.flash_attention_backward(dout, q, ke, ve, out, lse, False, ctx.sm_scale)
            dq = dq + dq2
            d_earlier = [dk_e, dv_e]
        dk, dv = cp.reduce_dkv(d_earlier, [dk_l, dv_l])
        return dq, dk, dv, None, None


def gathered_causal_attention(q, k, v, sm_scale, cp: CPFused):
    return _GatheredCausalAttention.apply(q, k, v, sm_scale, cp)
