"""Ulysses context parallelism with its all-to-alls done by peer-memory store kernels.

``heads_to_seq`` trades this rank's sequence shard of all heads for the whole sequence of its share
of the heads; ``seq_to_heads`` is the inverse. Each is one kernel that writes directly into the
peers' symmetric buffers in the ``[b, s, h, d]`` layout the attention kernels read (no chunk /
concatenate copies around a library all-to-all, as in picotron/context_parallel/ulysses.py:39-51),
then raises a flag; the receiver waits for all flags and copies the result out of the shared buffer.
The two are each other's backward (ulysses.py:54-67).
"""
from __future__ import annotations

import os

import torch

from . import count_launch, ext

TO_SEQ_SLOTS = (40, 41)
TO_HEADS_SLOTS = (42, 43)


class UlyssesFused:
    def __init__(self, symm_group, batch: int, s_local: int, max_cols: int):
        """``max_cols``: widest row exchanged (query heads * head_dim of one rank before the exchange)."""
        self.sg = symm_group
        self.world, self.rank = symm_group.world, symm_group.rank
        self.batch, self.s_local, self.max_cols = batch, s_local, max_cols
        nbytes = batch * s_local * max_cols * 2
        self.buf_seq = [symm_group.alloc(nbytes) for _ in range(2)]
        self.buf_heads = [symm_group.alloc(nbytes) for _ in range(2)]
        self.n_seq = 0
        self.n_heads = 0
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))

    def matches(self, x: torch.Tensor, seq_sharded: bool) -> bool:
        b, s, h, d = x.shape
        s_loc = s if seq_sharded else s // self.world
        heads_ok = (h % self.world == 0) if seq_sharded else True
        width = h * d if seq_sharded else h * d * self.world
        return b == self.batch and s_loc == self.s_local and heads_ok and width <= self.max_cols and (h * d) % 8 == 0

    def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[b, s_local, H, d] -> [b, world * s_local, H / world, d]"""
        b, s_loc, H, d = x.shape
        h = H // self.world
        c = self.n_seq % 2
        self.n_seq += 1
        slot = TO_SEQ_SLOTS[c]
        epoch = self.sg.next_epoch(slot)
        x = x if x.is_contiguous() else x.contiguous()
        ext().a2a_push(x, self.buf_seq[c].ptrs, self.sg.flags.ptrs, self.world, self.rank, b, s_loc, h * d, True,
                       slot, epoch)
        self.sg.wait(slot, epoch, self.timeout_ms)
        count_launch()
        return self.buf_seq[c].view(torch.bfloat16, (b, self.world * s_loc, h, d)).clone()

    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[b, world * s_local, h, d] -> [b, s_local, world * h, d]"""
        b, s, h, d = x.shape
        s_loc = s // self.world
        c = self.n_heads % 2
        self.n_heads += 1
        slot = TO_HEADS_SLOTS[c]
        epoch = self.sg.next_epoch(slot)
        x = x if x.is_contiguous() else x.contiguous()
        ext().a2a_push(x, self.buf_heads[c].ptrs, self.sg.flags.ptrs, self.world, self.rank, b, s_loc, h * d, False,
                       slot, epoch)
        self.sg.wait(slot, epoch, self.timeout_ms)
        count_launch()
        return self.buf_heads[c].view(torch.bfloat16, (b, s_loc, self.world * h, d)).clone()


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, u: UlyssesFused):
        ctx.u = u
        return u.heads_to_seq(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.u.seq_to_heads(g), None


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, u: UlyssesFused):
        ctx.u = u
        return u.seq_to_heads(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.u.heads_to_seq(g), None


def heads_to_seq(x, u: UlyssesFused):
    return _HeadsToSeq.apply(x, u)


def seq_to_heads(x, u: UlyssesFused):
    return _SeqToHeads.apply(x, u)
