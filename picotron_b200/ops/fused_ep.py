"""Expert-parallel dispatch / combine through NVLink peer memory (fixed-capacity layout).

``EPFused`` owns the symmetric receive slabs of one expert-parallel group. ``dispatch`` sends
every (expert, slot) row of this rank — quantised on the fly to FP8 E4M3 with 1x128 block scales
when asked — straight into the slab of the rank that owns the expert, where it arrives already
grouped ``[local expert][source rank][slot]`` (so the experts run on fixed-size batches without
any regrouping); ``combine`` pushes the expert outputs back to their sources, where they arrive
indexed by global expert and slot. Both are autograd functions whose backward is the opposite
exchange. They replace the equal-split ``all_to_all`` calls (and the separate FP8 payload / scale
exchanges) of picotron/expert_parallel/capacity_moe.py:143-173 and ep_communications.py:94-98.

Two copies of each slab alternate between calls; every exchange needs data from all ranks before
it completes, so no rank can run two exchanges ahead of another.
"""
from __future__ import annotations

import os

import torch

from . import count_launch, ext

EXPERT_SLOTS = (20, 21)   # flags of exchanges that land in the expert-major slab
SOURCE_SLOTS = (22, 23)   # flags of exchanges that land in the source-major slab
LOAD_SLOTS = (24, 25)     # flags of the per-expert load tables


class PeerLoadSum:
    """Sum of small per-rank integer rows over the group through peer memory (needs ``sg``, ``ep``,
    ``rank``, ``timeout_ms``)."""

    n_load = 0
    load_tables = None                   # number of experts -> two [ep, E] int32 tables in symmetric memory

    def sum_over_ranks(self, counts: torch.Tensor) -> torch.Tensor:
        """counts: [E] int32 on the device. Returns their sum over the expert-parallel group as fp32 [E],
        without a collective call: every rank stores its row into all peers' ``[ep, E]`` table and adds the
        rows it received (the load all-reduce of picotron/expert_parallel/expert_parallel.py:205-212).
        Static shapes, nothing read on the host: safe inside a CUDA graph. The tables are created by
        the first call, which must therefore be an eager one made by every rank."""
        E = counts.numel()
        assert counts.dtype == torch.int32 and (E * 4) % 16 == 0
        if self.load_tables is None:
            self.load_tables = {}
        tabs = self.load_tables.get(E)
        if tabs is None:
            assert not torch.cuda.is_current_stream_capturing(), "the first load sum must run eagerly"
            tabs = self.load_tables[E] = [self.sg.alloc(self.ep * E * 4) for _ in range(2)]
            for t in tabs:
                t.local.zero_()
            torch.cuda.synchronize()
            self.sg.barrier()
        b = self.n_load % 2
        self.n_load += 1
        slot = LOAD_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        row = counts.contiguous().view(torch.bfloat16).view(1, 2 * E)          # raw bytes of the int32 row
        ext().push_rows(row, tabs[b].ptrs, self.sg.flags.ptrs, self.ep, self.rank, 1, 2 * E, slot, epoch, 0, 0)
        count_launch()
        self.sg.wait(slot, epoch, self.timeout_ms)
        return tabs[b].view(torch.int32, (self.ep, E)).sum(dim=0).float()


class EPFused(PeerLoadSum):
    def __init__(self, symm_group, num_local_experts: int, capacity: int, dim: int):
        self.sg = symm_group
        self.ep, self.rank = symm_group.world, symm_group.rank
        self.L, self.C, self.d = num_local_experts, capacity, dim
        rows = self.ep * self.L * self.C
        self.rows = rows
        self.expert_slab = [symm_group.alloc(rows * dim * 2) for _ in range(2)]       # bf16 or fp8 payload
        self.expert_scales = [symm_group.alloc(rows * max(1, dim // 128) * 4) for _ in range(2)]
        self.source_slab = [symm_group.alloc(rows * dim * 2) for _ in range(2)]
        self.n_expert = 0
        self.n_source = 0
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))

    def _next(self, kind: str):
        if kind == "expert":
            b = self.n_expert % 2
            self.n_expert += 1
            slot = EXPERT_SLOTS[b]
        else:
            b = self.n_source % 2
            self.n_source += 1
            slot = SOURCE_SLOTS[b]
        return b, slot, self.sg.next_epoch(slot)

    # expert-major result [L, ep*C, d]
    def dispatch_rows(self, tokens, row_of_slot, top_k: int, quant: bool):
        b, slot, epoch = self._next("expert")
        e = ext()
        e.ep_dispatch(tokens, row_of_slot, top_k, self.expert_slab[b].ptrs, self.expert_scales[b].ptrs,
                      self.sg.flags.ptrs, self.ep, self.rank, self.L, self.C, self.d, quant, slot, epoch)
        count_launch()
        if quant:
            out = torch.empty((self.rows, self.d), device=tokens.device, dtype=torch.bfloat16)
            e.ep_dequant(self.expert_slab[b].view(torch.uint8, (self.rows, self.d)),
                         self.expert_scales[b].view(torch.float32, (self.rows, self.d // 128)), out, self.rows, self.d,
                         self.sg.flags.local_ptr, self.ep, slot, epoch, self.timeout_ms)
            count_launch()
        else:
            self.sg.wait(slot, epoch, self.timeout_ms)
            out = self.expert_slab[b].view(torch.bfloat16, (self.rows, self.d)).clone()
        return out.view(self.L, self.ep * self.C, self.d)

    def to_expert_major(self, src_rows):
        """[E*C, d] at the sources -> [L, ep*C, d] at the expert owners (no quantisation)."""
        b, slot, epoch = self._next("expert")
        ext().ep_block_exchange(src_rows, self.expert_slab[b].ptrs, self.sg.flags.ptrs, self.ep, self.rank, self.L,
                                self.C, self.d, True, slot, epoch)
        count_launch()
        self.sg.wait(slot, epoch, self.timeout_ms)
        return self.expert_slab[b].view(torch.bfloat16, (self.rows, self.d)).clone().view(self.L, self.ep * self.C, self.d)

    def to_source_major(self, expert_rows):
        """[L, ep*C, d] at the expert owners -> [E*C, d] at the sources."""
        b, slot, epoch = self._next("source")
        ext().ep_block_exchange(expert_rows, self.source_slab[b].ptrs, self.sg.flags.ptrs, self.ep, self.rank, self.L,
                                self.C, self.d, False, slot, epoch)
        count_launch()
        self.sg.wait(slot, epoch, self.timeout_ms)
        return self.source_slab[b].view(torch.bfloat16, (self.rows, self.d)).clone()


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, row_of_slot, top_k, epf: EPFused, quant, idx, pos):
        ctx.epf, ctx.top_k = epf, top_k
        ctx.routed = idx is not None and pos is not None and epf.d % 8 == 0
        ctx.save_for_backward(row_of_slot, *((idx, pos) if ctx.routed else ()))
        ctx.num_tokens = tokens.shape[0]
        return epf.dispatch_rows(tokens.contiguous(), row_of_slot, top_k, quant)

    @staticmethod
    def backward(ctx, d_expert):
        row_of_slot = ctx.saved_tensors[0]
        epf = ctx.epf
        d_slots = epf.to_source_major(d_expert.contiguous().view(epf.rows, epf.d))     # [E*C, d]
        if ctx.routed:
            # a token's gradient is the sum over the slots its k routed copies took: the weighted-sum
            # kernel of the combine with unit weights (fixed order, no atomics, bf16 reads)
            idx, pos = ctx.saved_tensors[1:]
            d_tokens = torch.empty((ctx.num_tokens, epf.d), device=d_expert.device, dtype=torch.bfloat16)
            ones = torch.ones(idx.shape, device=d_expert.device, dtype=torch.float32)
            ext().moe_combine(d_slots, idx, pos, ones, d_tokens, ctx.top_k, epf.C)
            count_launch()
            return d_tokens, None, None, None, None, None, None
        valid = row_of_slot >= 0
        tok = torch.div(row_of_slot.clamp_min(0), ctx.top_k, rounding_mode="floor").long()
        d_tokens = torch.zeros((ctx.num_tokens, epf.d), device=d_expert.device, dtype=torch.float32)
        d_tokens.index_add_(0, tok, d_slots.float() * valid.unsqueeze(1))
        return d_tokens.to(d_expert.dtype), None, None, None, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, epf: EPFused):
        ctx.epf = epf
        return epf.to_source_major(expert_out.contiguous().view(epf.rows, epf.d))

    @staticmethod
    def backward(ctx, d_back):
        epf = ctx.epf
        return epf.to_expert_major(d_back.contiguous()), None


def dispatch(tokens, row_of_slot, top_k, epf: EPFused, quant: bool, idx=None, pos=None):
    """``idx`` [T, k] / ``pos`` [T, k] (int32, optional): the routing that built ``row_of_slot``; with them
    the backward pass gathers a token's gradient from its slots in one kernel."""
    if idx is not None and not (idx.dtype == torch.int32 and pos.dtype == torch.int32 and idx.is_contiguous()
                                and pos.is_contiguous() and tokens.dtype == torch.bfloat16):
        idx = pos = None
    return _DispatchFn.apply(tokens, row_of_slot, top_k, epf, quant, idx, pos)


def combine(expert_out, epf: EPFused):
    return _CombineFn.apply(expert_out, epf)
