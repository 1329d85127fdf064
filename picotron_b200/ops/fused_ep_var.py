"""Dropless expert-parallel dispatch and combine through NVLink peer memory, laid out on the device.

The variable-size exchange of the reference (picotron/expert_parallel/expert_parallel.py:260-269,
383-400: split sizes by ``all_to_all_single`` followed by ``.tolist()`` on the host, then two
``all_to_all_single`` calls with those splits) becomes:

1. every rank publishes its per-expert row counts into all peers' count tables (one store kernel);
2. one small kernel derives the whole layout from the ``[ep, E]`` table: where each outgoing block
   lands in the receiver's expert-major buffer, the receiver's expert segments padded to 128-row
   tiles (``seg_start`` / ``tile_group`` — exactly what the grouped expert GEMM reads from device
   memory), and the way back;
3. the rows are stored straight into the peers' buffers at those offsets; the outputs return the
   same way into the sender's expert-sorted order.

Nothing is copied to the host, no row is dropped and no capacity is needed; the receive buffer holds
``slack`` times the average load of a rank (a load beyond that is reported as an error, never written
out of bounds). Dispatch and return are each other's backward.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from . import count_launch, ext
from .fused_ep import PeerLoadSum
from .grouped_gemm import GroupLayout

COUNT_SLOTS = (50, 51)
DISPATCH_SLOTS = (52, 53)
RETURN_SLOTS = (54, 55)


@dataclass
class VarPlan:
    send_blocks: torch.Tensor      # [E, 4] int32
    return_blocks: torch.Tensor    # [ep * L, 4] int32
    seg_start: torch.Tensor        # [L + 1] int32
    seg_len: torch.Tensor          # [L] int32
    layout: GroupLayout            # device-side layout of the receive buffer for the grouped GEMM


class EPVarFused(PeerLoadSum):
    def __init__(self, symm_group, num_local_experts: int, dim: int, rows_per_rank: int, slack: float = 1.5,
                 fp8_dispatch: bool = False):
        """``fp8_dispatch``: forward dispatch rows travel as FP8 E4M3 with 1x128 block scales (quantised in
        the send kernel, dequantised at the receiver); gradients and the return path stay bf16, like the
        straight-through backward of picotron/expert_parallel/ep_communications.py:59-118."""
        self.sg = symm_group
        self.ep, self.rank = symm_group.world, symm_group.rank
        self.L, self.d = num_local_experts, dim
        self.E = self.ep * self.L
        self.rows_per_rank = rows_per_rank
        self.max_rows = (int(slack * rows_per_rank) + self.L * 128 + 127) // 128 * 128
        self.counts_buf = [symm_group.alloc(self.ep * self.E * 4) for _ in range(2)]
        self.recv_buf = [symm_group.alloc(self.max_rows * dim * 2) for _ in range(2)]
        self.ret_buf = [symm_group.alloc(rows_per_rank * dim * 2) for _ in range(2)]
        self.fp8 = bool(fp8_dispatch) and dim % 256 == 0
        self.q_buf = [symm_group.alloc(self.max_rows * dim) for _ in range(2)] if self.fp8 else []
        self.q_scales = [symm_group.alloc(self.max_rows * (dim // 128) * 4) for _ in range(2)] if self.fp8 else []
        for b in self.counts_buf + self.recv_buf + self.ret_buf + self.q_buf + self.q_scales:
            b.local.zero_()
        self.n = {"count": 0, "dispatch": 0, "return": 0}
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))
        torch.cuda.synchronize()
        self.sg.barrier()

    def _next(self, kind: str, slots):
        c = self.n[kind] % 2
        self.n[kind] += 1
        return c, slots[c], self.sg.next_epoch(slots[c])

    def plan(self, counts: torch.Tensor) -> VarPlan:
        """counts: [E] int32 (device), rows of this rank per global expert."""
        assert counts.dtype == torch.int32 and counts.numel() == self.E
        c, slot, epoch = self._next("count", COUNT_SLOTS)
        e = ext()
        row = counts.contiguous().view(torch.bfloat16).view(1, 2 * self.E)     # raw bytes of the int32 row
        e.push_rows(row, self.counts_buf[c].ptrs, self.sg.flags.ptrs, self.ep, self.rank, 1, 2 * self.E, slot, epoch,
                    0, 0)
        self.sg.wait(slot, epoch, self.timeout_ms)
        table = self.counts_buf[c].view(torch.int32, (self.ep, self.E))
        dev = counts.device
        send_blocks = torch.empty((self.E, 4), device=dev, dtype=torch.int32)
        return_blocks = torch.empty((self.ep * self.L, 4), device=dev, dtype=torch.int32)
        seg_start = torch.empty(self.L + 1, device=dev, dtype=torch.int32)
        seg_len = torch.empty(self.L, device=dev, dtype=torch.int32)
        tile_group = torch.empty(self.max_rows // 128, device=dev, dtype=torch.int32)
        e.ep_var_layout(table, self.ep, self.L, self.rank, self.max_rows, send_blocks, return_blocks, seg_start,
                        seg_len, tile_group)
        count_launch(3)
        layout = GroupLayout(self.L, self.max_rows, seg_start, tile_group, None)
        return VarPlan(send_blocks, return_blocks, seg_start, seg_len, layout)

    def dispatch(self, rows_sorted: torch.Tensor, plan: VarPlan, quant: bool = False) -> torch.Tensor:
        """[rows_per_rank, d] in this rank's expert-sorted order -> [max_rows, d] padded expert-major
        rows of the local experts (padding rows zero; rows past the last segment are unspecified)."""
        c, slot, epoch = self._next("dispatch", DISPATCH_SLOTS)
        e = ext()
        if quant and self.fp8:
            e.ep_var_exchange(rows_sorted, None, 1, plan.send_blocks, self.E, self.q_buf[c].ptrs,
                              self.q_scales[c].ptrs, self.sg.flags.ptrs, self.ep, self.rank, self.d, True, slot, epoch)
            self.sg.wait(slot, epoch, self.timeout_ms)
            out = torch.empty((self.max_rows, self.d), device=rows_sorted.device, dtype=torch.bfloat16)
            e.ep_var_dequant(self.q_buf[c].view(torch.uint8, (self.max_rows, self.d)),
                             self.q_scales[c].view(torch.float32, (self.max_rows, self.d // 128)), out,
                             plan.seg_start[self.L:], self.max_rows, self.d)
            e.ep_var_zero_padding(out, plan.seg_start, plan.seg_len, self.L, self.d)
            count_launch(4)
            return out
        e.ep_var_exchange(rows_sorted, None, 1, plan.send_blocks, self.E, self.recv_buf[c].ptrs, [],
                          self.sg.flags.ptrs, self.ep, self.rank, self.d, False, slot, epoch)
        self.sg.wait(slot, epoch, self.timeout_ms)
        buf = self.recv_buf[c].view(torch.bfloat16, (self.max_rows, self.d))
        out = torch.empty((self.max_rows, self.d), device=rows_sorted.device, dtype=torch.bfloat16)
        e.ep_var_copy_rows(buf, out, plan.seg_start[self.L:], self.max_rows, self.d)   # only the rows in use
        e.ep_var_zero_padding(out, plan.seg_start, plan.seg_len, self.L, self.d)
        count_launch(4)
        return out

    def give_back(self, rows_padded: torch.Tensor, plan: VarPlan) -> torch.Tensor:
        """[max_rows, d] padded expert-major rows -> [rows_per_rank, d] in the senders' sorted order."""
        c, slot, epoch = self._next("return", RETURN_SLOTS)
        ext().ep_var_exchange(rows_padded, None, 1, plan.return_blocks, self.ep * self.L, self.ret_buf[c].ptrs, [],
                              self.sg.flags.ptrs, self.ep, self.rank, self.d, False, slot, epoch)
        self.sg.wait(slot, epoch, self.timeout_ms)
        count_launch(2)
        return self.ret_buf[c].view(torch.bfloat16, (self.rows_per_rank, self.d)).clone()


class _VarDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows_sorted, plan: VarPlan, epv: EPVarFused):
        ctx.plan, ctx.epv = plan, epv
        return epv.dispatch(rows_sorted.contiguous(), plan, quant=True)

    @staticmethod
    def backward(ctx, g):
        return ctx.epv.give_back(g.contiguous(), ctx.plan), None, None


class _VarReturn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows_padded, plan: VarPlan, epv: EPVarFused):
        ctx.plan, ctx.epv = plan, epv
        return epv.give_back(rows_padded.contiguous(), plan)

    @staticmethod
    def backward(ctx, g):
        return ctx.epv.dispatch(g.contiguous(), ctx.plan), None, None


def var_dispatch(rows_sorted, plan: VarPlan, epv: EPVarFused):
    return _VarDispatch.apply(rows_sorted, plan, epv)


def var_return(rows_padded, plan: VarPlan, epv: EPVarFused):
    return _VarReturn.apply(rows_padded, plan, epv)


def var_layout_ref(counts_table, L: int, my_rank: int, max_rows: int):
    """Plain Python restatement of the layout kernel (test oracle). ``counts_table``: [ep][E] integers.
    Returns (send_blocks [E][4], return_blocks [ep*L][4], seg_start [L+1], seg_len [L], tile_group)."""
    ep = len(counts_table)
    E = ep * L
    pad = lambda n: (n + 127) // 128 * 128      # noqa: E731
    send = []
    for e in range(E):
        r, l = divmod(e, L)
        seg = 0
        for l2 in range(l):
            t = sum(counts_table[s][r * L + l2] for s in range(ep))
            if seg + pad(t) <= max_rows:
                seg += pad(t)
        total = sum(counts_table[s][e] for s in range(ep))
        before = sum(counts_table[s][e] for s in range(my_rank))
        fits = seg + pad(total) <= max_rows
        send.append([counts_table[my_rank][e] if fits else 0, sum(counts_table[my_rank][:e]), r,
                     seg + before if fits else 0])
    ret, seg_start, seg_len, seg = [], [], [], 0
    ret = [[0, 0, 0, 0] for _ in range(ep * L)]
    for l in range(L):
        e = my_rank * L + l
        total = sum(counts_table[s][e] for s in range(ep))
        fits = seg + pad(total) <= max_rows
        seg_start.append(seg)
        seg_len.append(total if fits else 0)
        within = 0
        for s in range(ep):
            c = counts_table[s][e]
            ret[s * L + l] = [c if fits else 0, seg + within, s, sum(counts_table[s][:e])]
            within += c
        if fits:
            seg += pad(total)
    seg_start.append(seg)
    tiles = []
    for t in range(max_rows // 128):
        row, g = t * 128, -1
        if row < seg:
            for l in range(L):
                if seg_start[l] <= row < seg_start[l + 1]:
                    g = l
        tiles.append(g)
    return send, ret, seg_start, seg_len, tiles
