"""Sequence-parallel linears whose collectives are fused into the GEMM kernels.

Column-parallel ("all-gather -> GEMM"): every rank *pushes* its activation shard into the gather
buffer of all ranks over NVLink (``push_rows``; peer stores + one flag per source) and the GEMM
starts on its own rows immediately, loading the other ranks' row blocks as their flags arrive
(``gemm_ex`` with A-side gating). Row-parallel ("GEMM -> reduce-scatter"): the GEMM epilogue
TMA-stores each output row block straight into the owning rank's staging buffer, one slot per
source rank; the owner adds the slots in rank order (``slot_sum``, deterministic) together with
an optional residual. No NCCL call is on either path. They replace
``all_gather_along_seq`` + matmul and matmul + ``reduce_scatter_along_seq`` of
picotron/sequence_parallel/sequence_parallel.py:20-72 (and the chunked P2P overlap of
overlap.py:40-118).

Rows are kept in *rank-major* order between fused ops: row block r of a gathered tensor is rank
r's ``[b, s/tp]`` shard flattened. Per-token ops (SwiGLU, the lm head + loss) run in that order
unchanged; only attention needs ``[b, s, ...]`` and converts with one copy each way.

Buffers alternate between two copies per kind; because every fused op needs data from all
ranks before it completes, no rank can be two ops ahead of another, which makes the second
copy sufficient without acknowledgement flags.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import count_launch, ext
from . import gemm as gemm_ops

BM = 128
GATHER_SLOTS = (0, 1)
SCATTER_SLOTS = (2, 3)
CE_SLOTS = (4, 5)


class PeerStatsExchange:
    """Vocabulary-parallel cross entropy without a collective call: the statistics kernel stores
    each row's (max, sum, target logit) of this rank's vocabulary shard into every rank's
    ``[world, rows, 3]`` table and raises a flag; the loss/gradient kernel waits for all ranks'
    flags and merges the triples itself. Replaces the three all-reduces of
    picotron/tensor_parallel/tp_communications.py:150,160,166."""

    def __init__(self, symm_group, max_rows: int, timeout_ms: int):
        self.sg = symm_group
        self.world, self.rank = symm_group.world, symm_group.rank
        self.max_rows = max_rows
        self.tables = [symm_group.alloc(self.world * max_rows * 3 * 4) for _ in range(2)]
        self.n = 0
        self.timeout_ms = timeout_ms

    def fits(self, rows: int) -> bool:
        return rows <= self.max_rows

    def stats_loss_grad(self, l2, targets, loss, dlogits, scale, vocab_start):
        rows, V = l2.shape
        b = self.n % 2
        self.n += 1
        slot = CE_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        ext().ce_stats_push(l2, l2.stride(0), targets, rows, V, vocab_start, self.tables[b].ptrs,
                            self.sg.flags.ptrs, self.world, self.rank, slot, epoch)
        table = self.tables[b].view(torch.float32, (self.world, rows, 3))
        ext().ce_loss_grad_gathered(l2, l2.stride(0), targets, table, loss, dlogits, dlogits.stride(0), scale, rows,
                                    V, vocab_start, self.sg.flags.local_ptr, self.world, slot, epoch,
                                    self.timeout_ms)
        count_launch(2)


class TPFused:
    def __init__(self, symm_group, m_local: int, max_cols: int):
        self.sg = symm_group
        self.world, self.rank = symm_group.world, symm_group.rank
        self.m_local = m_local
        self.m_full = m_local * self.world
        self.max_cols = max_cols
        self.gather = [symm_group.alloc(self.m_full * max_cols * 2) for _ in range(2)]
        self.staging = [symm_group.alloc(self.world * m_local * max_cols * 2) for _ in range(2)]
        self.n_gather = 0
        self.n_scatter = 0
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))
        self.ce_exchange = PeerStatsExchange(symm_group, self.m_full, self.timeout_ms)

    @staticmethod
    def usable(m_local: int) -> bool:
        return m_local % BM == 0

    # -- all-gather by pushing ----------------------------------------------------------------
    def gather_push(self, x2: torch.Tensor):
        """x2: [m_local, K] contiguous bf16. Returns (gathered view [m_full, K], slot, epoch)."""
        m, k = x2.shape
        assert m == self.m_local and k <= self.max_cols
        b = self.n_gather % 2
        self.n_gather += 1
        slot = GATHER_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        ext().push_rows(x2, self.gather[b].ptrs, self.sg.flags.ptrs, self.world, self.rank, m, k, slot, epoch)
        count_launch()
        return self.gather[b].view(torch.bfloat16, (self.m_full, k)), slot, epoch

    def gated_gemm(self, a_buf, weight, slot, epoch, b_mn_major: bool, n_out: int, out=None):
        """out[m_full, n_out] = a_buf @ op(weight), loading A row blocks as their flags arrive."""
        m, k = a_buf.shape
        if out is None:
            out = torch.empty((m, n_out), device=a_buf.device, dtype=torch.bfloat16)
        ext().gemm_ex(a_buf, weight, out, m, n_out, k, a_buf.stride(0), weight.stride(0), out.stride(0), False,
                      b_mn_major, 0, 0, self.sg.flags.local_ptr, slot, epoch, self.m_local, self.rank, [], 0,
                      self.rank * self.m_local, self.timeout_ms)
        count_launch()
        return out

    def wait_gather(self, slot, epoch):
        self.sg.wait(slot, epoch, self.timeout_ms)

    # -- reduce-scatter through the GEMM epilogue ------------------------------------------------
    def scatter_gemm(self, a2, weight, b_mn_major: bool, n_out: int):
        """Partial product a2[m_full, K] @ op(weight) stored row block r -> rank r's staging slot for
        this rank; raises this rank's flag afterwards. Returns (buffer index, slot, epoch)."""
        m, k = a2.shape
        assert m == self.m_full and n_out <= self.max_cols
        b = self.n_scatter % 2
        self.n_scatter += 1
        slot = SCATTER_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        off = self.rank * self.m_local * n_out * 2
        ext().gemm_ex(a2, weight, None, m, n_out, k, a2.stride(0), weight.stride(0), n_out, False, b_mn_major, 0,
                      0, 0, 0, 0, 0, 0, self.staging[b].peer_ptrs(off), self.m_local,
                      ((self.rank + 1) % self.world) * self.m_local, self.timeout_ms)
        self.sg.signal(slot, epoch)
        count_launch()
        return b, slot, epoch

    def scatter_sum(self, b, slot, epoch, n_out: int, addend: Optional[torch.Tensor] = None):
        out = torch.empty((self.m_local, n_out), device=self.sg.device, dtype=torch.bfloat16)
        stg = self.staging[b].view(torch.bfloat16, (self.world, self.m_local, n_out))
        ext().slot_sum(stg, self.world, self.m_local, n_out, addend, out, self.sg.flags.local_ptr, slot, epoch,
                       self.timeout_ms)
        count_launch()
        return out


def to_rank_major(x: torch.Tensor, world: int) -> torch.Tensor:
    """[b, s, C] -> [world*b*(s/world), C] with row block r = sequence chunk r of every batch row."""
    b, s, c = x.shape
    if b == 1:
        return x.reshape(s, c)
    return x.view(b, world, s // world, c).transpose(0, 1).reshape(b * s, c)


def from_rank_major(x2: torch.Tensor, world: int, b: int) -> torch.Tensor:
    """Inverse of ``to_rank_major``: [world*b*s_loc, C] -> [b, world*s_loc, C]."""
    m, c = x2.shape
    s_loc = m // (world * b)
    if b == 1:
        return x2.view(1, m, c)
    return x2.view(world, b, s_loc, c).transpose(0, 1).reshape(b, world * s_loc, c)


class _AGLinearFused(torch.autograd.Function):
    """y = gather(x) @ cat(weights).T. x: [b, s_loc, K] shard; returns rank-major [m_full, N] or,
    with ``batch_major``, [b, s, N]."""

    @staticmethod
    def forward(ctx, x, tp: TPFused, ws, batch_major, *params):
        b, s_loc, k = x.shape
        x2 = x.reshape(b * s_loc, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        buf, slot, epoch = tp.gather_push(x2)
        if ws.fused_weight is not None:
            y = tp.gated_gemm(buf, ws.fused_weight, slot, epoch, False, ws.out_features)
        else:
            y = torch.empty((tp.m_full, ws.out_features), device=x.device, dtype=x.dtype)
            col = 0
            for w in ws.params:
                tp.gated_gemm(buf, w, slot, epoch, False, w.shape[0], out=y[:, col:col + w.shape[0]])
                col += w.shape[0]
        ctx.save_for_backward(x2)
        ctx.tp, ctx.ws, ctx.batch_major, ctx.shape = tp, ws, batch_major, (b, s_loc, k)
        return from_rank_major(y, tp.world, b) if batch_major else y

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        tp, ws = ctx.tp, ctx.ws
        b, s_loc, k = ctx.shape
        dy2 = to_rank_major(dy, tp.world) if ctx.batch_major else dy
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # re-gather the input for the weight gradient first so the pushes overlap the dgrad GEMM
        buf, slot, epoch = tp.gather_push(x2)
        dx = None
        if ws.fused_weight is not None:
            pending = tp.scatter_gemm(dy2, ws.fused_weight, True, k)
        else:
            # separate weights: each partial product is reduced before the next one reuses the
            # staging buffers (only two copies exist)
            pending = None
            col = 0
            for w in ws.params:
                sb, sslot, sepoch = tp.scatter_gemm(dy2[:, col:col + w.shape[0]], w, True, k)
                dx = tp.scatter_sum(sb, sslot, sepoch, k, addend=dx)
                col += w.shape[0]
        tp.wait_gather(slot, epoch)
        _, grads = gemm_ops.backward_all(dy2, buf, ws, need_dx=False)
        if pending is not None:
            dx = tp.scatter_sum(*pending, k)
        return (dx.view(b, s_loc, k), None, None, None, *grads)


class _LinearRSFused(torch.autograd.Function):
    """y_shard = reduce_scatter(x @ w.T) (+ addend). x: rank-major [m_full, K_loc] or [b, s, K_loc]."""

    @staticmethod
    def forward(ctx, x, w, tp: TPFused, batch_major_in, shard_bs, addend):
        b, s_loc = shard_bs
        x2 = to_rank_major(x, tp.world) if batch_major_in else x
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        n = w.shape[0]
        sb, slot, epoch = tp.scatter_gemm(x2, w, False, n)
        add2 = None
        if addend is not None:
            add2 = addend.reshape(b * s_loc, n)
            if not add2.is_contiguous():
                add2 = add2.contiguous()
        y = tp.scatter_sum(sb, slot, epoch, n, addend=add2)
        ctx.save_for_backward(x2, w)
        ctx.tp, ctx.batch_major_in, ctx.b, ctx.has_addend = tp, batch_major_in, b, addend is not None
        return y.view(b, s_loc, n)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        tp = ctx.tp
        n = w.shape[0]
        dy2 = dy.reshape(-1, n)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        buf, slot, epoch = tp.gather_push(dy2)
        dx2 = tp.gated_gemm(buf, w, slot, epoch, True, w.shape[1])
        tp.wait_gather(slot, epoch)
        dw = gemm_ops.wgrad_into(w, buf, x2)
        dx = from_rank_major(dx2, tp.world, ctx.b) if ctx.batch_major_in else dx2
        return dx, dw, None, None, None, (dy if ctx.has_addend else None)


class _EmbeddingRSFused(torch.autograd.Function):
    """Vocabulary-parallel embedding under sequence parallelism without a collective call: every
    rank looks its vocabulary shard up for the whole sequence (rows of ids it does not own are
    zero), stores row block o into its slot of rank o's staging buffer and sums the slots it
    received; backward gathers the output gradient by pushing and scatters it into the table's
    gradient. ids: [b, s] (full sequence); returns [b, s/tp, H]."""

    @staticmethod
    def forward(ctx, ids, weight, vocab_start, tp: TPFused):
        b, s = ids.shape
        V, H = weight.shape
        ids_rm = ids.view(b, tp.world, s // tp.world).transpose(0, 1).reshape(-1).contiguous()
        part = torch.empty((tp.m_full, H), device=weight.device, dtype=weight.dtype)
        ext().embedding_fwd(weight, ids_rm, part, tp.m_full, H, V, vocab_start)
        sb = tp.n_scatter % 2
        tp.n_scatter += 1
        slot = SCATTER_SLOTS[sb]
        epoch = tp.sg.next_epoch(slot)
        ext().scatter_rows(part, tp.staging[sb].ptrs, tp.sg.flags.ptrs, tp.world, tp.rank, tp.world, tp.m_local, H,
                           slot, epoch)
        count_launch(2)
        y = tp.scatter_sum(sb, slot, epoch, H)
        ctx.save_for_backward(ids_rm, weight)
        ctx.tp, ctx.vocab_start, ctx.shape = tp, vocab_start, (b, s // tp.world, H)
        return y.view(b, s // tp.world, H)

    @staticmethod
    def backward(ctx, dy):
        ids_rm, weight = ctx.saved_tensors
        tp = ctx.tp
        V, H = weight.shape
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        buf, slot, epoch = tp.gather_push(dy2)
        tp.wait_gather(slot, epoch)
        main_grad = getattr(weight, "main_grad", None)
        acc = main_grad if main_grad is not None else torch.zeros((V, H), device=weight.device, dtype=torch.float32)
        ext().embedding_bwd(buf, ids_rm, acc, tp.m_full, H, V, ctx.vocab_start)
        count_launch()
        if main_grad is not None:
            hook = getattr(weight, "grad_ready_hook", None)
            if hook is not None:
                hook()
            return None, None, None, None
        return None, acc.to(weight.dtype), None, None


def embedding_rs(ids, weight, vocab_start: int, tp: TPFused):
    return _EmbeddingRSFused.apply(ids, weight, vocab_start, tp)


def ag_linear(x, tp: TPFused, mods, batch_major: bool):
    ws = gemm_ops.WeightSet.of(mods)
    return _AGLinearFused.apply(x, tp, ws, batch_major, *ws.params)


def linear_rs(x, w, tp: TPFused, batch_major_in: bool, shard_bs, addend=None):
    return _LinearRSFused.apply(x, w, tp, batch_major_in, shard_bs, addend)
