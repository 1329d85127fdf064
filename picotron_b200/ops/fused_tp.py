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

Gathered tensors are ordinary ``[b, s, C]`` tensors: the kernels know that a shard is ``b`` pieces
of ``s/tp`` rows and address piece ``(batch, rank)`` at its place in the full sequence (push, GEMM
tile order and flag gating, scattering epilogue all work on that piece geometry), so no layout
conversion copies surround attention or the loss.

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
KEPT_SLOT0 = 16            # flag slots 16 .. 16 + (number of kept gather buffers) - 1
MAX_KEPT = 224


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
    def __init__(self, symm_group, m_local: int, max_cols: int, s_local: Optional[int] = None):
        """``m_local`` rows per rank (micro-batch x sequence shard), made of pieces of ``s_local`` rows
        (the sequence shard of one batch row; default: one piece)."""
        self.sg = symm_group
        self.world, self.rank = symm_group.world, symm_group.rank
        self.m_local = m_local
        self.s_local = m_local if s_local is None else s_local
        assert m_local % self.s_local == 0 and self.s_local % BM == 0
        self.m_full = m_local * self.world
        self.max_cols = max_cols
        self.gather = [symm_group.alloc(self.m_full * max_cols * 2) for _ in range(2)]
        self.staging = [symm_group.alloc(self.world * m_local * max_cols * 2) for _ in range(2)]
        self.n_gather = 0
        self.n_scatter = 0
        self.timeout_ms = int(os.environ.get("PICO_COMM_TIMEOUT_MS", "20000"))
        self.ce_exchange = PeerStatsExchange(symm_group, self.m_full, self.timeout_ms)
        # Pushes run on their own stream so that they overlap the GEMM that consumes the gathered
        # rows: the GEMM starts on this rank's rows at once and picks the other ranks' row blocks
        # up as their flags arrive. PICO_TP_COMM_STREAM=0 keeps everything on one stream.
        self.comm_stream = torch.cuda.Stream(device=symm_group.device) \
            if os.environ.get("PICO_TP_COMM_STREAM", "1") != "0" else None
        self._pushing = []        # sources of pushes still in flight on the comm stream
        # Gathered inputs kept for the backward pass: the i-th column-parallel gather of a micro-batch
        # lands in its own symmetric buffer, which the weight-gradient GEMM reads later, so the backward
        # pass gathers nothing again. Needs one micro-batch in flight at a time (no pipeline
        # parallelism) and ``begin_micro_batch()`` before every forward pass; off by default.
        self.keep_gathered = False
        self.kept = []
        self._kept_idx = 0

    @staticmethod
    def usable(m_local: int, s_local: Optional[int] = None) -> bool:
        s_local = m_local if s_local is None else s_local
        return s_local % BM == 0 and m_local % s_local == 0

    def begin_micro_batch(self):
        """Start of a forward pass (engine). With kept gather buffers: a peer that already finished its
        backward pass must not push the next micro-batch's first rows while this rank's last
        weight-gradient GEMM still reads that buffer, hence a barrier over the group."""
        self._kept_idx = 0
        if self.keep_gathered:
            self.join()
            self.sg.barrier()

    # -- all-gather by pushing ----------------------------------------------------------------
    def gather_push(self, x2: torch.Tensor, keep: bool = False):
        """x2: [m_local, K] contiguous bf16. Returns (gathered view [m_full, K], slot, epoch). ``keep``:
        use this micro-batch's next kept buffer (valid until the same call of the next micro-batch)
        when ``keep_gathered`` is on; the returned view is then safe to hold for the backward pass."""
        m, k = x2.shape
        assert m == self.m_local and k <= self.max_cols
        if keep and self.keep_gathered:
            i = self._kept_idx
            self._kept_idx += 1
            if i == len(self.kept):
                assert i < MAX_KEPT, "too many kept gather buffers for the flag table"
                assert not torch.cuda.is_current_stream_capturing(), \
                    "kept gather buffers are created by an eager forward pass before any graph capture"
                self.kept.append(self.sg.alloc(self.m_full * self.max_cols * 2))
            target, slot = self.kept[i], KEPT_SLOT0 + i
        else:
            b = self.n_gather % 2
            self.n_gather += 1
            target, slot = self.gather[b], GATHER_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        view = target.view(torch.bfloat16, (self.m_full, k))
        sl = self.s_local
        if self.comm_stream is None:
            ext().push_rows(x2, target.ptrs, self.sg.flags.ptrs, self.world, self.rank, m, k, slot, epoch, 0, sl)
        else:
            self.comm_stream.wait_stream(torch.cuda.current_stream())      # x2 is complete
            with torch.cuda.stream(self.comm_stream):
                ext().push_rows(x2, target.ptrs, self.sg.flags.ptrs, self.world, self.rank, m, k, slot, epoch, 1, sl)
            self._pushing.append(x2)       # keeps the source alive until the main stream joins
            # this rank's own pieces are filled on the consumer's stream: the GEMM never waits for them
            ext().push_rows(x2, target.ptrs, self.sg.flags.ptrs, self.world, self.rank, m, k, slot, epoch, 2, sl)
            count_launch()
        count_launch()
        return view, slot, epoch

    def join(self):
        """Make the current stream wait for the pushes issued so far (their sources may be released
        afterwards). Called where a consumer needs the whole gathered buffer anyway, and before the
        end of a CUDA-graph capture."""
        if self.comm_stream is not None and self._pushing:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            self._pushing.clear()

    def gated_gemm(self, a_buf, weight, slot, epoch, b_mn_major: bool, n_out: int, out=None):
        """out[m_full, n_out] = a_buf @ op(weight), loading A row blocks as their flags arrive."""
        m, k = a_buf.shape
        if out is None:
            out = torch.empty((m, n_out), device=a_buf.device, dtype=torch.bfloat16)
        ext().gemm_ex(a_buf, weight, out, m, n_out, k, a_buf.stride(0), weight.stride(0), out.stride(0), False,
                      b_mn_major, 0, 0, self.sg.flags.local_ptr, slot, epoch, self.rank, [], self.s_local,
                      self.world, self.rank, self.timeout_ms)
        count_launch()
        return out

    def wait_gather(self, slot, epoch):
        self.join()
        self.sg.wait(slot, epoch, self.timeout_ms)

    # -- reduce-scatter through the GEMM epilogue ------------------------------------------------
    def scatter_gemm(self, a2, weight, b_mn_major: bool, n_out: int):
        """Partial product a2[m_full, K] @ op(weight); the rows of rank r's sequence pieces are stored into
        rank r's staging slot for this rank; raises this rank's flag afterwards. Returns (buffer index,
        slot, epoch)."""
        m, k = a2.shape
        assert m == self.m_full and n_out <= self.max_cols
        b = self.n_scatter % 2
        self.n_scatter += 1
        slot = SCATTER_SLOTS[b]
        epoch = self.sg.next_epoch(slot)
        off = self.rank * self.m_local * n_out * 2
        ext().gemm_ex(a2, weight, None, m, n_out, k, a2.stride(0), weight.stride(0), n_out, False, b_mn_major, 0,
                      0, 0, 0, 0, 0, self.staging[b].peer_ptrs(off), self.s_local, self.world,
                      (self.rank + 1) % self.world, self.timeout_ms)
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


class _AGLinearFused(torch.autograd.Function):
    """y = gather(x) @ cat(weights).T. x: [b, s_loc, K] shard; returns [b, s, N]."""

    @staticmethod
    def forward(ctx, x, tp: TPFused, ws, kept, *params):
        b, s_loc, k = x.shape
        x2 = x.reshape(b * s_loc, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        buf, slot, epoch = tp.gather_push(x2, keep=kept)
        if ws.fused_weight is not None:
            y = tp.gated_gemm(buf, ws.fused_weight, slot, epoch, False, ws.out_features)
        else:
            y = torch.empty((tp.m_full, ws.out_features), device=x.device, dtype=x.dtype)
            col = 0
            for w in ws.params:
                tp.gated_gemm(buf, w, slot, epoch, False, w.shape[0], out=y[:, col:col + w.shape[0]])
                col += w.shape[0]
        # kept: the gathered rows stay in their own symmetric buffer until the backward pass (every
        # block's flag was awaited by the GEMM above), so neither the shard nor a re-gather is needed
        ctx.kept = buf if kept else None
        ctx.save_for_backward(*(() if kept else (x2,)))
        ctx.tp, ctx.ws, ctx.shape = tp, ws, (b, s_loc, k)
        return y.view(b, s_loc * tp.world, ws.out_features)

    @staticmethod
    def backward(ctx, dy):
        tp, ws = ctx.tp, ctx.ws
        b, s_loc, k = ctx.shape
        dy2 = dy.reshape(tp.m_full, -1)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.kept is not None:
            buf, slot, epoch = ctx.kept, None, None
        else:
            # re-gather the input for the weight gradient first so the pushes overlap the dgrad GEMM
            (x2,) = ctx.saved_tensors
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
        if slot is not None:
            tp.wait_gather(slot, epoch)
        _, grads = gemm_ops.backward_all(dy2, buf, ws, need_dx=False)
        if pending is not None:
            dx = tp.scatter_sum(*pending, k)
        return (dx.view(b, s_loc, k), None, None, None, *grads)


def _units(ws):
    """GEMM operands of a weight set: the fused view when its parameters are stored back to back, else
    every parameter by itself."""
    return [ws.fused_weight] if ws.fused_weight is not None else list(ws.params)


class _AGLinearSetsFused(torch.autograd.Function):
    """One gather feeding several weight sets: y_i = gather(x) @ cat(weights of set i).T. The parallel
    transformer block reads the same normed rows for q/k/v and for gate/up
    (picotron/model.py:319-329). x: [b, s_loc, K] shard; returns one [b, s, N_i] tensor per set."""

    @staticmethod
    def forward(ctx, x, tp: TPFused, sets, kept, *params):
        b, s_loc, k = x.shape
        x2 = x.reshape(b * s_loc, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        buf, slot, epoch = tp.gather_push(x2, keep=kept)
        outs = []
        for ws in sets:
            y = torch.empty((tp.m_full, ws.out_features), device=x.device, dtype=x.dtype)
            col = 0
            for w in _units(ws):
                tp.gated_gemm(buf, w, slot, epoch, False, w.shape[0], out=y[:, col:col + w.shape[0]])
                col += w.shape[0]
            outs.append(y.view(b, s_loc * tp.world, ws.out_features))
        ctx.kept = buf if kept else None
        ctx.save_for_backward(*(() if kept else (x2,)))
        ctx.tp, ctx.sets, ctx.shape = tp, sets, (b, s_loc, k)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *dys):
        tp, sets = ctx.tp, ctx.sets
        b, s_loc, k = ctx.shape
        if ctx.kept is not None:
            buf, slot, epoch = ctx.kept, None, None
        else:
            (x2,) = ctx.saved_tensors
            buf, slot, epoch = tp.gather_push(x2)
        dy2s = []
        dx = None
        for ws, dy in zip(sets, dys):
            dy2 = dy.reshape(tp.m_full, -1)
            if not dy2.is_contiguous():
                dy2 = dy2.contiguous()
            dy2s.append(dy2)
            # each partial product is reduced before the next one reuses the two staging buffers
            col = 0
            for w in _units(ws):
                sb, sslot, sepoch = tp.scatter_gemm(dy2[:, col:col + w.shape[0]], w, True, k)
                dx = tp.scatter_sum(sb, sslot, sepoch, k, addend=dx)
                col += w.shape[0]
        if slot is not None:
            tp.wait_gather(slot, epoch)
        grads = []
        for ws, dy2 in zip(sets, dy2s):
            grads += gemm_ops.backward_all(dy2, buf, ws, need_dx=False)[1]
        return (dx.view(b, s_loc, k), None, None, None, *grads)


class _DualLinearRSFused(torch.autograd.Function):
    """y_shard = reduce_scatter(xa @ wa.T) + reduce_scatter(xb @ wb.T) (+ addend): the output side of the
    parallel transformer block, whose attention and feed-forward partial sums land on the same rows.
    Two scatter epilogues and two slot sums forward; backward gathers dy once for both branches."""

    @staticmethod
    def forward(ctx, xa, wa, xb, wb, tp: TPFused, addend):
        b, s_loc = tp.m_local // tp.s_local, tp.s_local
        n = wa.shape[0]
        xs = []
        for x in (xa, xb):
            x2 = x.reshape(tp.m_full, x.shape[-1])
            xs.append(x2 if x2.is_contiguous() else x2.contiguous())
        y = None
        if addend is not None:
            y = addend.reshape(b * s_loc, n)
            if not y.is_contiguous():
                y = y.contiguous()
        for x2, w in zip(xs, (wa, wb)):
            sb, slot, epoch = tp.scatter_gemm(x2, w, False, n)
            y = tp.scatter_sum(sb, slot, epoch, n, addend=y)
        ctx.save_for_backward(xs[0], wa, xs[1], wb)
        ctx.tp, ctx.shapes, ctx.has_addend = tp, (xa.shape, xb.shape), addend is not None
        return y.view(b, s_loc, n)

    @staticmethod
    def backward(ctx, dy):
        xa2, wa, xb2, wb = ctx.saved_tensors
        tp = ctx.tp
        dy2 = dy.reshape(-1, wa.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        buf, slot, epoch = tp.gather_push(dy2)
        dxa = tp.gated_gemm(buf, wa, slot, epoch, True, wa.shape[1])
        dxb = tp.gated_gemm(buf, wb, slot, epoch, True, wb.shape[1])
        tp.wait_gather(slot, epoch)
        dwa = gemm_ops.wgrad_into(wa, buf, xa2)
        dwb = gemm_ops.wgrad_into(wb, buf, xb2)
        return (dxa.view(ctx.shapes[0]), dwa, dxb.view(ctx.shapes[1]), dwb, None,
                (dy if ctx.has_addend else None))


class _LinearRSFused(torch.autograd.Function):
    """y_shard = reduce_scatter(x @ w.T) (+ addend). x: [b, s, K_loc] (or its [b*s, K_loc] view);
    returns [b, s/tp, N]."""

    @staticmethod
    def forward(ctx, x, w, tp: TPFused, addend):
        x2 = x.reshape(tp.m_full, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        b, s_loc = tp.m_local // tp.s_local, tp.s_local
        n = w.shape[0]
        sb, slot, epoch = tp.scatter_gemm(x2, w, False, n)
        add2 = None
        if addend is not None:
            add2 = addend.reshape(b * s_loc, n)
            if not add2.is_contiguous():
                add2 = add2.contiguous()
        y = tp.scatter_sum(sb, slot, epoch, n, addend=add2)
        ctx.save_for_backward(x2, w)
        ctx.tp, ctx.x_shape, ctx.has_addend = tp, x.shape, addend is not None
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
        return dx2.view(ctx.x_shape), dw, None, (dy if ctx.has_addend else None)


class _EmbeddingRSFused(torch.autograd.Function):
    """Vocabulary-parallel embedding under sequence parallelism without a collective call: every
    rank looks its vocabulary shard up for the whole sequence (rows of ids it does not own are
    zero), stores the rows of rank o's sequence pieces into its slot of rank o's staging buffer and
    sums the slots it received; backward gathers the output gradient by pushing and scatters it into
    the table's gradient. ids: [b, s] (full sequence); returns [b, s/tp, H]."""

    @staticmethod
    def forward(ctx, ids, weight, vocab_start, tp: TPFused):
        b, s = ids.shape
        V, H = weight.shape
        flat = ids.reshape(-1).contiguous()
        part = torch.empty((tp.m_full, H), device=weight.device, dtype=weight.dtype)
        ext().embedding_fwd(weight, flat, part, tp.m_full, H, V, vocab_start)
        sb = tp.n_scatter % 2
        tp.n_scatter += 1
        slot = SCATTER_SLOTS[sb]
        epoch = tp.sg.next_epoch(slot)
        ext().scatter_rows(part, tp.staging[sb].ptrs, tp.sg.flags.ptrs, tp.world, tp.rank, tp.world, tp.m_local, H,
                           slot, epoch, tp.s_local)
        count_launch(2)
        y = tp.scatter_sum(sb, slot, epoch, H)
        ctx.save_for_backward(flat, weight)
        ctx.tp, ctx.vocab_start = tp, vocab_start
        return y.view(b, s // tp.world, H)

    @staticmethod
    def backward(ctx, dy):
        flat, weight = ctx.saved_tensors
        tp = ctx.tp
        V, H = weight.shape
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        buf, slot, epoch = tp.gather_push(dy2)
        tp.wait_gather(slot, epoch)
        main_grad = getattr(weight, "main_grad", None)
        acc = main_grad if main_grad is not None else torch.zeros((V, H), device=weight.device, dtype=torch.float32)
        ext().embedding_bwd(buf, flat, acc, tp.m_full, H, V, ctx.vocab_start)
        count_launch()
        if main_grad is not None:
            hook = getattr(weight, "grad_ready_hook", None)
            if hook is not None:
                hook()
            return None, None, None, None
        return None, acc.to(weight.dtype), None, None


def embedding_rs(ids, weight, vocab_start: int, tp: TPFused):
    return _EmbeddingRSFused.apply(ids, weight, vocab_start, tp)


def ag_linear(x, tp: TPFused, mods):
    ws = gemm_ops.WeightSet.of(mods)
    kept = tp.keep_gathered and torch.is_grad_enabled()      # decided here: grad mode is off inside forward
    return _AGLinearFused.apply(x, tp, ws, kept, *ws.params)


def ag_linear_sets(x, tp: TPFused, mod_sets):
    """Several groups of projections on one gathered input; returns one output per group."""
    sets = [gemm_ops.WeightSet.of(mods) for mods in mod_sets]
    kept = tp.keep_gathered and torch.is_grad_enabled()
    return _AGLinearSetsFused.apply(x, tp, sets, kept, *[p for ws in sets for p in ws.params])


def linear_rs(x, w, tp: TPFused, addend=None):
    return _LinearRSFused.apply(x, w, tp, addend)


def dual_linear_rs(xa, wa, xb, wb, tp: TPFused, addend=None):
    return _DualLinearRSFused.apply(xa, wa, xb, wb, tp, addend)
