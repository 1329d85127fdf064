"""A host-side model of the peer-memory protocol of the fused tensor-parallel and expert-parallel paths.

``compute-sanitizer`` cannot be run on the GPUs this project is developed on, so the argument that the
flag/epoch protocol is free of races is checked here instead, by brute force: the operations one
micro-batch issues (pushes into gather buffers, flag-gated GEMMs, scattering GEMMs, slot sums, group
barriers; a main and a communication stream per rank) are replayed by a randomised scheduler that
interleaves ranks and streams arbitrarily and splits every multi-word write into chunks. Every word
written carries the identity of the operation that wrote it, every read states which operation's data
it expects; a read that sees anything else is a race (data overwritten too early, or read before it
arrived).

The model follows ``ops/fused_tp.py`` and ``csrc/runtime/flags.cuh``:

* a *push* stores this rank's block into every peer's buffer, then raises flag ``[slot][rank]`` to the
  operation's epoch on every peer (release after the data);
* a *gated GEMM* reads block ``r`` of its local buffer only after flag ``[slot][r]`` reached the epoch
  (its own block is filled by its own stream and never waited for);
* a *scattering GEMM* stores its partial result into slot ``rank`` of every peer's staging buffer and
  raises a flag; a *slot sum* waits for all flags and reads all slots;
* two copies of the gather and of the staging buffer are used alternately; "kept" gather buffers are
  used once per micro-batch and read again by the backward pass; a group barrier opens every
  micro-batch when buffers are kept.

``build_program`` writes down one rank's operation list for a number of layers and micro-batches
(``build_moe_program`` does the same for the exchanges of mixture-of-experts layers, ``ops/fused_ep.py``),
``simulate`` runs all ranks under a seeded random schedule and returns the list of violations.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class Op:
    kind: str                      # push | fill | gemm_gated | read_all | scatter | slot_sum | barrier | join | fork
    stream: str = "main"           # main | comm
    buf: Optional[str] = None      # buffer name
    slot: Optional[int] = None
    epoch: int = 0
    tag: Optional[Tuple] = None    # identity of the data this op writes / expects
    wait_main: int = -1            # comm-stream ops: index of the main-stream op that must have finished


@dataclass
class _Rank:
    ops: Dict[str, List[Op]]
    pc: Dict[str, int] = field(default_factory=lambda: {"main": 0, "comm": 0})
    step: Dict[str, int] = field(default_factory=lambda: {"main": 0, "comm": 0})   # progress inside the current op
    done_main: int = -1


def build_program(layers: int, micro_batches: int, keep_gathered: bool, barrier: bool, comm_stream: bool = True,
                  double_buffer: bool = True) -> List[Op]:
    """One rank's operations (identical on every rank apart from the rank index, which the simulator
    supplies). Per layer and direction: a column-parallel projection (push + gated GEMM) and a
    row-parallel one (scattering GEMM + slot sum); the backward pass re-reads kept buffers or gathers
    again."""
    ops: List[Op] = []
    epochs: Dict[int, int] = {}
    n_gather = n_scatter = 0

    def next_epoch(slot):
        epochs[slot] = epochs.get(slot, 0) + 1
        return epochs[slot]

    def gather(tag, kept_index=None):
        nonlocal n_gather
        if kept_index is not None:
            buf, slot = f"kept{kept_index}", 16 + kept_index
        else:
            b = n_gather % 2 if double_buffer else 0
            n_gather += 1
            buf, slot = f"gather{b}", b
        e = next_epoch(slot)
        main_index = sum(1 for o in ops if o.stream == "main") - 1
        ops.append(Op("push", "comm" if comm_stream else "main", buf, slot, e, tag, wait_main=main_index))
        ops.append(Op("fill", "main", buf, slot, e, tag))            # own block, on the consumer's stream
        return buf, slot, e

    def scatter(tag):
        nonlocal n_scatter
        b = n_scatter % 2 if double_buffer else 0
        n_scatter += 1
        buf, slot = f"staging{b}", 2 + b
        e = next_epoch(slot)
        ops.append(Op("scatter", "main", buf, slot, e, tag))
        return buf, slot, e

    def slot_sum(where, tag):
        ops.append(Op("slot_sum", "main", *where, tag))

    for mb in range(micro_batches):
        if barrier:
            ops.append(Op("join"))
            ops.append(Op("barrier", slot=255, epoch=next_epoch(255)))
        kept = []
        for layer in range(layers):                                 # forward
            tag = ("x", mb, layer)
            buf, slot, e = gather(tag, kept_index=layer if keep_gathered else None)
            ops.append(Op("gemm_gated", "main", buf, slot, e, tag))  # column-parallel projection
            kept.append((buf, tag))
            slot_sum(scatter(("y", mb, layer)), ("y", mb, layer))    # row-parallel projection
        for layer in reversed(range(layers)):                       # backward
            tag = ("dy", mb, layer)
            buf, slot, e = gather(tag)                               # row-parallel: gather dy, gated dgrad ...
            ops.append(Op("gemm_gated", "main", buf, slot, e, tag))
            ops.append(Op("join"))
            ops.append(Op("read_all", "main", buf, slot, e, tag))    # ... and a weight gradient over all of it
            if keep_gathered:                                        # column-parallel: dgrad scattered, wgrad on
                where = scatter(("dx", mb, layer))                   # the input kept since the forward pass
                ops.append(Op("read_all", "main", kept[layer][0], None, 0, kept[layer][1]))
                slot_sum(where, ("dx", mb, layer))
            else:                                                    # ... or on the input gathered again
                xbuf, xslot, xe = gather(("x", mb, layer))
                where = scatter(("dx", mb, layer))
                ops.append(Op("join"))
                ops.append(Op("read_all", "main", xbuf, xslot, xe, ("x", mb, layer)))
                slot_sum(where, ("dx", mb, layer))
    ops.append(Op("join"))
    return ops


def build_moe_program(layers: int, micro_batches: int, double_buffer: bool = True, load_sum: bool = True,
                      tiles: int = 1) -> List[Op]:
    """One rank's operations for mixture-of-experts layers on the capacity path of ``ops/fused_ep.py``:
    per layer forward the expert-load rows (every rank stores its row into all peers' table, then adds the
    rows), the dispatch into the expert-major slabs and the combine exchange into the source-major slabs;
    backward the two exchanges in the opposite direction. Every exchange is "each rank writes block
    ``rank`` of every peer's buffer, raises its flag, and the consumer reads all blocks after all flags",
    i.e. the model's scatter / slot_sum pair on the buffers and flag slots of that file; the two copies
    of each buffer alternate per kind of exchange. ``tiles`` > 1 issues the forward dispatches of that many
    token tiles back to back before their combines (exchanges of one kind in a row, which is what the
    second copy of a slab is for: with kinds strictly alternating, every exchange in between already
    orders the reuse of a slab after its last read)."""
    ops: List[Op] = []
    epochs: Dict[int, int] = {}
    counts = {"load": 0, "expert": 0, "source": 0}
    slots = {"load": 24, "expert": 20, "source": 22}

    def exchange(kind, tag):
        b = counts[kind] % 2 if double_buffer else 0
        counts[kind] += 1
        slot = slots[kind] + b
        epochs[slot] = epochs.get(slot, 0) + 1
        ops.append(Op("scatter", "main", f"{kind}{b}", slot, epochs[slot], tag))
        ops.append(Op("slot_sum", "main", f"{kind}{b}", slot, epochs[slot], tag))

    for mb in range(micro_batches):
        for layer in range(layers):                                 # forward
            if load_sum:
                exchange("load", ("load", mb, layer))
            for t in range(tiles):
                exchange("expert", ("dispatch", mb, layer, t))
            for t in range(tiles):
                exchange("source", ("combine", mb, layer, t))
        for layer in reversed(range(layers)):                       # backward: combine's, then dispatch's
            exchange("expert", ("d_combine", mb, layer))
            exchange("source", ("d_dispatch", mb, layer))
    return ops


def simulate(world: int, program: List[Op], seed: int, chunks: int = 2, max_steps: int = 2_000_000) -> List[str]:
    """Run ``program`` on ``world`` ranks under a random interleaving. Returns the violations found
    (empty = none); raises if the schedule deadlocks."""
    rng = random.Random(seed)
    ranks = [_Rank({"main": [o for o in program if o.stream == "main"], "comm": [o for o in program if o.stream == "comm"]})
             for _ in range(world)]
    mem: Dict[Tuple[int, str, int], List] = {}      # (rank, buffer, block) -> per-chunk tags
    flags: Dict[Tuple[int, int, int], int] = {}     # (rank, slot, source) -> epoch
    violations: List[str] = []

    def cell(r, buf, blk):
        return mem.setdefault((r, buf, blk), [None] * chunks)

    def check(r, buf, blk, tag, who):
        got = cell(r, buf, blk)
        if any(g != (tag, blk) for g in got):
            violations.append(f"rank {r} {who}: block {blk} of {buf} holds {got}, expected {(tag, blk)}")

    def runnable(r, stream):
        rk = ranks[r]
        if rk.pc[stream] >= len(rk.ops[stream]):
            return None
        op = rk.ops[stream][rk.pc[stream]]
        if stream == "comm" and op.wait_main > rk.done_main:
            return None
        st = rk.step[stream]
        if op.kind == "gemm_gated":
            blk = (r + st) % world                                   # own block first
            if blk != r and flags.get((r, op.slot, blk), 0) < op.epoch:
                return None
        if op.kind in ("slot_sum", "read_all") and op.slot is not None and st == 0:
            if any(flags.get((r, op.slot, s), 0) < op.epoch for s in range(world) if not (op.kind == "read_all" and s == r)):
                return None
        if op.kind == "barrier" and st == 1:
            if any(flags.get((r, op.slot, s), 0) < op.epoch for s in range(world)):
                return None
        if op.kind == "join" and rk.pc["comm"] < sum(1 for o in rk.ops["comm"] if o.wait_main <= rk.done_main):
            return None
        return op

    def advance(r, stream, op):
        rk = ranks[r]
        st = rk.step[stream]
        finished = False
        if op.kind == "push":                                        # chunk by chunk to every peer, then the flags
            total = (world - 1) * chunks
            if st < total:
                peer = [p for p in range(world) if p != r][st // chunks]
                cell(peer, op.buf, r)[st % chunks] = (op.tag, r)
            else:
                for p in range(world):
                    flags[(p, op.slot, r)] = max(flags.get((p, op.slot, r), 0), op.epoch)
                finished = True
        elif op.kind == "fill":
            cell(r, op.buf, r)[st] = (op.tag, r)
            finished = st + 1 == chunks
        elif op.kind == "gemm_gated":
            blk = (r + st) % world
            check(r, op.buf, blk, op.tag, "gated GEMM")
            finished = st + 1 == world
        elif op.kind == "read_all":
            for blk in range(world):
                check(r, op.buf, blk, op.tag, "full read")
            finished = True
        elif op.kind == "scatter":                                   # partial for owner o -> slot r of o's staging
            total = world * chunks
            if st < total:
                cell(st // chunks, op.buf, r)[st % chunks] = (op.tag, r)
            else:
                for p in range(world):
                    flags[(p, op.slot, r)] = max(flags.get((p, op.slot, r), 0), op.epoch)
                finished = True
        elif op.kind == "slot_sum":
            for blk in range(world):
                check(r, op.buf, blk, op.tag, "slot sum")
            finished = True
        elif op.kind == "barrier":
            if st == 0:
                for p in range(world):
                    flags[(p, op.slot, r)] = max(flags.get((p, op.slot, r), 0), op.epoch)
            finished = st == 1
        elif op.kind == "join":
            finished = True
        if finished:
            rk.step[stream] = 0
            rk.pc[stream] += 1
            if stream == "main":
                rk.done_main += 1
        else:
            rk.step[stream] = st + 1

    for _ in range(max_steps):
        choices = [(r, s) for r in range(world) for s in ("main", "comm") if runnable(r, s) is not None]
        if not choices:
            if all(rk.pc[s] >= len(rk.ops[s]) for rk in ranks for s in ("main", "comm")):
                return violations
            raise RuntimeError("deadlock in the protocol model")
        r, s = rng.choice(choices)
        advance(r, s, runnable(r, s))
    raise RuntimeError("protocol model did not finish")
