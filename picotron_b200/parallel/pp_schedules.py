"""Pipeline schedules as data, one executor for all of them.

A schedule is, per pipeline rank, an ordered list of actions ``(kind, chunk, micro_batch)`` with
``kind`` in F (forward), B (backward: input gradients, plus weight gradients unless split) and
W (deferred weight gradients, zero-bubble only). ``plan_rounds`` places the actions of all
ranks on a common round grid by simulating their data dependencies; every activation or
gradient that crosses ranks is transferred *in the round its producer ran*, by one batched
isend/irecv group per rank and round, so sends and receives always pair up in the same order
on both sides whatever the schedule (the idea behind the reference's ZB-V executor,
picotron/pipeline_parallel/pp_schedules.py:508-589, applied to every schedule).

Generators:
* ``afab_order``        all forwards, then all backwards (pipeline_parallel.py:173-231)
* ``one_f_one_b_order`` warm-up ``min(p-rank-1, m)``, steady 1F1B, cool-down (pipeline_parallel.py:234-349)
* ``interleaved_order`` Megatron interleaved 1F1B with v virtual stages per rank; chunk c of
  rank r is global stage ``c*p + r`` (pp_schedules.py:160-358)
* ``zero_bubble_order`` ZB-H1: B and W split, W fills the cool-down bubbles (pp_schedules.py:65-152)
* ``zbv_order``         ZB-V: rank r owns global stages r and 2p-1-r; greedy list schedule with
  priority B > F (in-flight cap 2p) > W (pp_schedules.py:441-496)

The public ``train_step_pipeline_{zb,interleaved,zbv}`` functions keep the reference signature
``(model, data_loader, tensor_shapes, device, dtype)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

F, B, W = "F", "B", "W"
Action = Tuple[str, int, int]  # (kind, chunk, micro_batch)


@dataclass(frozen=True)
class StageMap:
    """Which rank runs which global stage. ``stage_of(rank, chunk)`` / ``rank_of(stage)``."""
    p: int
    v: int
    vshape: bool = False

    @property
    def num_stages(self) -> int:
        return self.p * self.v

    def stage_of(self, rank: int, chunk: int) -> int:
        if self.vshape:
            assert self.v == 2
            return rank if chunk == 0 else 2 * self.p - 1 - rank
        return chunk * self.p + rank

    def rank_of(self, stage: int) -> int:
        if self.vshape:
            return stage if stage < self.p else 2 * self.p - 1 - stage
        return stage % self.p

    def chunk_of(self, stage: int) -> int:
        if self.vshape:
            return 0 if stage < self.p else 1
        return stage // self.p


# ------------------------------------------------------------------------------------------
# order generators (per rank)
# ------------------------------------------------------------------------------------------
def afab_order(p: int, m: int) -> List[List[Action]]:
    return [[(F, 0, i) for i in range(m)] + [(B, 0, i) for i in range(m)] for _ in range(p)]


def one_f_one_b_order(p: int, m: int) -> List[List[Action]]:
    orders = []
    for rank in range(p):
        warm = min(p - rank - 1, m)
        acts: List[Action] = [(F, 0, i) for i in range(warm)]
        for i in range(m - warm):
            acts += [(F, 0, warm + i), (B, 0, i)]
        acts += [(B, 0, i) for i in range(m - warm, m)]
        orders.append(acts)
    return orders


def interleaved_order(p: int, m: int, v: int = 2) -> List[List[Action]]:
    assert m % p == 0, "interleaved 1F1B needs the number of micro-batches divisible by the pipeline size"
    total = m * v

    def fwd(k):
        return (F, (k % (p * v)) // p, (k // (p * v)) * p + k % p)

    def bwd(k):
        return (B, v - 1 - (k % (p * v)) // p, (k // (p * v)) * p + k % p)

    orders = []
    for rank in range(p):
        warm = min((p - rank - 1) * 2 + (v - 1) * p, total)
        acts = [fwd(k) for k in range(warm)]
        for k in range(total - warm):
            acts += [fwd(warm + k), bwd(k)]
        acts += [bwd(k) for k in range(total - warm, total)]
        orders.append(acts)
    return orders


def _list_schedule(smap: StageMap, m: int, cap: Callable[[int], int], split_w: bool) -> List[List[Action]]:
    """Greedy unit-time list scheduling: each round every rank runs its best ready action with
    priority B > F (while fewer than cap(rank) forwards await their backward) > W."""
    p, S = smap.p, smap.num_stages
    done: Dict[Tuple[str, int, int], int] = {}       # (kind, stage, mb) -> round
    next_f = [[0] * smap.v for _ in range(p)]          # next micro-batch to forward per chunk
    next_b = [[0] * smap.v for _ in range(p)]
    pending_w: List[List[Tuple[int, int]]] = [[] for _ in range(p)]
    in_flight = [0] * p
    orders: List[List[Action]] = [[] for _ in range(p)]
    total = m * smap.v
    finished_b = [0] * p
    t = 0
    while any(finished_b[r] < total or pending_w[r] for r in range(p)):
        chosen = []
        for r in range(p):
            pick = None
            # backward: deepest chunk first (its gradient unblocks upstream stages)
            for c in sorted(range(smap.v), key=lambda c: -smap.stage_of(r, c)):
                i = next_b[r][c]
                if i >= m:
                    continue
                s = smap.stage_of(r, c)
                if done.get((F, s, i), t) >= t:
                    continue
                if s < S - 1 and done.get((B, s + 1, i), t) >= t:
                    continue
                pick = (B, c, i)
                break
            if pick is None and in_flight[r] < cap(r):
                # forward: deepest ready chunk first (closest to producing a backward)
                for c in sorted(range(smap.v), key=lambda c: -smap.stage_of(r, c)):
                    i = next_f[r][c]
                    if i >= m:
                        continue
                    s = smap.stage_of(r, c)
                    if s > 0 and done.get((F, s - 1, i), t) >= t:
                        continue
                    pick = (F, c, i)
                    break
            if pick is None and pending_w[r]:
                c, i = pending_w[r][0]
                pick = (W, c, i)
            if pick is not None:
                chosen.append((r, pick))
        assert chosen, "pipeline schedule deadlocked"
        for r, (kind, c, i) in chosen:
            s = smap.stage_of(r, c)
            done[(kind, s, i)] = t
            orders[r].append((kind, c, i))
            if kind == F:
                next_f[r][c] += 1
                in_flight[r] += 1
            elif kind == B:
                next_b[r][c] += 1
                in_flight[r] -= 1
                finished_b[r] += 1
                if split_w:
                    pending_w[r].append((c, i))
            else:
                pending_w[r].pop(0)
        t += 1
    return orders


def zero_bubble_order(p: int, m: int) -> List[List[Action]]:
    """ZB-H1: the in-flight cap of 1F1B (p - rank) with weight gradients deferred into bubbles."""
    return _list_schedule(StageMap(p, 1), m, cap=lambda r: p - r, split_w=True)


def zbv_order(p: int, m: int) -> List[List[Action]]:
    return _list_schedule(StageMap(p, 2, vshape=True), m, cap=lambda r: 2 * p, split_w=True)


# ------------------------------------------------------------------------------------------
# round planning
# ------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Message:
    kind: str      # "act" (forward activation) or "grad" (backward gradient)
    src_stage: int
    dst_stage: int
    mb: int
    src_rank: int
    dst_rank: int

    @property
    def key(self):
        return (self.kind, self.dst_stage, self.mb)


@dataclass
class RoundPlan:
    timeline: List[List[Optional[Action]]]     # [rank][round] -> action or None
    messages: List[List[Message]]              # [round] -> cross-rank messages produced in it
    num_rounds: int


def plan_rounds(orders: List[List[Action]], smap: StageMap) -> RoundPlan:
    """Lock-step simulation: an action runs in the first round after all its inputs exist (an
    input produced in round t is usable from round t+1, the transfer happening in round t)."""
    p, S = smap.p, smap.num_stages
    ptr = [0] * p
    done: Dict[Tuple[str, int, int], int] = {}
    timeline: List[List[Optional[Action]]] = [[] for _ in range(p)]
    messages: List[List[Message]] = []
    t = 0
    while any(ptr[r] < len(orders[r]) for r in range(p)):
        running = []
        for r in range(p):
            if ptr[r] >= len(orders[r]):
                continue
            kind, c, i = orders[r][ptr[r]]
            s = smap.stage_of(r, c)
            if kind == F:
                ready = s == 0 or done.get((F, s - 1, i), t) < t
            elif kind == B:
                ready = done.get((F, s, i), t) < t and (s == S - 1 or done.get((B, s + 1, i), t) < t)
            else:
                ready = done.get((B, s, i), t) < t
            if ready:
                running.append((r, (kind, c, i), s))
        assert running, f"schedule cannot make progress at round {t}"
        msgs = []
        for r in range(p):
            timeline[r].append(None)
        for r, act, s in running:
            kind, c, i = act
            done[(kind, s, i)] = t
            timeline[r][t] = act
            ptr[r] += 1
            if kind == F and s < S - 1 and smap.rank_of(s + 1) != r:
                msgs.append(Message("act", s, s + 1, i, r, smap.rank_of(s + 1)))
            if kind == B and s > 0 and smap.rank_of(s - 1) != r:
                msgs.append(Message("grad", s, s - 1, i, r, smap.rank_of(s - 1)))
        messages.append(msgs)
        t += 1
    return RoundPlan(timeline, messages, t)


def bubble_fraction(plan: RoundPlan, f_cost: float = 1.0, b_cost: float = 2.0, w_cost: float = 1.0,
                    split_w: bool = False) -> float:
    """Idle share of the round grid under a simple cost model (for comparing schedules offline)."""
    cost = {F: f_cost, B: (b_cost - w_cost) if split_w else b_cost, W: w_cost}
    busy = sum(cost[a[0]] for row in plan.timeline for a in row if a is not None)
    per_round = [max((cost[row[t][0]] if row[t] is not None else 0.0) for row in plan.timeline)
                 for t in range(plan.num_rounds)]
    total = sum(per_round) * len(plan.timeline)
    return 1.0 - busy / total if total else 0.0


SCHEDULES = {
    "afab": lambda p, m, v: (afab_order(p, m), StageMap(p, 1), False),
    "1f1b": lambda p, m, v: (one_f_one_b_order(p, m), StageMap(p, 1), False),
    "zb": lambda p, m, v: (zero_bubble_order(p, m), StageMap(p, 1), True),
    "interleaved": lambda p, m, v: (interleaved_order(p, m, v), StageMap(p, v), False),
    "zbv": lambda p, m, v: (zbv_order(p, m), StageMap(p, 2, vshape=True), True),
}


def build_plan(engine: str, p: int, m: int, v: int = 2):
    orders, smap, split_w = SCHEDULES[engine](p, m, v)
    return plan_rounds(orders, smap), smap, split_w


# ------------------------------------------------------------------------------------------
# reference-compatible entry points (implemented by the executor in pipeline_parallel.py)
# ------------------------------------------------------------------------------------------
def train_step_pipeline_zb(model, data_loader, tensor_shapes, device, dtype):
    from .pipeline_parallel import run_schedule
    return run_schedule("zb", model, data_loader, tensor_shapes, device, dtype)


def train_step_pipeline_interleaved(model, data_loader, tensor_shapes, device, dtype):
    from .pipeline_parallel import run_schedule
    return run_schedule("interleaved", model, data_loader, tensor_shapes, device, dtype)


def train_step_pipeline_zbv(model, data_loader, tensor_shapes, device, dtype):
    from .pipeline_parallel import run_schedule
    return run_schedule("zbv", model, data_loader, tensor_shapes, device, dtype)


def __getattr__(name):
    # InterleavedPipelineParallel / VShapePipelineParallel live with the other stage wrappers
    if name in ("InterleavedPipelineParallel", "VShapePipelineParallel"):
        from . import pipeline_parallel
        return getattr(pipeline_parallel, name)
    raise AttributeError(name)
