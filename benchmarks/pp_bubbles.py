"""Offline comparison of the pipeline schedules (no GPU): rounds of the plan, makespan and idle share
of a dataflow simulation under a cost model (forward 1, backward 2 = input gradient 1 + weight
gradients 1 for a rank's whole layer share, divided by the number of chunks the rank's layers are
split into; transfers free) and the peak number of
micro-batches whose activations a rank holds — the quantities behind the schedule table of
picotron/pipeline_parallel/README.md:215-221 (8 stages, 16 / 32 / 64 micro-batches).

    python benchmarks/pp_bubbles.py [--p 8] [--m 16 32 64] [--v 2]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200.parallel import pp_schedules as sched  # noqa: E402


def peak_in_flight(plan) -> int:
    """Largest number of (chunk, micro-batch) forward results a rank holds before their backward."""
    worst = 0
    for row in plan.timeline:
        held = 0
        for act in row:
            if act is None:
                continue
            if act[0] == sched.F:
                held += 1
                worst = max(worst, held)
            elif act[0] == sched.B:
                held -= 1
    return worst


def simulate(plan, smap, split_w: bool, f_cost=1.0, b_cost=2.0, w_cost=1.0):
    """Dataflow timing: every rank runs its actions in schedule order, each as soon as the rank is free
    and its inputs exist (transfers are free). Returns (makespan, idle share)."""
    cost = {sched.F: f_cost, sched.B: (b_cost - w_cost) if split_w else b_cost, sched.W: w_cost}
    S = smap.num_stages
    per_stage = len(plan.timeline)          # p ranks
    orders = [[a for a in row if a is not None] for row in plan.timeline]
    ptr = [0] * per_stage
    free = [0.0] * per_stage
    end = {}
    remaining = sum(len(o) for o in orders)
    while remaining:
        progressed = False
        for r in range(per_stage):
            while ptr[r] < len(orders[r]):
                kind, c, i = orders[r][ptr[r]]
                s = smap.stage_of(r, c)
                if kind == sched.F:
                    deps = [(sched.F, s - 1, i)] if s > 0 else []
                elif kind == sched.B:
                    deps = [(sched.F, s, i)] + ([(sched.B, s + 1, i)] if s < S - 1 else [])
                else:
                    deps = [(sched.B, s, i)]
                if any(d not in end for d in deps):
                    break
                start = max([free[r]] + [end[d] for d in deps])
                free[r] = start + cost[kind]
                end[(kind, s, i)] = free[r]
                ptr[r] += 1
                remaining -= 1
                progressed = True
        assert progressed, "schedule deadlocks"
    makespan = max(free)
    busy = sum(cost[a[0]] for o in orders for a in o)
    return makespan, 1.0 - busy / (makespan * per_stage)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--p", type=int, default=8)
    ap.add_argument("--m", type=int, nargs="+", default=[16, 32, 64])
    ap.add_argument("--v", type=int, default=2)
    args = ap.parse_args()
    print(f"# p = {args.p} stages, v = {args.v} virtual stages for interleaved; cost model F=1, B=2 (1 + 1 when the "
          f"weight gradients are split off)")
    print(f"{'m':>4} {'schedule':>12} {'rounds':>7} {'makespan':>9} {'bubble':>7} {'time vs 1f1b':>13} {'peak in-flight':>15}")
    for m in args.m:
        base = None
        for name in ("afab", "1f1b", "zb", "interleaved", "zbv"):
            plan, smap, split_w = sched.build_plan(name, args.p, m, args.v)
            chunks = smap.v if hasattr(smap, "v") else 1
            # a chunk holds 1/chunks of a rank's layers, so its actions cost that share
            t, bub = simulate(plan, smap, split_w, 1.0 / chunks, 2.0 / chunks, 1.0 / chunks)
            if name == "afab":
                afab_t = t
            if name == "1f1b":
                base = t
            peak = peak_in_flight(plan)
            rel = t / base if base else float("nan")
            print(f"{m:>4} {name:>12} {plan.num_rounds:>7} {t:>9.1f} {bub:>7.3f} {rel:>13.3f} "
                  f"{peak:>9} / {chunks} chunk(s)")
        print()


if __name__ == "__main__":
    main()
