"""Micro-benchmark of the tcgen05 GEMM on the layer shapes of the SmolLM-1.7B and Llama-2-7B
configs, next to ``torch.matmul`` (cuBLAS) on the same operands.

CUDA-event timing after warm-up, L2 flushed between timed iterations by writing a 256 MiB
buffer. Prints one line per shape and layout: microseconds, TFLOP/s and the fraction of the
measured cuBLAS bf16 peak found in MEASURED_PEAKS.json (burst figure) when that file exists.

    python benchmarks/bench_gemm.py [--iters 20] [--small]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200 import ops  # noqa: E402
from picotron_b200.ops import gemm  # noqa: E402


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) * 1e3)
    times.sort()
    return times[len(times) // 2]


def grouped(args, peak, flush):
    """(experts, rows per expert, in, out): gate+up and down projections of the MoE benchmark config
    (64 experts of FFN 1024 at h2048, capacity 960 rows per expert and source rank) at EP = 8 and 2,
    and an uneven dropless split."""
    from picotron_b200.ops import grouped_gemm as gg
    cases = [("ep8 gate+up", [7680] * 8, 2048, 2048), ("ep8 down", [7680] * 8, 1024, 2048),
             ("ep2 gate+up", [1920] * 32, 2048, 2048), ("ep2 down", [1920] * 32, 1024, 2048),
             ("uneven gate+up", [9000, 300, 4100, 77, 12000, 2500, 640, 5], 2048, 2048)]
    if args.small:
        cases = [("small gate+up", [3072] * 8, 2048, 2048)]
    for name, counts, d_in, d_out in cases:
        G, n = len(counts), sum(counts)
        layout = gg.GroupLayout.from_counts(counts, "cuda")
        x = layout.pad(torch.randn(n, d_in, device="cuda", dtype=torch.bfloat16))
        dy = layout.pad(torch.randn(n, d_out, device="cuda", dtype=torch.bfloat16))
        w = torch.randn(G * d_out, d_in, device="cuda", dtype=torch.bfloat16)
        dw32 = torch.zeros(G * d_out, d_in, device="cuda", dtype=torch.float32)
        seg = layout.seg_start.tolist()
        flops = 2.0 * n * d_in * d_out

        def lib_fwd():
            for e in range(G):
                torch.matmul(x[seg[e]:seg[e + 1]], w[e * d_out:(e + 1) * d_out].t())

        def lib_dgrad():
            for e in range(G):
                torch.matmul(dy[seg[e]:seg[e + 1]], w[e * d_out:(e + 1) * d_out])

        def lib_wgrad():
            for e in range(G):
                torch.matmul(dy[seg[e]:seg[e + 1]].t(), x[seg[e]:seg[e + 1]])

        rows = [("fwd", lambda: gg.grouped_gemm_nt(x, w, layout, d_out), lib_fwd),
                ("dgrad", lambda: gg.grouped_gemm_nn(dy, w, layout, d_out), lib_dgrad),
                ("wgrad+acc", lambda: gg.grouped_gemm_tn(dy, x, layout, dw32, accumulate=True), lib_wgrad)]
        for rn, ours, lib in rows:
            t_ours = time_fn(ours, args.iters, flush)
            t_lib = time_fn(lib, args.iters, flush)
            tf = flops / t_ours / 1e6
            line = (f"{name:15s} G={G:2d} rows={n:6d} {d_in}->{d_out} {rn:10s} grouped {t_ours:8.1f} us {tf:7.1f} TFLOP/s | "
                    f"{G} cuBLAS calls {t_lib:8.1f} us {flops / t_lib / 1e6:7.1f} TFLOP/s")
            if peak:
                line += f" | {tf / peak:.3f} of measured"
            print(line, flush=True)
        ops.check_status(name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="one small shape (for profiler captures)")
    ap.add_argument("--grouped", action="store_true",
                    help="grouped expert GEMMs (one launch for all local experts) vs one cuBLAS call per expert")
    args = ap.parse_args()
    peak = None
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops")
    flush = torch.empty(64 * 1024 * 1024, device="cuda", dtype=torch.int32)
    if args.grouped:
        return grouped(args, peak, flush)
    shapes = [(8192, 6144, 2048), (8192, 2048, 2048), (8192, 16384, 2048), (8192, 2048, 8192),
              (8192, 49152, 2048), (4096, 12288, 4096), (4096, 22016, 4096), (4096, 4096, 11008)]
    if args.small:
        shapes = [(4096, 4096, 4096)]
    for (M, N, K) in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        dw32 = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        flops = 2.0 * M * N * K
        rows = [
            ("fwd  nt", lambda: gemm.gemm_nt(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
            ("dgrad nn", lambda: gemm.gemm_nn(dy, w, out=dx), lambda: torch.matmul(dy, w, out=dx)),
            ("wgrad tn+acc", lambda: gemm.gemm_tn(dy, x, out=dw32, accumulate=True),
             lambda: torch.matmul(dy.t(), x)),
        ]
        for name, ours, lib in rows:
            t_ours = time_fn(ours, args.iters, flush)
            t_lib = time_fn(lib, args.iters, flush)
            tf = flops / t_ours / 1e6
            line = (f"M={M} N={N} K={K} {name:13s} ours {t_ours:8.1f} us {tf:7.1f} TFLOP/s | "
                    f"cuBLAS {t_lib:8.1f} us {flops / t_lib / 1e6:7.1f} TFLOP/s")
            if peak:
                line += f" | {tf / peak:.3f} of measured"
            print(line, flush=True)
        ops.check_status(f"after shape {(M, N, K)}")


if __name__ == "__main__":
    main()
