"""Micro-benchmark of the tcgen05 flash-attention kernels next to torch SDPA (library flash
attention) on the attention shapes of the benchmark configs. CUDA-event timing, median of
``--iters`` runs after warm-up, a 256 MiB buffer written between iterations to flush L2.

    python benchmarks/bench_attention.py [--iters 20] [--small]
"""
import argparse
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200 import ops  # noqa: E402
from picotron_b200.ops import attention as A  # noqa: E402


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    flush = torch.empty(64 * 1024 * 1024, device="cuda", dtype=torch.int32)
    shapes = [(4, 2048, 32, 32, 64), (1, 4096, 32, 32, 128), (1, 16384, 32, 8, 64), (2, 4096, 16, 16, 128)]
    if args.small:
        shapes = [(2, 2048, 16, 16, 64)]
    for (b, s, H, Hkv, d) in shapes:
        q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16)
        go = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
        fwd_flops = 4.0 * b * H * s * s * d / 2          # causal
        out, lse = A.flash_attention_forward(q, k, v, True)
        t_f = time_fn(lambda: A.flash_attention_forward(q, k, v, True), args.iters, flush)
        t_b = time_fn(lambda: A.flash_attention_backward(go, q, k, v, out, lse, True), args.iters, flush)
        qt, kt, vt = (t.transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
        gqa = H != Hkv

        def lib_fwd():
            return F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=gqa)
        o_lib = lib_fwd()
        t_lf = time_fn(lib_fwd, args.iters, flush)
        got = go.transpose(1, 2)

        def lib_bwd():
            torch.autograd.grad(o_lib, (qt, kt, vt), got, retain_graph=True)
        t_lb = time_fn(lib_bwd, args.iters, flush)
        print(f"b={b} s={s} H={H} Hkv={Hkv} d={d} causal | fwd ours {t_f:8.1f} us {fwd_flops / t_f / 1e6:6.1f} TF/s"
              f" lib {t_lf:8.1f} us {fwd_flops / t_lf / 1e6:6.1f} TF/s | bwd ours {t_b:8.1f} us "
              f"{2.5 * fwd_flops / t_b / 1e6:6.1f} TF/s lib {t_lb:8.1f} us {2.5 * fwd_flops / t_lb / 1e6:6.1f} TF/s",
              flush=True)
        ops.check_status("bench attention")


if __name__ == "__main__":
    main()
