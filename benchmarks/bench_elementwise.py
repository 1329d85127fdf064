"""Micro-benchmark of the memory-bound kernels (RMSNorm, SwiGLU, RoPE, cross entropy, AdamW,
embedding) at the SmolLM-1.7B micro-batch shapes: achieved GB/s of algorithmic traffic and the
fraction of the measured copy bandwidth (MEASURED_PEAKS.json). CUDA events, median, L2 flushed
between iterations.

    python benchmarks/bench_elementwise.py [--iters 20] [--small]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200 import ops  # noqa: E402


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
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak = json.load(open(pk))["hbm_gbs"] if os.path.exists(pk) else 6650.0
    e = ops.ext()
    dev = "cuda"
    M, H, I, V = (8192, 2048, 8192, 49152) if not args.small else (4096, 2048, 4096, 16384)
    flush = torch.empty(64 * 1024 * 1024, device=dev, dtype=torch.int32)
    bf = torch.bfloat16
    x = torch.randn(M, H, device=dev, dtype=bf)
    res = torch.randn(M, H, device=dev, dtype=bf)
    w = torch.ones(H, device=dev, dtype=bf)
    y, h = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(M, device=dev)
    dh = torch.empty_like(x)
    part = torch.empty(e.rmsnorm_bwd_num_partials() * H, device=dev)
    dw = torch.zeros(H, device=dev)
    gu = torch.randn(M, 2 * I, device=dev, dtype=bf)
    act = torch.empty(M, I, device=dev, dtype=bf)
    dgu = torch.empty_like(gu)
    logits = torch.randn(M, V, device=dev, dtype=bf)
    tgt = torch.randint(0, V, (M,), device=dev)
    stats = torch.empty(M, 3, device=dev)
    loss = torch.empty(M, device=dev)
    n = 256 * 1024 * 1024 if not args.small else 32 * 1024 * 1024
    p = torch.randn(n, device=dev).to(bf)
    g = torch.randn(n, device=dev)
    m1, m2 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    qk = torch.randn(4, M // 4, 32, 64, device=dev, dtype=bf)
    cos = torch.randn(M // 4, 32, device=dev)
    emb_w = torch.randn(V, H, device=dev, dtype=bf)
    ids = torch.randint(0, V, (M,), device=dev)
    emb_out = torch.empty(M, H, device=dev, dtype=bf)
    emb_dw = torch.zeros(V, H, device=dev)
    E, K = 64, 6
    r_logits = torch.randn(4 * M, E, device=dev, dtype=bf)
    r_probs = torch.empty(4 * M, E, device=dev)
    r_idx = torch.empty(4 * M, K, device=dev, dtype=torch.int32)
    r_w = torch.empty(4 * M, K, device=dev)
    r_counts = torch.zeros(E, device=dev, dtype=torch.int32)
    mb, ms, mh, md = 1, M, 32, 64
    oa = torch.randn(mb, ms, mh, md, device=dev)
    ob = torch.randn(mb, ms, mh, md, device=dev, dtype=bf)
    la, lb = torch.randn(mb, mh, ms, device=dev), torch.randn(mb, mh, ms, device=dev)
    lnew = torch.empty_like(la)
    cases = [
        ("rmsnorm_fwd(+residual)", lambda: e.rmsnorm_fwd(x, res, w, y, h, rstd, M, H, 1e-5), M * H * 2 * 4),
        ("rmsnorm_bwd", lambda: e.rmsnorm_bwd(x, h, w, rstd, res, dh, part, dw, None, True, M, H), M * H * 2 * 4),
        ("swiglu_fwd", lambda: e.swiglu_fwd(gu, 2 * I, act, M, I, None), M * I * 2 * 3),
        ("swiglu_bwd", lambda: e.swiglu_bwd(act, gu, 2 * I, dgu, 2 * I, M, I, None), M * I * 2 * 5),
        ("rope_inplace", lambda: e.rope_inplace(qk, qk.stride(1), M, M // 4, 0, 32, 64, cos, cos, 1), M * 2048 * 2 * 2),
        ("ce_stats", lambda: e.ce_stats(logits, V, tgt, stats, M, V, 0), M * V * 2),
        ("ce_loss_grad(in place)", lambda: e.ce_loss_grad(logits, V, tgt, stats, loss, logits, V, 1.0, M, V, 0), M * V * 2 * 2),
        ("adamw(bf16 p, fp32 g/m/v)", lambda: e.adamw(p, None, g, m1, m2, n, 1e-4, 0.9, 0.95, 1e-8, 0.01, 0.1, 0.1, 1.0, True),
         n * (2 * 2 + 4 * 6)),
        ("embedding_fwd", lambda: e.embedding_fwd(emb_w, ids, emb_out, M, H, V, 0), M * H * 2 * 2),
        ("embedding_bwd(fp32 acc)", lambda: e.embedding_bwd(x, ids, emb_dw, M, H, V, 0), M * H * (2 + 4 * 2)),
        ("moe_route(E=64,k=6)", lambda: e.moe_route(r_logits, None, r_probs, r_idx, r_w, r_counts, K, True),
         4 * M * (E * 2 + E * 4 + K * 8)),
        ("attn_merge(fp32 acc += bf16 block)", lambda: e.attn_merge(oa, la, ob, lb, oa, lnew),
         mb * ms * mh * md * (4 + 2 + 4)),
    ]
    for name, fn, nbytes in cases:
        t = time_fn(fn, args.iters, flush)
        gbs = nbytes / t / 1e3
        print(f"{name:28s} {t:9.1f} us {gbs:8.1f} GB/s  {gbs / peak:.3f} of measured copy bandwidth", flush=True)
    ops.check_status("bench elementwise")


if __name__ == "__main__":
    main()
