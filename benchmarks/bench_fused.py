"""Each fused compute + collective path timed in isolation on N GPUs, next to the same operation done
with NCCL and a separate kernel, and reported as a fraction of its roofline: the slower of (FLOPs at the
measured GEMM peak) and (bytes that must cross NVLink per GPU at the measured peer bandwidth).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_fused.py [--iters 20]

CUDA-event timing on the launching stream, median over ``--iters`` after warm-up, max over ranks.
Shapes are those of the SmolLM-1.7B benchmark layer (hidden 2048, FFN 8192, 8192 tokens per
micro-batch), of the MoE benchmark (capacity 960, 64 experts of width 2048) and of the long-context
benchmark (16384 tokens per rank, 8 KV heads of 64).
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200 import ops  # noqa: E402
from picotron_b200.ops import gemm as gemm_ops  # noqa: E402
from picotron_b200.ops.fused_cp import CPFused  # noqa: E402
from picotron_b200.ops.fused_ep import EPFused  # noqa: E402
from picotron_b200.ops.fused_tp import TPFused  # noqa: E402
from picotron_b200.runtime.symm import SymmGroup  # noqa: E402
from picotron_b200.runtime.timing import roofline_fraction  # noqa: E402


def timed(fn, iters, world):
    """Median device time of fn() in seconds, max over ranks. A barrier before each timed call keeps
    the ranks aligned so the collective part is not hidden by skew."""
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e-3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def report(rank, name, t_fused, t_nccl, flops, link_bytes):
    if rank != 0:
        return
    rf = roofline_fraction(t_fused, flops=flops, nvlink_bytes=link_bytes)
    print(f"{name:44s} fused {t_fused * 1e6:8.1f} us | nccl+kernel {t_nccl * 1e6:8.1f} us | bound {rf['bound']:7s} "
          f"{rf['bound_seconds'] * 1e6:7.1f} us | {rf['fraction']:.2f} of roofline ({rf['peaks']})", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    sg = SymmGroup(dist.group.WORLD, device=dev)
    bf = torch.bfloat16

    # ---- tensor parallel with sequence parallelism: all-gather -> GEMM and GEMM -> reduce-scatter
    tokens, hidden, ffn = 8192, 2048, 8192
    m_local = tokens // world
    tp = TPFused(sg, m_local, max(hidden, 2 * ffn // world))
    x_shard = torch.randn(m_local, hidden, device=dev, dtype=bf)
    for name, n_out in (("qkv", 3 * hidden // world), ("gate+up", 2 * ffn // world)):
        w = torch.randn(n_out, hidden, device=dev, dtype=bf) * 0.02
        gathered = torch.empty(tokens, hidden, device=dev, dtype=bf)

        def fused():
            buf, slot, epoch = tp.gather_push(x_shard)
            tp.gated_gemm(buf, w, slot, epoch, False, n_out)
            tp.wait_gather(slot, epoch)

        def nccl():
            dist.all_gather_into_tensor(gathered, x_shard)
            gemm_ops.gemm_nt(gathered, w)

        report(rank, f"all-gather -> GEMM ({name}, tp{world})", timed(fused, args.iters, world),
               timed(nccl, args.iters, world), 2.0 * tokens * n_out * hidden,
               (world - 1) * m_local * hidden * 2)
    for name, k_loc in (("out_proj", hidden // world), ("down_proj", ffn // world)):
        w = torch.randn(hidden, k_loc, device=dev, dtype=bf) * 0.02
        a = torch.randn(tokens, k_loc, device=dev, dtype=bf)
        shard = torch.empty(m_local, hidden, device=dev, dtype=bf)

        def fused():
            sb, slot, epoch = tp.scatter_gemm(a, w, False, hidden)
            tp.scatter_sum(sb, slot, epoch, hidden)

        def nccl():
            dist.reduce_scatter_tensor(shard, gemm_ops.gemm_nt(a, w))

        report(rank, f"GEMM -> reduce-scatter ({name}, tp{world})", timed(fused, args.iters, world),
               timed(nccl, args.iters, world), 2.0 * tokens * hidden * k_loc,
               (world - 1) * m_local * hidden * 2)

    # ---- expert parallel: capacity dispatch (bf16 and FP8 with 1x128 block scales) and combine
    E, C, d, top_k = 64, 960, 2048, 6
    L = E // world
    ep = EPFused(sg, L, C, d)
    n_tok = 8192
    toks = torch.randn(n_tok, d, device=dev, dtype=bf)
    row_of_slot = torch.randint(0, n_tok * top_k, (E * C,), device=dev, dtype=torch.int32)
    send = torch.randn(E * C, d, device=dev, dtype=bf)
    recv = torch.empty_like(send)
    rows_remote = (world - 1) * L * C
    for quant in (False, True):
        def fused():
            ep.dispatch_rows(toks, row_of_slot, top_k, quant)

        def nccl():
            # gather the rows into the send buffer, then exchange (bf16; the reference's FP8 variant adds
            # separate quantise / scale-exchange / dequantise kernels)
            src = toks[(row_of_slot // top_k).long()]
            dist.all_to_all_single(recv, src)

        payload = d * (1 if quant else 2) + (d // 128 * 4 if quant else 0)
        report(rank, f"MoE dispatch ({'fp8 1x128' if quant else 'bf16'}, ep{world})", timed(fused, args.iters, world),
               timed(nccl, args.iters, world), 0.0, rows_remote * payload)
    out_rows = torch.randn(L, world * C, d, device=dev, dtype=bf)

    def fused():
        ep.to_source_major(out_rows)

    def nccl():
        dist.all_to_all_single(recv, out_rows.view(L, world, C, d).transpose(0, 1).reshape(E * C, d))

    report(rank, f"MoE combine exchange (bf16, ep{world})", timed(fused, args.iters, world),
           timed(nccl, args.iters, world), 0.0, rows_remote * d * 2)

    # ---- context parallel: K/V gather for causal attention
    s_loc, kv_cols = 16384, 8 * 64
    cp = CPFused(sg, 1, s_loc, kv_cols)
    k = torch.randn(1, s_loc, 8, 64, device=dev, dtype=bf)
    v = torch.randn_like(k)
    kv_all = torch.empty(world * 2 * s_loc * kv_cols, device=dev, dtype=bf)
    kv_loc = torch.cat([k.flatten(), v.flatten()])

    def fused():
        c, slot, epoch = cp.gather_kv(k, v)
        cp.wait(slot, epoch)

    def nccl():
        dist.all_gather_into_tensor(kv_all, kv_loc)

    report(rank, f"K/V gather (cp{world}, 16384 tokens per rank)", timed(fused, args.iters, world),
           timed(nccl, args.iters, world), 0.0, (world - 1) * 2 * s_loc * kv_cols * 2)
    ops.check_status("bench_fused")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
