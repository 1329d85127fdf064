"""Throughput of the other benchmark configurations through ``TrainEngine`` (the headline
SmolLM-1.7B configuration lives in ``bench.py``):

  pp    Llama-2-7B-shaped (32L, h4096, 32 heads, FFN 11008, vocab 32000), seq 4096, micro-batch 1,
        16 micro-batches, TP2 x PP2 x DP2 on 8 GPUs (TP2 x PP2 on 4, PP2 on 2), ``--pp-engine``
        interleaved | zb | 1f1b | afab | zbv
  moe   DeepSeek-style MoE (16L, h2048, 16 heads, 64 routed experts of FFN 1024, top-6, shared expert
        of FFN 2048, aux loss 1e-3 + loss-free bias, capacity 1.25, FP8 dispatch), seq 4096,
        micro-batch 2, EP = number of GPUs with EP acting as data parallelism for the dense weights
  cp    long-context Llama (16L, h2048, 32 q / 8 kv heads, FFN 5632, vocab 32000, rope theta 5e5),
        seq 16384 per GPU (131072 on 8), micro-batch 1, CP = number of GPUs, ``--cp-attention``
        ring | ulysses

Launch with ``python -m torch.distributed.run --nproc-per-node N benchmarks/bench_configs.py
--config <name> [--layers L] [--steps K] [--warmup W]``. CUDA-event timing, max over ranks; rank
0 prints one JSON line. ``--layers`` shrinks the depth for quick checks (reported in the line).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks.config_specs import flops_per_token, make_spec  # noqa: E402
from picotron_b200 import ops  # noqa: E402
from picotron_b200.engine import TrainEngine  # noqa: E402


def build_cfg(args, world):
    """(engine config, label) of a configuration; the definitions live in ``config_specs``."""
    variant = {"pp": args.pp_engine, "cp": args.cp_attention,
               "moe": "capacity" if args.capacity > 0 else "dropless"}[args.config]
    spec = make_spec(args.config, world, variant, args.layers, args.seq)
    cfg = spec["engine_cfg"]
    if args.config == "moe":
        cfg["model"]["ep_capacity_dropless"] = bool(args.dropless)
        if args.capacity <= 0:
            cfg["model"]["ep_backend"] = args.ep_backend
        else:
            cfg["model"]["ep_capacity_factor"] = args.capacity
    return cfg, spec["label"]


def mfu_percent(mc, seq_len: int, tokens_per_s_per_gpu: float, peak_flops: float, model: dict) -> float:
    return 100.0 * tokens_per_s_per_gpu * flops_per_token(model, seq_len) / peak_flops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["pp", "moe", "cp"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--pp-engine", default="interleaved")
    ap.add_argument("--cp-attention", default="ring")
    ap.add_argument("--dropless", action="store_true")
    ap.add_argument("--ep-backend", default="torch",
                    help="moe with --capacity 0: 'fused' = dropless exchange through peer memory, layout on device")
    ap.add_argument("--capacity", type=float, default=1.25,
                    help="moe: capacity factor; 0 selects the variable-size tiled exchange")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg, label = build_cfg(args, world)
    eng = TrainEngine(cfg, device=dev)
    for _ in range(args.warmup):
        eng.train_step()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ops.launches()
    s.record()
    loss = None
    for _ in range(args.steps):
        loss = eng.train_step()
    e.record()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ops.check_status("bench_configs")
    lossv = torch.tensor([eng.average_loss(loss)], device=dev)
    dist.all_reduce(lossv, op=dist.ReduceOp.MAX)   # the last pipeline stage holds the loss
    lossv = lossv.item()
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=dev)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    if rank == 0:
        step_ms = ms.item() / args.steps
        from picotron_b200.runtime.timing import measured_peaks
        tps = eng.tokens_per_step / step_ms * 1e3
        variant = {"pp": args.pp_engine, "cp": args.cp_attention,
                   "moe": "capacity" if args.capacity > 0 else "dropless"}[args.config]
        model = make_spec(args.config, world, variant, args.layers, args.seq)["model"]
        mfu_b200 = mfu_percent(eng.model_config, cfg["training"]["seq_length"], tps / world,
                               measured_peaks()["bf16_tflops"] * 1e12, model)
        mfu_h100 = mfu_percent(eng.model_config, cfg["training"]["seq_length"], tps / world, 989.5e12, model)
        print(json.dumps({"mfu_percent_b200_measured_peak": round(mfu_b200, 2),
                          "mfu_percent_h100_constant": round(mfu_h100, 2),"config": args.config, "layout": label, "n_gpus": world, "layers": cfg["model"]["num_hidden_layers"],
                          "seq_len": cfg["training"]["seq_length"], "tokens_per_step": eng.tokens_per_step,
                          "ms_per_step": round(step_ms, 2), "tokens_per_s": round(eng.tokens_per_step / step_ms * 1e3, 1),
                          "loss": round(lossv, 4), "peak_mem_gib": round(mem.item(), 1),
                          "gpu_launches": ops.launches() - l0, "steps": args.steps, "warmup": args.warmup}), flush=True)
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
