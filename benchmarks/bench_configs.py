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
from picotron_b200 import ops  # noqa: E402
from picotron_b200.engine import TrainEngine  # noqa: E402


def build_cfg(args, world):
    if args.config == "pp":
        tp = 2 if world >= 4 else 1
        pp = 2 if world >= 2 else 1
        dp = world // (tp * pp)
        layers = args.layers or 32
        return {
            "distributed": dict(tp_size=tp, pp_size=pp, dp_size=dp, pp_engine=args.pp_engine, num_virtual_stages=2,
                                sequence_parallel=tp > 1, vocab_parallel_ce=tp > 1, zero_stage=1 if dp > 1 else 0),
            "model": dict(name="meta-llama/Llama-2-7b-hf", num_hidden_layers=layers, init_std=0.02),
            "training": dict(seed=1, learning_rate=3e-4, seq_length=args.seq or 4096, micro_batch_size=1,
                             gradient_accumulation_steps=16, num_samples=1 << 14),
            "dataset": dict(name="synthetic"),
        }, f"tp{tp}xpp{pp}xdp{dp} {args.pp_engine}"
    if args.config == "moe":
        layers = args.layers or 16
        return {
            "distributed": dict(ep_size=world, ep_as_dp=world > 1),
            "model": dict(name="moe-ep8-bench", num_hidden_layers=layers, init_std=0.02, num_experts=64,
                          num_experts_per_tok=6, num_shared_experts=0, shared_expert_intermediate_size=2048,
                          ep_capacity_factor=args.capacity, ep_capacity_dropless=args.dropless, ep_fp8_dispatch=True,
                          ep_num_tiles=4, router_aux_loss_coef=1e-3, router_bias_update_rate=1e-3,
                          ep_backend=args.ep_backend),
            "training": dict(seed=1, learning_rate=3e-4, seq_length=args.seq or 4096, micro_batch_size=2,
                             gradient_accumulation_steps=1, num_samples=1 << 14),
            "dataset": dict(name="synthetic"),
        }, (f"ep{world} capacity{args.capacity} {'dropless' if args.dropless else 'drop'} fp8-dispatch"
            if args.capacity > 0 else
            (f"ep{world} dropless, peer-memory exchange with device-side layout" if args.ep_backend == "fused"
             else f"ep{world} tiled-4 variable-size exchange fp8-dispatch"))
    if args.config == "cp":
        layers = args.layers or 16
        seq = args.seq or 16384 * world
        return {
            "distributed": dict(cp_size=world, cp_attention=args.cp_attention),
            "model": dict(name="long-context-bench", num_hidden_layers=layers, init_std=0.02,
                          max_position_embeddings=seq),
            "training": dict(seed=1, learning_rate=3e-4, seq_length=seq, micro_batch_size=1,
                             gradient_accumulation_steps=1, num_samples=256),
            "dataset": dict(name="synthetic"),
        }, f"cp{world} {args.cp_attention}"
    raise SystemExit(f"unknown config {args.config}")


def active_params(mc) -> float:
    """Parameters that take part in one token's forward pass (routed experts count top-k times)."""
    h, L, v = mc.hidden_size, mc.num_hidden_layers, mc.vocab_size
    hd = h // mc.num_attention_heads
    attn = 2 * h * h + 2 * h * mc.num_key_value_heads * hd
    ffn = 3 * h * mc.intermediate_size
    experts = getattr(mc, "num_experts", 1) or 1
    if experts > 1:
        shared = getattr(mc, "shared_expert_intermediate_size", None) or \
            mc.intermediate_size * (getattr(mc, "num_shared_experts", 0) or 0)
        ffn = mc.num_experts_per_tok * 3 * h * mc.intermediate_size + 3 * h * shared + h * experts
    return L * (attn + ffn) + v * h


def mfu_percent(mc, seq_len: int, tokens_per_s_per_gpu: float, peak_flops: float) -> float:
    """The reference's formula (picotron/utils.py:51-62) on the active parameters."""
    flops_per_token = 6 * active_params(mc) + 12 * mc.num_hidden_layers * mc.hidden_size * seq_len
    return 100.0 * tokens_per_s_per_gpu * flops_per_token / peak_flops


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
        mfu_b200 = mfu_percent(eng.model_config, cfg["training"]["seq_length"], tps / world,
                               measured_peaks()["bf16_tflops"] * 1e12)
        mfu_h100 = mfu_percent(eng.model_config, cfg["training"]["seq_length"], tps / world, 989.5e12)
        print(json.dumps({"mfu_percent_b200_measured_peak": round(mfu_b200, 2),
                          "mfu_percent_h100_constant": round(mfu_h100, 2),"config": args.config, "layout": label, "n_gpus": world, "layers": cfg["model"]["num_hidden_layers"],
                          "seq_len": cfg["training"]["seq_length"], "tokens_per_step": eng.tokens_per_step,
                          "ms_per_step": round(step_ms, 2), "tokens_per_s": round(eng.tokens_per_step / step_ms * 1e3, 1),
                          "loss": round(lossv, 4), "peak_mem_gib": round(mem.item(), 1),
                          "gpu_launches": ops.launches() - l0, "steps": args.steps, "warmup": args.warmup}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
