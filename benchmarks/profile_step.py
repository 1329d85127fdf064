"""One or two optimizer steps of the flagship model with a single micro-batch each, for kernel
launch lists and profiler captures (the workload behind ``profiles/``).

    python benchmarks/profile_step.py [--layers 24] [--steps 2] [--grad-acc 1] [--seq 2048] [--mbs 4]
    python -m torch.distributed.run --nproc-per-node 2 ... benchmarks/profile_step.py --config moe --layers 4

Under ``torch.distributed.run`` with N processes the model is tensor-parallel over all of them
(sequence parallel, vocabulary-parallel cross entropy) and the step time (CUDA events, max over ranks) is
printed too, which separates launch-bound from device-bound regimes when ``--mbs`` is varied.

Prints the number of kernels of this library launched per step so a capture can skip the first
(warm-up) step with ``-s``.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from picotron_b200 import ops  # noqa: E402
from picotron_b200.engine import TrainEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--grad-acc", type=int, default=1)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--config", default="smollm", choices=("smollm", "moe", "cp", "pp"),
                    help="smollm: the flagship model, tensor parallel over all ranks; moe / cp / pp: the benchmark "
                         "configuration of that name (benchmarks/config_specs.py) at --layers layers")
    ap.add_argument("--variant", default=None)
    ap.add_argument("--kernel-table", action="store_true",
                    help="after the timed steps, run one more step under torch.profiler and print rank 0's "
                         "kernels by device time (shares only: a profiled step is slower than a plain one)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl")
    cfg = {
        "distributed": dict(tp_size=world, dp_size=1, sequence_parallel=world > 1, vocab_parallel_ce=world > 1),
        "model": dict(name="HuggingFaceTB/SmolLM-1.7B", num_hidden_layers=args.layers, init_std=0.02),
        "training": dict(seed=0, learning_rate=3e-4, seq_length=args.seq, micro_batch_size=args.mbs,
                         gradient_accumulation_steps=args.grad_acc, num_samples=4096),
        "dataset": dict(name="synthetic"),
    }
    if args.config != "smollm":
        from benchmarks.config_specs import make_spec
        cfg = make_spec(args.config, world, args.variant, layers=args.layers)["engine_cfg"]
    engine = TrainEngine(cfg, device=torch.device("cuda", local))
    for i in range(args.steps):
        before = ops.launches()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        loss = engine.train_step()
        e.record()
        torch.cuda.synchronize()
        ms = torch.tensor([s.elapsed_time(e)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if local == 0:
            print(f"step {i}: loss {loss.item():.4f}, {ops.launches() - before} library kernels, "
                  f"{ms.item():.1f} ms", flush=True)
    ops.check_status("profile_step")
    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            engine.train_step()
            torch.cuda.synchronize()
        if local == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=70),
                  flush=True)
            # busy time (union of kernel intervals) against the span from first to last kernel
            iv = sorted((ev.time_range.start, ev.time_range.end) for ev in prof.events()
                        if ev.device_type == torch.autograd.DeviceType.CUDA)
            if iv:
                busy, cur_s, cur_e = 0.0, iv[0][0], iv[0][1]
                for a, b in iv[1:]:
                    if a > cur_e:
                        busy += cur_e - cur_s
                        cur_s, cur_e = a, b
                    else:
                        cur_e = max(cur_e, b)
                busy += cur_e - cur_s
                span = iv[-1][1] - iv[0][0]
                print(f"device busy {busy / 1e3:.1f} ms of a {span / 1e3:.1f} ms span "
                      f"({100.0 * busy / span:.1f} %), {len(iv)} kernels/copies", flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
