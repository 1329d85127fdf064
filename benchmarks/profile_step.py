"""One or two optimizer steps of the flagship model with a single micro-batch each, for kernel
launch lists and profiler captures (the workload behind ``profiles/``).

    python benchmarks/profile_step.py [--layers 24] [--steps 2] [--grad-acc 1] [--seq 2048] [--mbs 4]

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
    args = ap.parse_args()
    torch.cuda.set_device(0)
    cfg = {
        "distributed": dict(tp_size=1, dp_size=1),
        "model": dict(name="HuggingFaceTB/SmolLM-1.7B", num_hidden_layers=args.layers, init_std=0.02),
        "training": dict(seed=0, learning_rate=3e-4, seq_length=args.seq, micro_batch_size=args.mbs,
                         gradient_accumulation_steps=args.grad_acc, num_samples=4096),
        "dataset": dict(name="synthetic"),
    }
    engine = TrainEngine(cfg, device=torch.device("cuda", 0))
    for i in range(args.steps):
        before = ops.launches()
        loss = engine.train_step()
        torch.cuda.synchronize()
        print(f"step {i}: loss {loss.item():.4f}, {ops.launches() - before} library kernels", flush=True)
    ops.check_status("profile_step")


if __name__ == "__main__":
    main()
