"""Training entry point: ``torchrun --nproc_per_node N train.py --config <config.json>``.

Follows the reference's train.py:84-379 — environment, process group, topology, data loader,
model + parallel wrappers, optimizer, optional checkpoint load, then the step loop with the same
one-line log format (``Step | Loss | Global batch size | Tokens/s | Tokens/s/GPU | Tokens | MFU |
Memory usage``, parsed by extract_metrics.py) — built on ``picotron_b200.engine.TrainEngine``,
which also wires in sequence parallelism, vocabulary-parallel cross entropy, ZeRO and all five
pipeline schedules. Step time is measured on the device with CUDA events and reduced with MAX over
ranks; MFU is printed against the H100 constant of the reference formula (for comparison with its
published numbers), the JSONL metrics file also has the figure against the measured B200 peak.
"""
import argparse
import datetime
import json
import os
import time

import torch
import torch.distributed as dist

from picotron_b200 import process_group_manager as pgm
from picotron_b200.checkpoint import CheckpointManager
from picotron_b200.config import load_config, world_size_of
from picotron_b200.engine import TrainEngine
from picotron_b200.runtime.status import raise_if_failed
from picotron_b200.runtime.watchdog import StepWatchdog
from picotron_b200.utils import (get_mfu, get_num_params, measured_peak_flops, print, set_all_seed,
                                 to_readable_format)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--profile", type=int, default=0, help="wrap this many steps in torch.profiler")
    args = ap.parse_args()
    cfg = load_config(args.config)
    d, t = cfg["distributed"], cfg["training"]
    for k in ("OMP_NUM_THREADS", "TOKENIZERS_PARALLELISM"):
        os.environ[k] = str(cfg["environment"][k])
    use_cpu = d["use_cpu"] or not torch.cuda.is_available()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == world_size_of(cfg), \
        f"WORLD_SIZE ({world}) != tp*cp*ep*pp*dp ({world_size_of(cfg)})"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if use_cpu:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(minutes=3))
    else:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(minutes=3),
                                device_id=device)
    pgm.setup_process_group_manager(d["tp_size"], d["cp_size"], d["pp_size"], d["dp_size"], d["ep_size"])
    m = pgm.process_group_manager
    is_log_rank = m.tp_rank == 0 and m.dp_rank == 0 and m.cp_rank == 0 and m.ep_rank == 0 and m.pp_is_last_stage
    set_all_seed(t["seed"])
    cfg["distributed"]["use_cpu"] = use_cpu
    engine = TrainEngine(cfg, device=device)
    num_params = get_num_params(engine.model)
    print(f"Number of parameters: {to_readable_format(num_params)}", is_print_rank=is_log_rank)
    print(str(m), is_print_rank=is_log_rank)

    wandb = None
    if is_log_rank and cfg["logging"]["use_wandb"]:
        import wandb as _wandb
        wandb = _wandb
        wandb.init(project=cfg["logging"]["project_name"], name=cfg["logging"]["run_name"], config=cfg)
    ckpt = CheckpointManager()
    if cfg["checkpoint"]["load_path"]:
        steps, tokens = ckpt.load_checkpoint(engine.model, engine.optimizer, cfg["checkpoint"]["load_path"],
                                             data_loader=engine.data_loader,
                                             sharded_optimizer=engine.optimizer_is_sharded)
        engine.trained_steps, engine.trained_tokens = steps, tokens
    metrics_path = cfg["logging"].get("metrics_jsonl")
    if cfg["logging"].get("step_breakdown") and metrics_path:
        # per-step device time of forward+backward / optimizer sections, MAX over ranks, in the JSONL
        from picotron_b200.runtime.timing import EventTimer
        engine.timer = EventTimer(device)
    watchdog = StepWatchdog.from_env(rank, world)
    prof = None
    if args.profile > 0:
        prof = torch.profiler.profile(schedule=torch.profiler.schedule(wait=1, warmup=1, active=args.profile),
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler("profiler_traces"))
        prof.start()

    dist.barrier()
    model_cfg = engine.model_config
    # logging.log_frequency = N: the host synchronises with the device, reads the loss and prints only
    # every N-th step (and at checkpoints and at the end); in between, steps are enqueued back to back
    # and the printed step time is the mean over the window. N = 1 is the reference's behaviour
    # (train.py:323-379 there: one loss all-reduce and .item() per step).
    log_every = max(1, int(cfg["logging"].get("log_frequency") or 1))
    in_window = 0
    while t["max_tokens"] is None or engine.trained_tokens < t["max_tokens"]:
        if in_window == 0:
            if device.type == "cuda":
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            else:
                t0 = time.perf_counter()
        loss_t = engine.train_step()
        in_window += 1
        step = engine.trained_steps
        watchdog.beat(step)
        last = step >= t["total_train_steps"] or (t["max_tokens"] is not None
                                                  and engine.trained_tokens >= t["max_tokens"])
        if not (step % log_every == 0 or last or step % cfg["checkpoint"]["save_frequency"] == 0):
            if prof is not None:
                prof.step()
            continue
        if device.type == "cuda":
            end.record()
            end.synchronize()
            # a kernel that gave up a bounded wait (peer flag, mbarrier) or overflowed a dropless
            # expert buffer only records that and returns: stop here, before the state it left
            # behind is trained on or written to a checkpoint (the device is already idle, so this
            # costs one small read)
            raise_if_failed(f"train step {engine.trained_steps}")
            step_ms = torch.tensor([start.elapsed_time(end) / in_window], device=device)
        else:
            step_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / in_window])
        in_window = 0
        dist.all_reduce(step_ms, op=dist.ReduceOp.MAX)
        loss = engine.average_loss(loss_t)
        sections = engine.timer.collect() if engine.timer is not None else None
        step_s = float(step_ms.item()) / 1e3
        tok_s = engine.tokens_per_step / step_s
        tok_s_gpu = tok_s / world
        mfu = get_mfu(tok_s_gpu, num_params, num_layers=model_cfg.num_hidden_layers,
                      hidden_size=model_cfg.hidden_size, seq_len=t["seq_length"])
        mem = torch.cuda.memory_reserved() / 1e9 if device.type == "cuda" else 0.0
        max_tok = ("/" + to_readable_format(t["max_tokens"])) if t["max_tokens"] else ""
        print(f"[rank {m.global_rank}] Step: {step:<5d} | Loss: {loss:6.4f} | "
              f"Global batch size: {to_readable_format(engine.tokens_per_step):>7s} | "
              f"Tokens/s: {to_readable_format(tok_s):>7s} | "
              f"Tokens/s/GPU: {to_readable_format(tok_s_gpu):>7s} | "
              f"Tokens: {to_readable_format(engine.trained_tokens):>7s}{max_tok} | "
              f"MFU: {mfu:5.2f}% | Memory usage: {mem:6.2f}GB", is_print_rank=is_log_rank)
        if is_log_rank and metrics_path:
            with open(metrics_path, "a") as fh:
                fh.write(json.dumps({"step": step, "loss": loss, "step_ms": step_s * 1e3, "tokens_per_s": tok_s,
                                     "tokens_per_s_per_gpu": tok_s_gpu, "mfu_h100_const": mfu,
                                     "mfu_b200_measured": get_mfu(tok_s_gpu, num_params,
                                                                  theoretical_flops=measured_peak_flops(),
                                                                  num_layers=model_cfg.num_hidden_layers,
                                                                  hidden_size=model_cfg.hidden_size,
                                                                  seq_len=t["seq_length"]),
                                     "memory_gb": mem, **({"sections_ms": sections} if sections else {})}) + "\n")
        if wandb is not None:
            wandb.log({"loss": loss, "tokens_per_step": engine.tokens_per_step, "tokens_per_second": tok_s,
                       "mfu": mfu, "tokens_per_second_per_gpu": tok_s_gpu, "memory_usage": mem,
                       "trained_tokens": engine.trained_tokens})
        if prof is not None:
            prof.step()
        if step % cfg["checkpoint"]["save_frequency"] == 0:
            if device.type == "cuda":
                raise_if_failed("before saving a checkpoint")
            ckpt.save_checkpoint(engine.model, engine.optimizer, step, engine.trained_tokens,
                                 os.path.join(cfg["checkpoint"]["save_dir"], str(step)),
                                 data_loader=engine.data_loader, sharded_optimizer=engine.optimizer_is_sharded)
        if step >= t["total_train_steps"]:
            break
    if prof is not None:
        prof.stop()
    if wandb is not None:
        wandb.finish()
    watchdog.stop()
    engine.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
