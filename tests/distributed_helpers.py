"""Spawn CPU ranks over gloo for the multi-process tests."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, fn, args, errors):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world_size)
        fn(rank, world_size, *args)
        dist.barrier()
    except Exception:
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world_size: int, *args, timeout: float = 120.0):
    """Run fn(rank, world_size, *args) on ``world_size`` gloo ranks; raise if any rank fails."""
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, errors)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    msgs = []
    while not errors.empty():
        rank, tb = errors.get()
        msgs.append(f"--- rank {rank} ---\n{tb}")
    if hung:
        msgs.append(f"{len(hung)} rank(s) did not finish within {timeout}s")
    bad = [p.exitcode for p in procs if p.exitcode not in (0, None)]
    if msgs or bad:
        raise AssertionError("distributed test failed\n" + "\n".join(msgs) + f"\nexit codes: {bad}")
