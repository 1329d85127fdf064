"""Headline benchmark: training throughput (tokens/s, MFU) of the SmolLM-1.7B-shaped Llama
(24 layers, hidden 2048, 32 heads, FFN 8192, vocab 49152; seq 2048, micro-batch 4, 8 gradient
accumulation steps, AdamW lr 3e-4, bf16, random init N(0, 0.02), seeded uniform tokens) on N
GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...     # the unmodified reference package from baseline/_ref
    ... bench.py --config moe|cp|pp [--variant V] [--layers L]   # the other benchmark configurations
                                                                 # (benchmarks/config_specs.py), both arms

Layouts (all with sequence parallelism, vocabulary-parallel cross entropy and ZeRO-1 where the
axis exists): 1 GPU = no parallelism, 2 = TP2, 4 = TP4, 8 = DP2 x TP4.

Two measurements per run, both as max over ranks:
* ``value``: K optimizer steps timed with CUDA events on the device, micro-batches already
  resident on the GPU (kernel-only view)
* ``e2e``: the same K steps driven through ``TrainEngine.train_step()`` with every
  micro-batch copied from pinned host memory and the step's loss read back to the host

The working set of a step (3.4 GB of parameters, several GB of activations) is far larger
than the 126 MB L2, so no explicit flush runs between iterations. Rank 0 prints one JSON line.

On 2 GPUs and more the same process then measures the mixture-of-experts configuration with EP = N (same
arm, 3 steps after 3 warm-up steps) and reports it under ``"secondary"`` of that line. The headline
cannot lose by it: the line exists before the secondary measurement starts, an exception there only
records ``{"unavailable": ...}``, and a deadline thread prints the line and ends every rank with exit code 0
should the secondary part hang (``PICO_BENCH_SECONDARY=0`` skips it, ``PICO_BENCH_SECONDARY_TIMEOUT`` sets the
deadline in seconds).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
from types import SimpleNamespace

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MODEL = dict(name="HuggingFaceTB/SmolLM-1.7B", hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
             num_attention_heads=32, num_key_value_heads=32, vocab_size=49152, max_position_embeddings=2048,
             rms_norm_eps=1e-5, rope_theta=10000.0)
SEQ, MBS, GRAD_ACC, LR = 2048, 4, 8, 3e-4
LAYOUTS = {1: dict(tp=1, dp=1), 2: dict(tp=2, dp=1), 4: dict(tp=4, dp=1), 8: dict(tp=4, dp=2)}
PUBLISHED_MFU_PERCENT = 50.0          # "nearly 50%" SmolLM-1.7B on 8 x H100 (reference README.md:7)
H100_PEAK = 989.5e12                  # constant of the reference's MFU formula


def num_params(m=MODEL) -> float:
    h, i, L, v = m["hidden_size"], m["intermediate_size"], m["num_hidden_layers"], m["vocab_size"]
    kv = m["num_key_value_heads"] * (h // m["num_attention_heads"])
    per_layer = h * h * 2 + 2 * h * kv + 3 * h * i + 2 * h
    return float(L * per_layer + 2 * v * h + h)


def flops_per_token() -> float:
    return 6.0 * num_params() + 12.0 * MODEL["num_hidden_layers"] * MODEL["hidden_size"] * SEQ


class ClockSampler:
    """Samples SM clock and throttle reasons of this process's GPU with nvidia-smi while the
    timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc, self.path = None, None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, smax = [], set(), None
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    smax = float(parts[1])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            clocks.sort()
            out.update(sm_mhz=clocks[len(clocks) // 2], sm_max_mhz=smax, reasons=sorted(reasons),
                       samples=len(clocks))
        return out


def setup_distributed(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == n_gpus, f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    if not dist.is_initialized():
        dist.init_process_group(backend="nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local_rank))
    return rank, local_rank, world


def timed(fn, steps: int, device) -> float:
    """Milliseconds for ``steps`` calls of fn, CUDA events bracketed by barrier + synchronize,
    max over ranks."""
    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([start.elapsed_time(end)], device=device, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def result_line(args, layout, world, ms_total, e2e_ms_total, h2d, d2h, clocks, launches, impl, extra=None):
    tokens_per_step = MBS * SEQ * GRAD_ACC * layout["dp"]
    ms_per_step = ms_total / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    per_gpu = value / world
    fpt = flops_per_token()
    from picotron_b200.utils import measured_peak_flops
    line = {
        "metric": "training throughput, SmolLM-1.7B (tokens/s, whole job)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
        # 1, 2 and 4 GPUs split the same global batch of 32 sequences (tensor parallelism: total work fixed);
        # 8 GPUs add a data-parallel replica and double the global batch
        "scaling": "strong" if world <= 4 else "weak",
        "vs_baseline": round(per_gpu * fpt / H100_PEAK * 100.0 / PUBLISHED_MFU_PERCENT, 4),
        "dtype": "bf16", "data": "synthetic seeded uniform tokens, random-init N(0,0.02) weights",
        "impl": impl,
        "mfu_percent_h100_constant": round(per_gpu * fpt / H100_PEAK * 100.0, 2),
        "mfu_percent_b200_measured_peak": round(per_gpu * fpt / measured_peak_flops() * 100.0, 2),
        "config": {"model": "SmolLM-1.7B-shaped Llama (24L h2048 32h ffn8192 v49152)",
                   "global_batch": MBS * GRAD_ACC * layout["dp"], "seq_len": SEQ, "micro_batch": MBS,
                   "grad_accum": GRAD_ACC, "optimizer": "AdamW lr 3e-4",
                   "parallelism": f"dp{layout['dp']}xtp{layout['tp']}"
                                  + ("+sp+vocab_ce" if layout["tp"] > 1 else "")
                                  + ("+zero1" if layout["dp"] > 1 else ""),
                   "scaling_note": "global batch 32 sequences at 1/2/4 GPUs (fixed total work, tp1/tp2/tp4); "
                                   "64 at 8 GPUs (dp2 x tp4: per-replica work fixed)",
                   "l2": "per-step working set (GBs of parameters and activations) exceeds the 126 MB L2; no explicit flush",
                   "vs_baseline_note": "per-GPU MFU by the reference formula (H100 constant) / published ~50% MFU on 8xH100"},
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                   "reasons": clocks.get("reasons", [])},
        "e2e": {"value": round(tokens_per_step / (e2e_ms_total / args.steps / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    if extra:
        line.update(extra)
    return line


class Deadline:
    """Ends the process with exit code 0 when ``seconds`` have passed, after printing ``line`` (rank 0 holds
    one, the other ranks hold None) unless it was printed already. Guards the part of a run that comes
    after the headline measurement."""

    def __init__(self, seconds: float, line):
        self.line = line
        self.lock = threading.Lock()
        self.printed = False
        self.timer = threading.Timer(seconds, self._fire)
        self.timer.daemon = True

    def start(self):
        self.timer.start()
        return self

    def print_line(self, line) -> None:
        """Print the result line once (whichever of the main thread and the deadline comes first)."""
        with self.lock:
            if not self.printed and line is not None:
                print(json.dumps(line), flush=True)
            self.printed = True

    def _fire(self):
        self.print_line(self.line)
        sys.stdout.flush()
        os._exit(0)

    def cancel(self):
        self.timer.cancel()


def finish_with_secondary(args, line, rank, world, device, reference: bool, teardown, release=None) -> None:
    """Print the headline ``line`` (rank 0; None elsewhere), adding the mixture-of-experts measurement with
    EP = world under ``"secondary"`` when the run has 2 GPUs or more, then run ``teardown``. ``release``
    frees what the headline measurement held (it runs first; if it fails the secondary part is skipped).
    Everything after the headline measurement happens under a deadline."""
    wanted = world >= 2 and os.environ.get("PICO_BENCH_SECONDARY", "1") != "0"
    timeout = float(os.environ.get("PICO_BENCH_SECONDARY_TIMEOUT", "240"))
    fallback = dict(line, secondary={"unavailable": f"not finished within {timeout:.0f} s"}) if line is not None and wanted \
        else line
    deadline = Deadline(timeout, fallback).start()
    try:
        if release is not None:
            try:
                release()
            except BaseException as exc:                         # noqa: BLE001
                if line is not None and wanted:
                    line = dict(line, secondary={"unavailable": f"release failed: {type(exc).__name__}: {exc}"[:300]})
                wanted = False
        if wanted:
            try:
                sub = SimpleNamespace(gpus=world, steps=min(args.steps, 3), warmup=3, config="moe", variant=None,
                                      layers=0, seq=0, impl="reference" if reference else "ours")
                sec = measure_config(sub, reference)
            except BaseException as exc:                         # noqa: BLE001  the headline must survive anything
                sec = {"unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:300] if str(exc) else ''}"}
            if line is not None:
                line = dict(line, secondary=sec if sec is not None else {"unavailable": "no result on rank 0"})
        deadline.print_line(line)
        try:
            teardown()
        except Exception as exc:                                 # noqa: BLE001  the result is out: report, do not fail
            print(f"tear-down failed: {type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
    finally:
        deadline.cancel()


# ------------------------------------------------------------------------------------------ ours
def run_ours(args):
    rank, local_rank, world = setup_distributed(args.gpus)
    device = torch.device("cuda", local_rank)
    layout = LAYOUTS[world]
    from picotron_b200 import ops
    from picotron_b200.engine import TrainEngine
    cfg = {
        "distributed": dict(tp_size=layout["tp"], dp_size=layout["dp"], sequence_parallel=layout["tp"] > 1,
                            vocab_parallel_ce=layout["tp"] > 1, zero_stage=1 if layout["dp"] > 1 else 0),
        "model": dict(MODEL, init_std=0.02, dtype="bfloat16"),
        "training": dict(seed=1234, learning_rate=LR, seq_length=SEQ, micro_batch_size=MBS,
                         gradient_accumulation_steps=GRAD_ACC, num_samples=1 << 16),
        "dataset": dict(name="synthetic"),
    }
    engine = TrainEngine(cfg, device=device)
    g = torch.Generator().manual_seed(99 + engine.pgm.dp_rank)
    resident = [(torch.randint(0, MODEL["vocab_size"], (MBS, SEQ), generator=g).to(device),
                 torch.randint(0, MODEL["vocab_size"], (MBS, SEQ), generator=g).to(device))
                for _ in range(GRAD_ACC)]

    def device_step():
        engine.train_step(device_batches=resident)

    last = {}

    def e2e_step():
        last["loss"] = float(engine.train_step().item())

    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    l0 = ops.launches()
    ms = timed(device_step, args.steps, device)
    launches = ops.launches() - l0
    clocks = sampler.stop() if sampler else {}
    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps, device)
    ops.check_status("bench")
    h2d = GRAD_ACC * 2 * MBS * SEQ * 8      # input_ids + target_ids, int64, per rank
    d2h = 4                                  # the fp32 step loss
    line = result_line(args, layout, world, ms, e2e_ms, h2d, d2h, clocks, launches, "picotron_b200",
                       {"final_loss": last.get("loss")}) if rank == 0 else None
    held = [engine, resident]
    del engine, resident

    def release():
        held[0].close()
        held.clear()
        torch.cuda.empty_cache()

    finish_with_secondary(args, line, rank, world, device, False, dist.destroy_process_group, release)


# ------------------------------------------------------------------------------------- reference
def run_reference(args):
    out = _reference_headline(args)
    if out is None:
        return
    line, rank, world, device = out

    def release():                    # the headline model and optimizer are out of scope: release their memory
        import gc
        gc.collect()
        torch.cuda.empty_cache()

    finish_with_secondary(args, line, rank, world, device, True, dist.destroy_process_group, release)


def _reference_headline(args):
    """The reference's arm of the headline configuration. Returns (result line on rank 0 else None, rank,
    world, device), or None after printing why the reference is unavailable."""
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "picotron")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/picotron is not installed"}))
        return None
    try:
        rank, local_rank, world = setup_distributed(args.gpus)
        device = torch.device("cuda", local_rank)
        layout = LAYOUTS[world]
        os.environ["FLASH_ATTEN"] = "1"
        os.environ["DEVICE"] = "cuda"
        os.environ["DTYPE"] = "bfloat16"
        import_reference(ref_root)
        import torch.nn.functional as F
        import picotron.process_group_manager as rpgm
        from picotron.model import Llama as RefLlama
        from picotron.tensor_parallel.tensor_parallel import apply_tensor_parallel as ref_apply_tp
        from picotron.tensor_parallel.tp_communications import vocab_parallel_cross_entropy as ref_vce
        from picotron.data_parallel.zero import DataParallelZero as RefZero, ShardedOptimizer as RefSharded
        from picotron.utils import set_all_seed

        rpgm.setup_process_group_manager(tp_size=layout["tp"], cp_size=1, pp_size=1, dp_size=layout["dp"], ep_size=1)
        pg = rpgm.process_group_manager
        set_all_seed(1234)
        mcfg = SimpleNamespace(**{k: v for k, v in MODEL.items() if k != "name"}, num_experts=1)
        model = RefLlama(mcfg)
        tp = layout["tp"]
        if tp > 1:
            ref_apply_tp(model, sequence_parallel=True, vocab_parallel_ce=True)
        with torch.no_grad():
            for p in model.parameters():          # N(0, 0.02) like our arm (norm weights stay 1)
                if p.dim() > 1:
                    p.normal_(0.0, 0.02)
        model.to(torch.bfloat16).to(device)
        if layout["dp"] > 1:
            dp_model = RefZero(model, stage=1)
            optimizer = RefSharded(dp_model, torch.optim.AdamW, lr=LR)
        else:
            dp_model = model
            optimizer = torch.optim.AdamW(model.parameters(), lr=LR)
        norm_params = [p for n, p in model.named_parameters() if "layernorm" in n or "final_norm" in n]

        g = torch.Generator().manual_seed(99 + pg.dp_rank)

        def host_batch():
            rows = torch.randint(0, MODEL["vocab_size"], (MBS, SEQ + 1), generator=g)
            return rows[:, :-1].contiguous().pin_memory(), rows[:, 1:].contiguous().pin_memory()

        resident = [tuple(t.to(device) for t in host_batch()) for _ in range(GRAD_ACC)]

        def micro_batch(inp, tgt, last):
            if layout["dp"] > 1:
                dp_model.require_backward_grad_sync = last
            logits = dp_model(input_ids=inp)
            b, s = inp.shape
            logits = logits.view(b * s, -1)
            if tp > 1:
                loss = ref_vce(logits.float(), tgt.reshape(-1)).mean() / GRAD_ACC
            else:
                loss = F.cross_entropy(logits, tgt.reshape(-1), reduction="mean") / GRAD_ACC
            loss.backward()
            return loss

        def finish_step():
            if tp > 1:   # sequence-parallel norm gradients, as the reference's own TP benchmark does
                for p in norm_params:
                    if p.grad is not None:
                        dist.all_reduce(p.grad, group=pg.tp_group)
            optimizer.step()
            optimizer.zero_grad()

        def device_step():
            for i, (inp, tgt) in enumerate(resident):
                micro_batch(inp, tgt, i == GRAD_ACC - 1)
            finish_step()

        last = {}

        def e2e_step():
            acc = 0.0
            for i in range(GRAD_ACC):
                inp, tgt = host_batch()
                loss = micro_batch(inp.to(device), tgt.to(device), i == GRAD_ACC - 1)
                acc += loss.item()                 # the reference's train_step reads every micro-batch loss
            finish_step()
            last["loss"] = acc

        for _ in range(args.warmup):
            device_step()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        ms = timed(device_step, args.steps, device)
        clocks = sampler.stop() if sampler else {}
        for _ in range(max(1, args.warmup // 2)):
            e2e_step()
        e2e_ms = timed(e2e_step, args.steps, device)
        h2d = GRAD_ACC * 2 * MBS * SEQ * 8
        d2h = GRAD_ACC * 4
        line = result_line(args, layout, world, ms, e2e_ms, h2d, d2h, clocks, 0, "reference",
                           {"final_loss": last.get("loss")}) if rank == 0 else None
        return line, rank, world, device
    except Exception as exc:  # the reference could not run on this stack: say why, exit 0
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:300] if str(exc) else ''}"}),
                  flush=True)
        return None


# ------------------------------------------------------------ the other configurations, both arms
def config_line(args, spec, world, ms_total, e2e_ms_total, arm, clocks, launches, impl, final_loss):
    from benchmarks.config_specs import flops_per_token as fpt_of
    from picotron_b200.utils import measured_peak_flops
    tokens = arm["tokens_per_step"]
    ms_per_step = ms_total / args.steps
    value = tokens / (ms_per_step / 1e3)
    fpt = fpt_of(spec["model"], spec["seq"])
    return {
        "metric": f"training throughput, {spec['name']} configuration (tokens/s, whole job)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic seeded uniform tokens, random-init N(0,0.02) weights", "impl": impl,
        "mfu_percent_h100_constant": round(value / world * fpt / H100_PEAK * 100.0, 2),
        "mfu_percent_b200_measured_peak": round(value / world * fpt / measured_peak_flops() * 100.0, 2),
        "config": {"model": spec["model_label"], "layers": spec["model"]["num_hidden_layers"],
                   "global_batch_tokens": tokens, "seq_len": spec["seq"], "micro_batch": spec["mbs"],
                   "grad_accum": spec["grad_acc"], "optimizer": "AdamW lr 3e-4", "variant": spec["variant"],
                   "parallelism": arm.get("parallelism", spec["label"]),
                   "l2": "per-step working set exceeds the 126 MB L2; no explicit flush"},
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                   "reasons": clocks.get("reasons", [])},
        "e2e": {"value": round(tokens / (e2e_ms_total / args.steps / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": arm["h2d_bytes_per_step"], "d2h_bytes_per_step": arm["d2h_bytes_per_step"]},
        "gpu_launches": launches, "final_loss": final_loss,
    }


def build_ours_arm(spec, device):
    """This framework's arm of a configuration: ``TrainEngine`` on the spec's engine config."""
    from picotron_b200.engine import TrainEngine
    engine = TrainEngine(spec["engine_cfg"], device=device)
    dl = engine.data_loader
    g = torch.Generator().manual_seed(99 + dl.dp_rank)
    vocab = engine.model_config.vocab_size
    shape = (dl.micro_batch_size, dl.seq_length_per_gpu)
    resident = [(torch.randint(0, vocab, shape, generator=g).to(device), torch.randint(0, vocab, shape, generator=g).to(device))
                for _ in range(dl.grad_acc_steps)]

    def e2e_step():
        return engine.average_loss(engine.train_step())

    return dict(device_step=lambda: engine.train_step(device_batches=resident), e2e_step=e2e_step,
                tokens_per_step=engine.tokens_per_step,
                h2d_bytes_per_step=dl.grad_acc_steps * 2 * shape[0] * shape[1] * 8, d2h_bytes_per_step=4,
                parallelism=spec["label"], close=engine.close)


def measure_config(args, reference: bool):
    """One of the non-headline configurations on the running process group: returns the result line on
    rank 0 (None elsewhere). Raises what the arm raises."""
    from benchmarks.config_specs import make_spec
    ref_root = os.path.join(REPO, "baseline", "_ref")
    rank, local_rank, world = setup_distributed(args.gpus)
    device = torch.device("cuda", local_rank)
    spec = make_spec(args.config, world, args.variant, args.layers, args.seq)
    if reference:
        import_reference(ref_root)
        from baseline import reference_arms
        arm = {"moe": reference_arms.build_moe, "cp": reference_arms.build_cp,
               "pp": reference_arms.build_pp}[args.config](spec, device, world)
    else:
        arm = build_ours_arm(spec, device)
    ops = None
    if not reference:
        from picotron_b200 import ops
    for _ in range(args.warmup):
        arm["device_step"]()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    l0 = 0 if reference else ops.launches()
    ms = timed(arm["device_step"], args.steps, device)
    launches = 0 if reference else ops.launches() - l0
    clocks = sampler.stop() if sampler else {}
    last = {}

    def e2e():
        last["loss"] = arm["e2e_step"]()

    for _ in range(max(1, args.warmup // 2)):
        e2e()
    e2e_ms = timed(e2e, args.steps, device)
    if not reference:
        ops.check_status("bench")
    # under pipeline parallelism only the last stage knows the loss: report the largest value seen
    lt = torch.tensor([float(last.get("loss") or 0.0)], device=device)
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    last["loss"] = float(lt.item())
    line = config_line(args, spec, world, ms, e2e_ms, arm, clocks, launches,
                       "reference" if reference else "picotron_b200", last.get("loss")) if rank == 0 else None
    if "close" in arm:
        arm["close"]()
    return line


def run_config(args):
    reference = args.impl == "reference"
    if reference and not os.path.isdir(os.path.join(REPO, "baseline", "_ref", "picotron")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/picotron is not installed"}))
        return
    try:
        line = measure_config(args, reference)
        if line is not None:
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
    except Exception as exc:
        if not reference:
            raise
        if int(os.environ.get("RANK", "0")) == 0:   # the reference could not run on this stack: say why, exit 0
            print(json.dumps({"impl": "reference", "config": args.config,
                              "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:300] if str(exc) else ''}"}),
                  flush=True)


def import_reference(ref_root: str) -> None:
    """Put the installed reference first on the import path and make sure ``picotron`` resolves to it
    (this repository also ships a ``picotron`` package: aliases of its own modules)."""
    for name in [n for n in sys.modules if n == "picotron" or n.startswith("picotron.")]:
        del sys.modules[name]
    if REPO in sys.path:
        sys.path.remove(REPO)
    sys.path.insert(0, ref_root)
    import picotron
    assert os.path.abspath(picotron.__file__).startswith(os.path.abspath(ref_root)), picotron.__file__
    sys.path.append(REPO)       # behind the reference: for baseline.reference_arms and the result line only


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="smollm", choices=["smollm", "moe", "cp", "pp"],
                    help="smollm = the headline configuration; the others are described in benchmarks/config_specs.py")
    ap.add_argument("--variant", default=None, help="moe: capacity|dropless, cp: ring|ulysses, pp: interleaved|zb|1f1b|afab")
    ap.add_argument("--layers", type=int, default=0, help="non-headline configurations only: reduced depth for quick checks")
    ap.add_argument("--seq", type=int, default=0, help="non-headline configurations only: sequence length override")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)   # never time a cold run
    if args.config != "smollm":
        run_config(args)
        return
    assert args.gpus in LAYOUTS, f"--gpus must be one of {sorted(LAYOUTS)}"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
