"""Device-side timing helpers: CUDA-event stopwatches, max-over-ranks reduction, NVTX ranges and
the roofline arithmetic used in the benchmark reports."""
from __future__ import annotations

import contextlib
import json
import time
from pathlib import Path

import torch
import torch.distributed as dist


class EventTimer:
    """Accumulates named device-time intervals with CUDA events (wall clock on CPU)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.pending = []
        self.totals = {}

    @contextlib.contextmanager
    def section(self, name: str):
        if self.device.type == "cuda":
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)
            s.record()
            yield
            e.record()
            torch.cuda.nvtx.range_pop()
            self.pending.append((name, s, e))
        else:
            t0 = time.perf_counter()
            yield
            self.totals[name] = self.totals.get(name, 0.0) + (time.perf_counter() - t0) * 1e3

    def collect(self, group=None) -> dict:
        """Milliseconds per section, MAX-reduced over ``group`` when distributed."""
        if self.pending:
            torch.cuda.synchronize(self.device)
            for name, s, e in self.pending:
                self.totals[name] = self.totals.get(name, 0.0) + s.elapsed_time(e)
            self.pending = []
        out = dict(self.totals)
        if dist.is_initialized() and dist.get_world_size(group) > 1 and out:
            names = sorted(out)
            t = torch.tensor([out[n] for n in names], dtype=torch.float64,
                             device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = dict(zip(names, t.tolist()))
        self.totals = {}
        return out


def measured_peaks() -> dict:
    """Measured copy bandwidth and cuBLAS bf16 throughput of this machine (MEASURED_PEAKS.json at
    the repository root), or the documented fallback figures when the file is absent."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


NVLINK_PEER_GBS = 770.0   # measured peer copy bandwidth per direction per GPU on this pool


def roofline_fraction(seconds: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
                      sustained: bool = False) -> dict:
    """achieved / bound, where the bound is the slowest of compute at the measured GEMM peak, HBM
    traffic at the measured copy bandwidth and NVLink traffic at the measured peer bandwidth."""
    pk = measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_compute = flops / tf if flops else 0.0
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_link = nvlink_bytes / (NVLINK_PEER_GBS * 1e9) if nvlink_bytes else 0.0
    bound = max(t_compute, t_hbm, t_link)
    which = {t_compute: "compute", t_hbm: "hbm", t_link: "nvlink"}[bound] if bound > 0 else "none"
    return {"bound_seconds": bound, "bound": which, "fraction": bound / seconds if seconds > 0 else 0.0,
            "peaks": pk["source"]}
