"""Small utilities with the names of picotron/utils.py: rank-safe ``print``, seeding,
readable number formatting, MFU, parameter counting and loss averaging."""
from __future__ import annotations

import builtins
import fcntl
import json
import os
import random
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from .. import process_group_manager as pgm

H100_BF16_PEAK_FLOPS = 989.5e12  # constant of picotron/utils.py:55, kept for comparable MFU figures


def print(*args, is_print_rank: bool = True, **kwargs):
    """Serialised print: one rank at a time through an advisory file lock (utils.py:15-24)."""
    if not is_print_rank:
        return
    with open(__file__, "r") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            builtins.print(*args, **kwargs)
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def set_all_seed(seed: int) -> None:
    for module in (random, np.random):
        module.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def to_readable_format(num: float, precision: int = 3) -> str:
    num_str = str(num)
    length = len(num_str)

    def format_with_precision(main, decimal, suffix):
        if precision == 0:
            return f"{main}{suffix}"
        return f"{main}.{decimal[:precision]}{suffix}"

    if "." in num_str or "e" in num_str:
        num_str = str(int(float(num)))
        length = len(num_str)
    for digits, suffix in ((12, "T"), (9, "B"), (6, "M"), (3, "K")):
        if length > digits:
            return format_with_precision(num_str[:-digits], num_str[-digits:], suffix)
    return num_str


def measured_peak_flops(default: float = 1.59e15) -> float:
    """bf16 peak used for the B200 MFU figure: the sustained cuBLAS throughput measured on this
    machine when MEASURED_PEAKS.json is present next to the package, else ``default``."""
    here = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(here.read_text())["bf16_tflops_sustained"]) * 1e12
    except Exception:
        return default


def flops_per_token(num_params: float, num_layers: int, hidden_size: int, seq_len: int) -> float:
    """6N for the matmuls plus 12*L*h*s for attention (utils.py:51-62)."""
    return 6.0 * num_params + 12.0 * num_layers * hidden_size * seq_len


def get_mfu(tokens_per_second: float, num_params: float, model_config=None,
            theoretical_flops: float = H100_BF16_PEAK_FLOPS, num_layers=None, hidden_size=None, seq_len=None) -> float:
    """Model FLOPs utilisation in percent of ONE GPU's peak: ``tokens_per_second`` is the per-GPU rate (the
    parameter keeps the reference's name, utils.py:51 there; its trainer passes tokens/s/GPU). Defaults to the
    reference's H100 constant; pass ``theoretical_flops=measured_peak_flops()`` for the B200 figure."""
    if model_config is not None:
        num_layers = model_config.num_hidden_layers
        hidden_size = model_config.hidden_size
        seq_len = model_config.max_position_embeddings
    fpt = flops_per_token(num_params, num_layers, hidden_size, seq_len)
    return tokens_per_second * fpt / theoretical_flops * 100.0


def get_num_params(model) -> int:
    """Global parameter count from this rank's shards: TP-sharded tensors count ``tp`` times,
    local experts ``ep`` times, and pipeline stages are summed (utils.py:65-101). Works on CPU."""
    m = pgm.get_pgm()
    local = 0
    for name, p in model.named_parameters():
        n = p.numel()
        if "mlp.local_experts." in name:
            n *= m.ep_world_size
        elif "mlp.gate." in name or "mlp.shared_expert." in name or "_latent" in name:
            pass
        elif any(k in name for k in ("attention", "mlp", "embed", "final_proj")):
            if m.tp_world_size > 1 and getattr(p, "_tp_replicated", False) is False and _is_tp_sharded(model, name):
                n *= m.tp_world_size
        local += n
    if m.pp_world_size > 1 and dist.is_initialized():
        t = torch.tensor([local], dtype=torch.int64, device=next(model.parameters()).device)
        dist.all_reduce(t, group=m.pp_group)
        return int(t.item())
    return local


def _is_tp_sharded(model, param_name: str) -> bool:
    from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
    mod_name = param_name.rsplit(".", 1)[0]
    try:
        mod = model.get_submodule(mod_name)
    except AttributeError:
        return False
    return isinstance(mod, (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding))


def assert_no_meta_tensors(model) -> None:
    bad = [n for n, p in model.named_parameters() if p.device.type == "meta"]
    bad += [n for n, b in model.named_buffers() if b.device.type == "meta"]
    assert not bad, f"tensors still on the meta device: {bad}"


def average_loss_across_dp_cp_ranks(loss, device) -> float:
    """Mean of the last pipeline stage's loss over the CP x DP replicas (utils.py:117-122)."""
    m = pgm.get_pgm()
    t = torch.tensor([loss if loss is not None else 0.0], dtype=torch.float32, device=device)
    if m.pp_is_last_stage and m.cp_dp_world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=m.cp_dp_group)
        t /= m.cp_dp_world_size
    return float(t.item())


def download_model(model_name: str, hf_token=None, local_dir: str = "hf_model_safetensors"):
    """Fetch ``config.json`` and safetensors of a Hugging Face model into
    ``<local_dir>/<model_name>`` unless they are already there. Needs network access."""
    dst = Path(local_dir) / model_name
    if (dst / "config.json").exists():
        return str(dst)
    from huggingface_hub import snapshot_download
    snapshot_download(repo_id=model_name, local_dir=str(dst), token=hf_token,
                      allow_patterns=["*.json", "*.safetensors"])
    return str(dst)
