"""FP8 (E4M3) quantisation of activations for expert-parallel dispatch.

Two granularities: ``block`` — one fp32 scale per 1x128 block of a row (DeepSeek-V3 style, the
default here) — and ``row`` — one scale per token row, which is what
picotron/expert_parallel/ep_communications.py:63-68 does. scale = absmax / 448, values are
clamped to the E4M3 range; dequantisation multiplies back. Pure torch restatement (CPU capable);
the CUDA dispatch kernel fuses the same arithmetic into the send.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
BLOCK = 128


def quantize_fp8(x: torch.Tensor, granularity: str = "block"):
    """x: [rows, d] -> (payload uint8 [rows, d], scales fp32 [rows, nblocks])."""
    rows, d = x.shape
    xf = x.float()
    if granularity == "row":
        blocks = xf.view(rows, 1, d)
    else:
        pad = (-d) % BLOCK
        if pad:
            xf = torch.nn.functional.pad(xf, (0, pad))
        blocks = xf.view(rows, -1, BLOCK)
    amax = blocks.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12)
    scale = amax / E4M3_MAX
    q = (blocks / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    payload = q.view(rows, -1)[:, :d].contiguous().view(torch.uint8)
    return payload, scale.squeeze(-1).contiguous()


def dequantize_fp8(payload: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype, granularity: str = "block"):
    rows, d = payload.shape
    q = payload.view(torch.float8_e4m3fn).float()
    if granularity == "row":
        return (q * scales.view(rows, 1)).to(dtype)
    pad = (-d) % BLOCK
    if pad:
        q = torch.nn.functional.pad(q, (0, pad))
    out = (q.view(rows, -1, BLOCK) * scales.view(rows, -1, 1)).view(rows, -1)[:, :d]
    return out.to(dtype)
