"""Rotary position embedding, half-split (non-interleaved) convention.

``get_cos_sin`` builds the tables the way picotron/model.py:39-51 does (angles
``pos * theta^(-2i/d)``, halves duplicated); the kernel only needs the first half, in fp32.
``apply_rope(x, cos, sin, pos_offset)`` rotates ``x[b, s, heads, d]``; the CUDA path works in
place on a view of the fused QKV projection output and its backward is the inverse rotation.

Reference: picotron/model.py:29-36 (apply_rotary_pos_emb), picotron/model.py:185-190.
"""
from __future__ import annotations

import torch

from . import count_launch, ext, use_kernels


def get_cos_sin(seq_length: int, head_dim: int, base: float = 500000.0, device="cpu",
                dtype=torch.float32):
    assert head_dim % 2 == 0
    theta = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    position = torch.arange(seq_length, dtype=torch.float32).unsqueeze(1)
    angles = position * theta.unsqueeze(0)  # [seq, d/2]
    cos = torch.cos(angles).repeat(1, 2).to(device=device, dtype=dtype)
    sin = torch.sin(angles).repeat(1, 2).to(device=device, dtype=dtype)
    return cos, sin


def rotate_half(x):
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos_offset: int = 0):
    """x: [b, s, heads, d]; cos/sin: [max_pos, d] (duplicated halves)."""
    s = x.shape[1]
    c = cos[pos_offset:pos_offset + s].to(x.dtype)[None, :, None, :]
    sn = sin[pos_offset:pos_offset + s].to(x.dtype)[None, :, None, :]
    return x * c + rotate_half(x) * sn


class _RopeFn(torch.autograd.Function):
    """Out-of-place rotation; the backward is the inverse rotation of the incoming gradient."""

    @staticmethod
    def forward(ctx, x, cos_half, sin_half, pos_offset):
        y = x.clone(memory_format=torch.contiguous_format)
        b, s, nh, d = y.shape
        ext().rope_inplace(y, y.stride(1), b * s, s, pos_offset, nh, d, cos_half, sin_half, 1)
        count_launch()
        ctx.save_for_backward(cos_half, sin_half)
        ctx.pos_offset = pos_offset
        return y

    @staticmethod
    def backward(ctx, dy):
        cos_half, sin_half = ctx.saved_tensors
        dx = dy.clone(memory_format=torch.contiguous_format)
        b, s, nh, d = dx.shape
        ext().rope_inplace(dx, dx.stride(1), b * s, s, ctx.pos_offset, nh, d, cos_half, sin_half, -1)
        count_launch()
        return dx, None, None, None


def rope_tables_for_kernel(cos: torch.Tensor, sin: torch.Tensor):
    """fp32 [max_pos, d/2] tables (first half of the duplicated tables)."""
    half = cos.shape[-1] // 2
    return cos[:, :half].float().contiguous(), sin[:, :half].float().contiguous()


def rope_inplace_(x: torch.Tensor, cos_half: torch.Tensor, sin_half: torch.Tensor, pos_offset: int, sign: int):
    """Raw in-place rotation (no autograd). x: [b, s, heads, d] view with unit inner strides."""
    b, s, nh, d = x.shape
    ext().rope_inplace(x, x.stride(1), b * s, s, pos_offset, nh, d, cos_half, sin_half, sign)
    count_launch()
    return x


def apply_rope(x, cos, sin, pos_offset: int = 0, tables=None):
    if use_kernels(x) and x.shape[-1] % 16 == 0:
        ch, sh = tables if tables is not None else rope_tables_for_kernel(cos, sin)
        return _RopeFn.apply(x, ch, sh, pos_offset)
    return apply_rope_ref(x, cos, sin, pos_offset)
