"""Tensor-parallel layers and the model surgery that installs them.

``apply_tensor_parallel(model, async_tp, sequence_parallel, vocab_parallel_ce, overlap_comm)``
swaps the projections of a ``Llama`` for Megatron column / row parallel linears and the
embedding for a vocabulary-parallel one, mirroring
picotron/tensor_parallel/tensor_parallel.py:24-115. Each layer initialises the *full* master
weight with the single-GPU initialiser and keeps its own slice (tensor_parallel.py:173-186),
so a TP run starts from exactly the weights a single-GPU run would.

Differences from the reference by design:
* layers know their group and mode; nothing is read from globals or the environment in forward
* projections that share an input (q/k/v, gate/up) go through ``multi_linear`` and share one
  input collective (one all-gather under sequence parallelism instead of one per projection)
* ``overlap_comm`` selects the chunked ring all-gather / pipelined reduce-scatter pair of
  ``sp_overlap.py``
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn as nn

from .. import process_group_manager as pgm
from ..ops import embedding as emb_ops
from ..ops import gemm as gemm_ops
from . import sequence_parallel as sp
from . import tp_communications as tpc
from .dist_utils import group_rank, group_size


def _uniform_fan_in_(tensor: torch.Tensor, init_std=None) -> None:
    """Reference initialiser U(-1/sqrt(fan_in), 1/sqrt(fan_in)) (picotron/model.py:146-156), or
    N(0, init_std) when the config asks for a fixed standard deviation."""
    if init_std is not None:
        nn.init.normal_(tensor, mean=0.0, std=init_std)
        return
    bound = math.sqrt(1.0 / tensor.size(1))
    nn.init.uniform_(tensor, -bound, bound)


class Linear(nn.Module):
    """Bias-free linear on the GEMM kernel; the unsharded building block of the model."""

    def __init__(self, in_features: int, out_features: int, init_std=None, bias: bool = False):
        super().__init__()
        assert not bias, "bias is not supported"
        self.in_features, self.out_features = in_features, out_features
        self.init_std = init_std
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            _uniform_fan_in_(self.weight, self.init_std)

    def forward(self, x):
        return gemm_ops.linear(x, self.weight)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias=False"


class ColumnParallelLinear(nn.Module):
    """Y = X W^T with W split along its output rows: rank r holds ``W[r*out/tp:(r+1)*out/tp]``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, gather_output: bool = False,
                 async_all_reduce: bool = False, sequence_parallel: bool = False, overlap_comm: bool = False,
                 group=None, init_std=None, ptb: bool = False):
        """``ptb`` (the reference's name, tensor_parallel.py:188-191 there): start in the no-collective mode of
        the parallel transformer block, which ``DecoderLayer.configure_tensor_parallel`` otherwise sets."""
        super().__init__()
        assert not bias, "bias is not supported"
        self.init_std = init_std
        self.group = group if group is not None else pgm.get_pgm().tp_group
        self.tp_world_size = group_size(self.group)
        self.tp_rank = group_rank(self.group)
        assert out_features % self.tp_world_size == 0
        self.in_features, self.out_features = in_features, out_features
        self.output_size_per_partition = out_features // self.tp_world_size
        self.gather_output = gather_output
        self.async_all_reduce = async_all_reduce
        self.sequence_parallel = sequence_parallel
        self.overlap_comm = overlap_comm
        self.raw = bool(ptb)  # parallel-block mode: caller owns the input collective
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, in_features))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type == "meta":
            return
        master = torch.empty(self.out_features, self.in_features, dtype=self.weight.dtype)
        _uniform_fan_in_(master, self.init_std)
        lo = self.tp_rank * self.output_size_per_partition
        with torch.no_grad():
            self.weight.copy_(master[lo:lo + self.output_size_per_partition])

    def forward(self, x):
        return multi_linear([self], x)[0]

    def extra_repr(self):
        return (f"in={self.in_features}, out={self.out_features}/{self.tp_world_size}, "
                f"sp={self.sequence_parallel}, async={self.async_all_reduce}, overlap={self.overlap_comm}")


def _fused_ctx(mod, x):
    """The fused tensor-parallel context of a layer if it applies to ``x`` (bf16 CUDA activations of
    the micro-batch shape the symmetric buffers were sized for), else None."""
    tp = getattr(mod, "fused", None)
    if tp is None or not x.is_cuda or x.dtype != torch.bfloat16 or not mod.sequence_parallel:
        return None
    rows = x.numel() // x.shape[-1]
    if rows not in (tp.m_local, tp.m_full):
        return None
    return tp


def multi_linear(mods: Sequence[nn.Module], x: torch.Tensor, cat: bool = False):
    """Apply several bias-free projections to the same input, sharing the input collective and,
    when the weights are stored back to back, the GEMM. Returns the list of outputs (column
    slices of one buffer), or that buffer itself ``[..., sum(out_i)]`` with ``cat=True``."""
    first = mods[0]
    splits = [m.weight.shape[0] for m in mods]
    if not isinstance(first, ColumnParallelLinear):
        y = gemm_ops.multi_linear_cat(x, mods)
        return y if cat else list(y.split(splits, dim=-1))
    group = first.group
    tp = None if (first.raw or first.tp_world_size == 1) else _fused_ctx(first, x)
    if tp is not None and x.dim() == 3 and x.shape[0] * x.shape[1] == tp.m_local:
        from ..ops import fused_tp
        y = fused_tp.ag_linear(x, tp, mods)
    elif first.raw or first.tp_world_size == 1:
        y = gemm_ops.multi_linear_cat(x, mods)
    elif first.sequence_parallel:
        if first.overlap_comm:
            from .sp_overlap import ring_all_gather_linear
            y = ring_all_gather_linear(x, mods, group)
        else:
            y = sp.column_linear_sequence_parallel(x, mods, group)
    elif first.async_all_reduce:
        y = torch.cat([tpc.linear_with_async_all_reduce(x, m.weight, group=group) for m in mods], dim=-1)
    else:
        y = gemm_ops.multi_linear_cat(tpc.CopyToModelParallelRegion.apply(x, group), mods)
    if cat:
        assert not any(m.gather_output for m in mods)
        return y
    outs = y.split(splits, dim=-1)
    return [tpc.GatherFromModelParallelRegion.apply(o, group) if m.gather_output else o
            for o, m in zip(outs, mods)]


def install_fused_tp(model, tp_ctx) -> int:
    """Attach a fused tensor-parallel context (``ops.fused_tp.TPFused``) to every sequence-parallel
    column / row linear of ``model``. Returns the number of layers switched."""
    n = 0
    for mod in model.modules():
        if isinstance(mod, (ColumnParallelLinear, RowParallelLinear)) and mod.sequence_parallel \
                and not mod.overlap_comm and mod.tp_world_size > 1:
            mod.fused = tp_ctx
            n += 1
        elif isinstance(mod, VocabParallelEmbedding) and mod.sequence_parallel and mod.tp_world_size > 1:
            mod.fused = tp_ctx
            n += 1
    return n


class RowParallelLinear(nn.Module):
    """Y = X W^T with W split along its input columns; partial outputs are summed over the group
    (all-reduce, or reduce-scatter along the sequence under sequence parallelism)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, sequence_parallel: bool = False,
                 overlap_comm: bool = False, group=None, init_std=None, ptb: bool = False):
        """``ptb`` (the reference's name): start in the mode that returns the un-reduced partial sum."""
        super().__init__()
        assert not bias, "bias is not supported"
        self.init_std = init_std
        self.group = group if group is not None else pgm.get_pgm().tp_group
        self.tp_world_size = group_size(self.group)
        self.tp_rank = group_rank(self.group)
        assert in_features % self.tp_world_size == 0
        self.in_features, self.out_features = in_features, out_features
        self.input_size_per_partition = in_features // self.tp_world_size
        self.sequence_parallel = sequence_parallel
        self.overlap_comm = overlap_comm
        self.raw = bool(ptb)  # parallel-block mode: return the un-reduced partial sum
        self.weight = nn.Parameter(torch.empty(out_features, self.input_size_per_partition))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type == "meta":
            return
        master = torch.empty(self.out_features, self.in_features, dtype=self.weight.dtype)
        _uniform_fan_in_(master, self.init_std)
        lo = self.tp_rank * self.input_size_per_partition
        with torch.no_grad():
            self.weight.copy_(master[:, lo:lo + self.input_size_per_partition])

    def forward(self, x, addend=None, residual=None):
        """``addend`` (parallel block, overlap mode) is a second partial sum folded into the
        same reduction; ``residual`` is added once to the reduced result."""
        tp = _fused_ctx(self, x)
        if tp is not None and addend is None and not self.raw and x.numel() // x.shape[-1] == tp.m_full:
            from ..ops import fused_tp
            return fused_tp.linear_rs(x, self.weight, tp, addend=residual)
        if self.raw or self.tp_world_size == 1:
            y = gemm_ops.linear(x, self.weight)
            y = y if addend is None else y + addend
            return y if residual is None else y + residual
        if self.sequence_parallel and self.overlap_comm:
            from .sp_overlap import linear_pipelined_reduce_scatter
            y = linear_pipelined_reduce_scatter(x, self.weight, self.group, addend)
            return y if residual is None else y + residual
        y = gemm_ops.linear(x, self.weight)
        if addend is not None:
            y = y + addend
        if self.sequence_parallel:
            y = sp.ReduceScatterToSequenceParallelRegion.apply(y, self.group)
        else:
            y = tpc.ReduceFromModelParallelRegion.apply(y, self.group)
        return y if residual is None else y + residual

    def extra_repr(self):
        return (f"in={self.in_features}/{self.tp_world_size}, out={self.out_features}, "
                f"sp={self.sequence_parallel}, overlap={self.overlap_comm}")


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary; rows owned elsewhere contribute zeros and the
    partial lookups are summed (all-reduce, or reduce-scatter under sequence parallelism)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, sequence_parallel: bool = False, group=None,
                 init_std=None, padding_idx=None, max_norm=None, norm_type: float = 2.0,
                 scale_grad_by_freq: bool = False, sparse: bool = False):
        """The ``nn.Embedding`` options that the reference's signature lists (tensor_parallel.py:296-306 there)
        are accepted by keyword at their defaults; none of them is implemented by either framework."""
        super().__init__()
        assert padding_idx is None and max_norm is None and not scale_grad_by_freq and not sparse, \
            "padding_idx / max_norm / scale_grad_by_freq / sparse are not supported"
        self.init_std = init_std
        self.group = group if group is not None else pgm.get_pgm().tp_group
        self.tp_world_size = group_size(self.group)
        self.tp_rank = group_rank(self.group)
        assert num_embeddings % self.tp_world_size == 0
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.num_embeddings_per_partition = num_embeddings // self.tp_world_size
        self.vocab_start_index = self.tp_rank * self.num_embeddings_per_partition
        self.vocab_end_index = self.vocab_start_index + self.num_embeddings_per_partition
        self.sequence_parallel = sequence_parallel
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type == "meta":
            return
        master = torch.empty(self.num_embeddings, self.embedding_dim, dtype=self.weight.dtype)
        nn.init.normal_(master, mean=0.0, std=self.init_std if self.init_std is not None else 1.0)
        with torch.no_grad():
            self.weight.copy_(master[self.vocab_start_index:self.vocab_end_index])

    def forward(self, input_ids):
        tp = getattr(self, "fused", None)
        if tp is not None and self.sequence_parallel and input_ids.is_cuda and input_ids.dim() == 2 \
                and input_ids.numel() == tp.m_full and self.weight.dtype == torch.bfloat16 \
                and self.embedding_dim <= tp.max_cols and self.embedding_dim % 8 == 0:
            from ..ops import fused_tp
            return fused_tp.embedding_rs(input_ids, self.weight, self.vocab_start_index, tp)
        out = emb_ops.embedding(input_ids, self.weight, self.vocab_start_index)
        if self.tp_world_size == 1:
            return out
        if self.sequence_parallel:
            return sp.ReduceScatterToSequenceParallelRegion.apply(out, self.group)
        return tpc.ReduceFromModelParallelRegion.apply(out, self.group)


def apply_tensor_parallel(model, async_tp: bool = False, sequence_parallel: bool = False,
                          vocab_parallel_ce: bool = False, overlap_comm: bool = False, group=None):
    """Replace the model's projections / embedding / lm head by their tensor-parallel versions.

    MoE feed-forward blocks are left alone (experts are sharded by expert parallelism instead,
    as in tensor_parallel.py:104-107). Returns the model; sets ``model.sequence_parallel`` and
    ``model.vocab_parallel_ce`` so the trainer and the schedules know the activation layout and
    which loss to use.
    """
    group = group if group is not None else pgm.get_pgm().tp_group
    assert not overlap_comm or sequence_parallel, "overlap_comm needs sequence_parallel"

    def column(old, gather_output=False):
        return ColumnParallelLinear(old.in_features, old.out_features, gather_output=gather_output,
                                    async_all_reduce=async_tp, sequence_parallel=sequence_parallel,
                                    overlap_comm=overlap_comm, group=group, init_std=old.init_std)

    def row(old):
        return RowParallelLinear(old.in_features, old.out_features, sequence_parallel=sequence_parallel,
                                 overlap_comm=overlap_comm, group=group, init_std=old.init_std)

    tp = group_size(group)
    for layer in model.decoder_layers_iter():
        attn = layer.attention
        assert attn.num_heads % tp == 0 and attn.num_key_values % tp == 0, \
            "attention heads and KV heads must be divisible by the TP size"
        for name in ("q_proj", "k_proj", "v_proj"):
            setattr(attn, name, column(getattr(attn, name)))
        attn.out_proj = row(attn.out_proj)
        attn.num_local_heads = attn.num_heads // tp
        attn.num_local_kv_heads = attn.num_key_values // tp
        mlp = layer.mlp
        if not getattr(mlp, "is_moe", False):
            for name in ("up_proj", "gate_proj"):
                setattr(mlp, name, column(getattr(mlp, name)))
            mlp.down_proj = row(mlp.down_proj)
    for layer in model.decoder_layers_iter():
        layer.configure_tensor_parallel(sequence_parallel, group)
    if getattr(model, "embedding", None) is not None and not isinstance(model.embedding, nn.Identity):
        old = model.embedding
        model.embedding = VocabParallelEmbedding(old.num_embeddings, old.embedding_dim,
                                                 sequence_parallel=sequence_parallel, group=group,
                                                 init_std=old.init_std)
    if getattr(model, "final_proj", None) is not None and not isinstance(model.final_proj, nn.Identity):
        # the lm head sees the full sequence: under sequence parallelism its own input gather
        # provides it; with vocab_parallel_ce the logits stay sharded along the vocabulary
        model.final_proj = column(model.final_proj, gather_output=not vocab_parallel_ce)
    final_norm = getattr(model, "final_norm", None)
    if final_norm is not None and hasattr(final_norm, "weight"):
        final_norm.weight.sequence_parallel_grad = sequence_parallel
    model.sequence_parallel = sequence_parallel
    model.vocab_parallel_ce = vocab_parallel_ce
    model.tp_group = group
    return model
