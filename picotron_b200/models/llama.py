"""Llama-style decoder-only transformer.

Same module tree and state-dict names as picotron/model.py:356-402 —
``embedding``, ``decoder_layers.{i}.{input_layernorm, attention.{q,k,v,out}_proj,
post_attention_layernorm, mlp.{up,gate,down}_proj}``, ``final_norm``, ``final_proj`` — with
pre-norm sequential blocks or the parallel transformer block (``config.parallel_block``:
``x + Attn(LN(x)) + MLP(LN(x))`` with a single norm, model.py:319-329), SwiGLU or MoE
feed-forward (``config.num_experts > 1``), grouped-query attention and half-split RoPE.

Design differences from the reference:
* the model never reads the environment or a global topology in ``forward``: parallel layers
  carry their group, the attention backend is an attribute (``attention.core``) that
  ``apply_context_parallel`` swaps, RoPE tables are built once per model
* q/k/v and gate/up share their input collective and, on the GPU, the residual add is folded
  into the following RMSNorm
* GQA is not expanded before attention
* hot ops dispatch to the hand-written kernels in ``picotron_b200.ops``
"""
from __future__ import annotations

from typing import Iterator, Optional

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import embedding as emb_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..ops import swiglu as swiglu_ops
from ..parallel.tensor_parallel import Linear, multi_linear


class RMSNorm(nn.Module):
    """x * rsqrt(mean(x^2) + eps) * weight with fp32 statistics (picotron/model.py:96-115)."""

    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.hidden_size = hidden_size
        self.weight = nn.Parameter(torch.ones(hidden_size))
        # under sequence parallelism every TP rank sees a different sequence shard, so this
        # weight's gradient must be summed over the TP group before the optimizer step
        self.weight.sequence_parallel_grad = False

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.ones_(self.weight)

    def forward(self, x, residual=None):
        if residual is None:
            return norm_ops.rmsnorm(x, self.weight, self.eps)
        return norm_ops.add_rmsnorm(x, residual, self.weight, self.eps)


LlamaRMSNorm = RMSNorm


class TritonRMSNorm(RMSNorm):
    """The reference's second norm class (picotron/model.py:61-93, a Triton layer-norm call): the same
    module here, on this library's kernel. Its optional arguments are accepted; dropout and the
    pre-norm return are not supported (the reference's model never uses them)."""

    def __init__(self, hidden_size: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__(hidden_size, eps)
        if device is not None or dtype is not None:
            self.to(device=device, dtype=dtype)

    def forward(self, hidden_states, residual=None, dropout_p: float = 0.0, prenorm: bool = False,
                residual_in_fp32: bool = False, return_dropout_mask: bool = False):
        assert dropout_p == 0.0 and not prenorm and not return_dropout_mask, "only the plain RMSNorm call is supported"
        if residual is None:
            return super().forward(hidden_states)
        return super().forward(hidden_states, residual)[0]


def get_cos_sin(seq_length: int, head_dim: int, base: float = 500000.0):
    """Rotary tables ``[seq_length, head_dim]`` (duplicated halves) on the device and in the dtype that
    the ``DEVICE`` / ``DTYPE`` / ``LOCAL_RANK`` environment variables name, like picotron/model.py:39-51."""
    import os
    dtype = torch.bfloat16 if os.environ.get("DTYPE", "bfloat16") == "bfloat16" else torch.float32
    on_gpu = os.environ.get("DEVICE", "cuda") == "cuda" and torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if on_gpu else torch.device("cpu")
    return rope_ops.get_cos_sin(seq_length, head_dim, base, device=device, dtype=dtype)


def apply_rotary_pos_emb(x, cos, sin):
    """x: ``[b, heads, s, d]``; cos / sin: ``[s, d]`` (picotron/model.py:29-36)."""
    return x * cos + rope_ops.rotate_half(x) * sin


def flash_attention(q, k, v, causal: bool = True):
    """q, k, v: ``[b, heads, s, d]`` -> ``[b, s, heads, d]`` (the layout flash-attn returns,
    picotron/model.py:54-58), on this library's attention kernels when the tensors allow."""
    return attn_ops.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, init_std=None, padding_idx=None):
        super().__init__()
        assert padding_idx is None, "padding_idx is not supported"
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.init_std = init_std
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, mean=0.0, std=self.init_std if self.init_std is not None else 1.0)

    def forward(self, input_ids):
        return emb_ops.embedding(input_ids, self.weight, 0)


class FinalProjection(Linear):
    """The lm head: hidden -> vocabulary logits."""

    def __init__(self, hidden_size: int, vocab_size: int, init_std=None, bias: bool = False):
        super().__init__(hidden_size, vocab_size, init_std, bias)


def _local_attention(q, k, v, causal, sm_scale=None):
    return attn_ops.attention(q, k, v, causal, sm_scale)


class Attention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_key_values = config.num_key_value_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_local_heads = self.num_heads          # divided by apply_tensor_parallel
        self.num_local_kv_heads = self.num_key_values
        std = getattr(config, "init_std", None)
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim, std)
        self.k_proj = Linear(config.hidden_size, self.num_key_values * self.head_dim, std)
        self.v_proj = Linear(config.hidden_size, self.num_key_values * self.head_dim, std)
        self.out_proj = Linear(config.hidden_size, config.hidden_size, std)
        self.layer_idx = layer_idx
        #: callable (q, k, v, causal) -> out on [b, s, heads, d] tensors; context parallelism
        #: replaces it with ring or Ulysses attention
        self.core = _local_attention

    def reset_parameters(self):
        for m in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            m.reset_parameters()

    def qkv(self, x, rope):
        b = x.shape[0]
        q, k, v = multi_linear([self.q_proj, self.k_proj, self.v_proj], x)
        s = q.shape[1]  # full sequence under sequence parallelism
        q = q.view(b, s, self.num_local_heads, self.head_dim)
        k = k.view(b, s, self.num_local_kv_heads, self.head_dim)
        v = v.view(b, s, self.num_local_kv_heads, self.head_dim)
        q = rope.apply(q)
        k = rope.apply(k)
        return q, k, v

    def _fused_local(self, x, rope):
        """Local attention on bf16 CUDA tensors: fused QKV GEMM -> in-place RoPE -> flash attention,
        with a backward that produces one dQKV buffer. None when the path does not apply (context
        parallelism, CPU, unsupported head size)."""
        if self.core is not _local_attention or not x.is_cuda or x.dtype != torch.bfloat16 \
                or self.head_dim not in (64, 128) or attn_ops.reference_ops_forced_():
            return None
        qkv = multi_linear([self.q_proj, self.k_proj, self.v_proj], x, cat=True)
        if qkv.dim() != 3 or not qkv.is_contiguous():
            return None
        _, _, half = rope.tables(x.device, x.dtype)
        return attn_ops.rope_attention_fused(qkv, self.num_local_heads, self.num_local_kv_heads, self.head_dim,
                                             half[0], half[1], rope.pos_offset)

    def forward(self, x, rope, out_addend=None, residual=None):
        """``residual`` (optional) is added to the projected output inside the row-parallel
        reduction, so the caller gets ``x_res + attention(x)`` without a separate add."""
        out = self._fused_local(x, rope)
        if out is None:
            q, k, v = self.qkv(x, rope)
            b, s = q.shape[0], q.shape[1]
            out = self.core(q, k, v, True)
            out = out.reshape(b, s, self.num_local_heads * self.head_dim)
        if out_addend is not None:
            return self.out_proj(out, out_addend)
        if residual is not None:
            return self.out_proj(out, residual=residual)
        return self.out_proj(out)


class MLP(nn.Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (picotron/model.py:236-258)."""

    is_moe = False

    def __init__(self, config, intermediate_size: Optional[int] = None):
        super().__init__()
        inter = intermediate_size if intermediate_size is not None else config.intermediate_size
        std = getattr(config, "init_std", None)
        self.up_proj = Linear(config.hidden_size, inter, std)
        self.gate_proj = Linear(config.hidden_size, inter, std)
        self.down_proj = Linear(inter, config.hidden_size, std)

    def reset_parameters(self):
        for m in (self.up_proj, self.gate_proj, self.down_proj):
            m.reset_parameters()

    def hidden(self, x):
        return swiglu_ops.swiglu(multi_linear([self.gate_proj, self.up_proj], x, cat=True))

    def forward(self, x, residual=None):
        if getattr(self.down_proj, "fused", None) is not None and residual is not None:
            # fused sequence parallelism: the reduce-scatter epilogue of the down projection adds the residual
            return self.down_proj(self.hidden(x), residual=residual)
        y = self.down_proj(self.hidden(x))
        return y if residual is None else y + residual


class RotaryTables:
    """cos/sin tables shared by all layers of a model, plus this rank's position offset
    (non-zero under context parallelism, where rank r holds positions [r*s_local, (r+1)*s_local))."""

    def __init__(self, max_positions: int, head_dim: int, theta: float):
        self.max_positions, self.head_dim, self.theta = max_positions, head_dim, theta
        self.pos_offset = 0
        #: zigzag context parallelism: the local tokens are several pieces of the sequence, given as
        #: (local start, length, global position of the first token); None = one piece at pos_offset
        self.pos_pieces = None
        self._cache = {}

    def tables(self, device, dtype):
        key = (str(device), dtype)
        t = self._cache.get(key)
        if t is None:
            cos, sin = rope_ops.get_cos_sin(self.max_positions, self.head_dim, self.theta, device=device,
                                            dtype=torch.float32)
            t = (cos, sin, rope_ops.rope_tables_for_kernel(cos, sin))
            self._cache[key] = t
        return t

    def apply(self, x):
        cos, sin, half = self.tables(x.device, x.dtype)
        if self.pos_pieces is None:
            return rope_ops.apply_rope(x, cos, sin, self.pos_offset, tables=half)
        return torch.cat([rope_ops.apply_rope(x[:, lo:lo + n], cos, sin, pos, tables=half)
                          for lo, n, pos in self.pos_pieces], dim=1)


class DecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.parallel_block = bool(getattr(config, "parallel_block", False))
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.attention = Attention(config, layer_idx)
        if getattr(config, "num_experts", 0) and config.num_experts > 1:
            from ..parallel.expert_parallel import MoELayer
            self.mlp = MoELayer(config)
        else:
            self.mlp = MLP(config)
        if not self.parallel_block:
            self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.layer_idx = layer_idx
        self.sequence_parallel = False
        self.tp_group = None

    def reset_parameters(self):
        self.input_layernorm.reset_parameters()
        self.attention.reset_parameters()
        self.mlp.reset_parameters()
        if not self.parallel_block:
            self.post_attention_layernorm.reset_parameters()

    def norms(self):
        out = [self.input_layernorm]
        if not self.parallel_block:
            out.append(self.post_attention_layernorm)
        return out

    def configure_tensor_parallel(self, sequence_parallel: bool, group):
        """Called by apply_tensor_parallel after the projections were swapped."""
        self.sequence_parallel = sequence_parallel
        self.tp_group = group
        for n in self.norms():
            n.weight.sequence_parallel_grad = sequence_parallel
        fused_ptb = self.parallel_block and sequence_parallel and not getattr(self.mlp, "is_moe", False)
        overlap = getattr(self.attention.out_proj, "overlap_comm", False)
        attn, mlp = self.attention, self.mlp
        if fused_ptb and not overlap:
            # one shared all-gather in, one reduce-scatter of the attn+mlp partial sums out; the
            # projections run without collectives of their own
            for m in (attn.q_proj, attn.k_proj, attn.v_proj, attn.out_proj, mlp.gate_proj, mlp.up_proj,
                      mlp.down_proj):
                m.raw = True
        elif fused_ptb:
            # chunked overlap: q/k/v and gate/up each ride a ring all-gather; the MLP partial sum
            # is folded into the out-projection's pipelined reduce-scatter
            mlp.down_proj.raw = True
        self.fused_ptb = fused_ptb
        self.ptb_overlap = fused_ptb and overlap

    def forward(self, x, rope):
        if self.parallel_block:
            return self._forward_parallel(x, rope)
        if getattr(self.attention.out_proj, "fused", None) is not None and not getattr(self.mlp, "is_moe", False):
            # the residual adds ride in the reduce-scatter epilogues of out_proj and down_proj
            h = self.attention(self.input_layernorm(x), rope, residual=x)
            return self.mlp(self.post_attention_layernorm(h), residual=h)
        a = self.attention(self.input_layernorm(x), rope)
        y, h = self.post_attention_layernorm(a, residual=x)
        return h + self.mlp(y)

    def _forward_parallel(self, x, rope):
        from ..parallel import sequence_parallel as sp
        n = self.input_layernorm(x)
        if getattr(self, "fused_ptb", False):
            tp = self._ptb_peer_ctx(n)
            if tp is not None:
                return self._forward_parallel_peer(x, n, rope, tp)
            if self.ptb_overlap:
                mlp_partial = self.mlp(n)  # un-reduced [b, s, h] partial sum (down_proj is raw)
                return x + self.attention(n, rope, out_addend=mlp_partial)
            ng = sp.GatherFromSequenceParallelRegion.apply(n, self.tp_group)
            partial = self.attention(ng, rope) + self.mlp(ng)
            return x + sp.ReduceScatterToSequenceParallelRegion.apply(partial, self.tp_group)
        return x + self.attention(n, rope) + self.mlp(n)

    def _ptb_peer_ctx(self, n):
        """The peer-memory tensor-parallel context when the whole block can run on it: projections in
        their no-collective form, local attention on the flash kernels, the micro-batch shape the
        symmetric buffers were sized for."""
        attn = self.attention
        if self.ptb_overlap or not attn.q_proj.raw:
            return None
        tp = getattr(attn.q_proj, "fused", None)
        if tp is None or not n.is_cuda or n.dtype != torch.bfloat16 or n.dim() != 3 \
                or n.shape[0] * n.shape[1] != tp.m_local:
            return None
        if attn.core is not _local_attention or attn.head_dim not in (64, 128) or attn_ops.reference_ops_forced_():
            return None
        return tp

    def _forward_parallel_peer(self, x, n, rope, tp):
        """Parallel block on the fused tensor-parallel kernels: one pushed gather feeds the q/k/v and
        the gate/up GEMMs as its row blocks arrive; the out- and down-projection partial sums leave
        through the GEMMs' scatter epilogues and are summed, with the residual, on the owner of the
        rows. No collective call (picotron/model.py:319-329 runs them on NCCL)."""
        from ..ops import fused_tp
        attn, mlp = self.attention, self.mlp
        qkv, gate_up = fused_tp.ag_linear_sets(n, tp, [[attn.q_proj, attn.k_proj, attn.v_proj],
                                                       [mlp.gate_proj, mlp.up_proj]])
        _, _, half = rope.tables(x.device, x.dtype)
        a = attn_ops.rope_attention_fused(qkv, attn.num_local_heads, attn.num_local_kv_heads, attn.head_dim,
                                          half[0], half[1], rope.pos_offset)
        act = swiglu_ops.swiglu(gate_up)
        return fused_tp.dual_linear_rs(a, attn.out_proj.weight, act, mlp.down_proj.weight, tp, addend=x)


def lm_head(model, x):
    """final norm + vocabulary projection."""
    return model.final_proj(model.final_norm(x))


class Llama(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.hidden_size % config.num_attention_heads == 0
        assert config.num_attention_heads % config.num_key_value_heads == 0
        self.config = config
        self.vocab_size = config.vocab_size
        self.hidden_size = config.hidden_size
        self.num_layers = config.num_hidden_layers
        std = getattr(config, "init_std", None)
        self.embedding = Embedding(config.vocab_size, config.hidden_size, std)
        self.decoder_layers = nn.ModuleList([DecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.final_norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.final_proj = FinalProjection(config.hidden_size, config.vocab_size, std)
        self.rope = RotaryTables(config.max_position_embeddings, config.hidden_size // config.num_attention_heads,
                                 getattr(config, "rope_theta", 500000.0))
        self.sequence_parallel = False
        self.vocab_parallel_ce = False
        self.tp_group = None

    def decoder_layers_iter(self) -> Iterator[DecoderLayer]:
        layers = self.decoder_layers
        return iter(layers.values()) if isinstance(layers, nn.ModuleDict) else iter(layers)

    def reset_parameters(self):
        self.embedding.reset_parameters()
        for layer in self.decoder_layers_iter():
            layer.reset_parameters()
        self.final_norm.reset_parameters()
        self.final_proj.reset_parameters()

    def forward(self, input_ids, position_ids=None, hidden_states=None):
        x = self.embedding(input_ids)
        for layer in self.decoder_layers_iter():
            x = layer(x, self.rope)
        return lm_head(self, x)
