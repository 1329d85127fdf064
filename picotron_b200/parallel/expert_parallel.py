"""Mixture-of-experts feed-forward with expert parallelism.

``MoELayer(config)`` keeps the parameter names and config knobs of
picotron/expert_parallel/expert_parallel.py:38-454: replicated router ``gate``; rank r owns
experts ``[r*L, (r+1)*L)`` as ``local_experts``; optional ``shared_expert``; optional LatentMoE
projections; persistent ``expert_bias``; routing = fp32 softmax, top-k on (probabilities + bias)
when loss-free balancing is on, weights from the unbiased probabilities, renormalised for k > 1;
auxiliary loss ``coef * sum_e f_e P_e`` and the sign-controller bias update; execution paths
``naive`` (dropless variable-size exchange), ``tiled`` (token tiles pipelined so that the exchange
of one tile overlaps the experts of another, forward and backward), ``capped`` (fixed-capacity
buffers, dropping or multi-round dropless) and FP8 dispatch on any of them.

Internal design (not the reference's):
* one ``RoutePlan`` per (tile of) routed rows: a stable sort by global expert makes the rows
  rank-major and expert-major at once; a single ``[ep, L]`` counts exchange tells every receiver the
  exact layout of what arrives, so no per-row expert ids travel and the receiver regroups rows by
  expert with an index computed from the counts table instead of a second sort
* the experts run as one grouped call over expert-contiguous rows
* ``ep_as_dp``: when set in the config every EP rank holds different tokens (DeepSeek-style); the
  layer itself is unchanged, only gradient reduction of non-expert weights spans the EP group
"""
from __future__ import annotations

import os
import types
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import process_group_manager as pgm
from ..ops import grouped_gemm
from ..ops import swiglu as swiglu_ops
from . import ep_communications as epc
from .dist_utils import group_rank, group_size
from .tensor_parallel import Linear


@dataclass
class RoutePlan:
    order: torch.Tensor          # [R] permutation: sorted position -> routed row
    inv_order: torch.Tensor      # [R]
    in_splits: List[int]         # rows sent to each rank
    out_splits: List[int]        # rows received from each rank
    recv_counts: torch.Tensor    # [ep, L] rows from rank s for local expert l
    regroup: Optional[torch.Tensor]      # [R_recv] gather index: expert-major position -> arrival position
    regroup_inv: Optional[torch.Tensor]
    expert_counts: List[int]     # rows per local expert after regrouping


def _argsort_inv(keys: torch.Tensor):
    order = torch.argsort(keys, stable=True)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return order, inv


class MoELayer(nn.Module):
    is_moe = True

    def __init__(self, config, ep_group=None):
        super().__init__()
        from ..models.llama import MLP
        self.hidden_size = config.hidden_size
        self.num_experts = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.norm_topk_prob = getattr(config, "norm_topk_prob", True)
        self.ep_group = ep_group if ep_group is not None else pgm.get_pgm().ep_group
        self.ep_world_size = group_size(self.ep_group)
        self.ep_rank = group_rank(self.ep_group)
        assert self.num_experts % self.ep_world_size == 0, \
            f"num_experts ({self.num_experts}) must be divisible by ep_size ({self.ep_world_size})"
        self.num_local_experts = self.num_experts // self.ep_world_size

        self.latent_dim = getattr(config, "moe_latent_dim", 0) or 0
        self.latent = 0 < self.latent_dim < self.hidden_size
        self.expert_dim = self.latent_dim if self.latent else self.hidden_size
        std = getattr(config, "init_std", None)
        self.gate = Linear(config.hidden_size, self.num_experts, std)
        if self.latent:
            self.down_proj_latent = Linear(self.hidden_size, self.latent_dim, std)
            self.up_proj_latent = Linear(self.latent_dim, self.hidden_size, std)
        expert_cfg = types.SimpleNamespace(hidden_size=self.expert_dim, intermediate_size=config.intermediate_size,
                                           init_std=std)
        self.local_experts = nn.ModuleList([MLP(expert_cfg) for _ in range(self.num_local_experts)])
        self._uniform_layouts = {}
        self.num_shared_experts = getattr(config, "num_shared_experts", 0) or 0
        shared_width = getattr(config, "shared_expert_intermediate_size", None)
        if shared_width is None and self.num_shared_experts > 0:
            shared_width = config.intermediate_size * self.num_shared_experts
        if shared_width:
            self.shared_expert = MLP(types.SimpleNamespace(hidden_size=self.hidden_size,
                                                           intermediate_size=shared_width, init_std=std))
        else:
            self.shared_expert = None

        self.ep_overlap = getattr(config, "ep_overlap", True)
        self.ep_num_tiles = getattr(config, "ep_num_tiles", 1) or 1
        self.ep_fp8_dispatch = getattr(config, "ep_fp8_dispatch", False)
        self.ep_fp8_granularity = getattr(config, "ep_fp8_granularity", "block")
        self.ep_backend = getattr(config, "ep_backend", "torch")
        self.ep_capacity_factor = getattr(config, "ep_capacity_factor", 0.0) or 0.0
        self.ep_capacity_dropless = getattr(config, "ep_capacity_dropless", True)
        self.ep_max_rounds = getattr(config, "ep_max_rounds", 8)
        self.router_aux_loss_coef = getattr(config, "router_aux_loss_coef", 0.0) or 0.0
        self.router_bias_update_rate = getattr(config, "router_bias_update_rate", 0.0) or 0.0
        self.use_loss_free = self.router_bias_update_rate > 0
        self.register_buffer("expert_bias", torch.zeros(self.num_experts), persistent=True)
        self.aux_loss = None
        self.last_dropped_fraction = None
        self._shared_stream = None
        #: optional ``ops.fused_ep.EPFused``: capacity-mode exchanges through NVLink peer memory
        self.fused_ep = None
        #: optional ``ops.fused_ep_var.EPVarFused``: dropless variable-size exchange through peer memory
        self.fused_ep_var = None

    def reset_parameters(self):
        # experts use the same RNG stream on every EP rank so replicated parameters stay in sync
        self.gate.reset_parameters()
        if self.latent:
            self.down_proj_latent.reset_parameters()
            self.up_proj_latent.reset_parameters()
        for e in self.local_experts:
            e.reset_parameters()
        if self.shared_expert is not None:
            self.shared_expert.reset_parameters()

    # ------------------------------------------------------------------------------ routing
    def _route(self, tokens):
        logits = self.gate(tokens)
        if logits.is_cuda and logits.dtype == torch.bfloat16 and self.num_experts <= 256 and self.top_k <= 8 \
                and os.environ.get("PICO_MOE_DEVICE_ROUTING", "1") != "0":
            # one kernel for softmax + bias + top-k + renormalisation + counts (ops/moe_route.py)
            from ..ops import moe_route as mr
            probs, idx, w, counts = mr.route(logits, self.expert_bias if self.use_loss_free else None, self.top_k,
                                             self.norm_topk_prob)
            self._balance(probs, idx, counts)
            return idx.long(), w.to(tokens.dtype)
        probs = F.softmax(logits, dim=-1, dtype=torch.float32)
        scores = probs + self.expert_bias.to(probs.dtype) if self.use_loss_free else probs
        topk_idx = torch.topk(scores, self.top_k, dim=-1).indices
        topk_w = probs.gather(-1, topk_idx)
        if self.norm_topk_prob and self.top_k > 1:
            topk_w = topk_w / topk_w.sum(dim=-1, keepdim=True)
        self._balance(probs, topk_idx)
        return topk_idx, topk_w.to(tokens.dtype)

    def _balance(self, probs, topk_idx, counts=None):
        """Auxiliary balancing loss and loss-free bias update from this forward pass's routing;
        ``counts`` (rows per expert) may come from the routing kernel."""
        self.aux_loss = None
        if not (self.training and (self.router_aux_loss_coef > 0 or self.use_loss_free)):
            return
        T = probs.shape[0]
        raw_counts = counts
        if counts is None:
            counts = torch.zeros(self.num_experts, device=probs.device, dtype=probs.dtype)
            counts.scatter_add_(0, topk_idx.reshape(-1), torch.ones(topk_idx.numel(), device=probs.device,
                                                                    dtype=probs.dtype))
        else:
            counts = counts.to(probs.dtype)
        if self.router_aux_loss_coef > 0:
            f = counts * (self.num_experts / (self.top_k * T))
            self.aux_loss = self.router_aux_loss_coef * (f * probs.mean(dim=0)).sum()
        if self.use_loss_free:
            with torch.no_grad():
                epf = self.fused_ep if self.fused_ep is not None else self.fused_ep_var
                if self.ep_world_size > 1 and epf is not None and raw_counts is not None \
                        and raw_counts.dtype == torch.int32 and self.num_experts % 4 == 0:
                    load = epf.sum_over_ranks(raw_counts).to(probs.dtype)     # through peer memory
                else:
                    load = counts.clone()
                    if self.ep_world_size > 1:
                        dist.all_reduce(load, group=self.ep_group)
                self.expert_bias += self.router_bias_update_rate * torch.sign(load.mean() - load)

    # ------------------------------------------------------------------------------ pieces
    def _shared_start(self, tokens):
        if self.shared_expert is None:
            return None, None
        if not (self.ep_overlap and self.ep_world_size > 1 and tokens.is_cuda):
            return self.shared_expert(tokens), None
        if self._shared_stream is None:
            self._shared_stream = torch.cuda.Stream()
        self._shared_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._shared_stream):
            out = self.shared_expert(tokens)
        return out, self._shared_stream

    def _finalize(self, y, shared):
        if self.latent:
            y = self.up_proj_latent(y)
        out, stream = shared
        if out is None:
            return y
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
            out.record_stream(torch.cuda.current_stream())
        return y + out

    def plan(self, expert_idx: torch.Tensor) -> RoutePlan:
        """Layout of one exchange for routed rows with global expert ids ``expert_idx`` [R]."""
        L, ep = self.num_local_experts, self.ep_world_size
        order, inv = _argsort_inv(expert_idx)
        counts = torch.bincount(expert_idx, minlength=self.num_experts).view(ep, L)
        if ep == 1:
            return RoutePlan(order, inv, [order.numel()], [order.numel()], counts, None, None,
                             counts.view(-1).tolist())
        recv_counts = epc.exchange_counts(counts, self.ep_group)            # [src, l]
        both = torch.stack([counts.sum(1), recv_counts.sum(1)]).tolist()      # one host read
        in_splits, out_splits = both
        # arrival order is (src, l); experts want (l, src): build the gather index from the table
        flat = recv_counts.reshape(-1)                                         # index s*L + l
        starts = torch.cumsum(flat, 0) - flat
        perm = torch.arange(ep * L, device=flat.device).view(ep, L).t().reshape(-1)   # (l, s) -> s*L + l
        seg_len = flat[perm]
        total = int(sum(out_splits))
        seg_id = torch.repeat_interleave(torch.arange(ep * L, device=flat.device), seg_len, output_size=total)
        seg_first = torch.cumsum(seg_len, 0) - seg_len
        regroup = starts[perm][seg_id] + (torch.arange(total, device=flat.device) - seg_first[seg_id])
        regroup_inv = torch.empty_like(regroup)
        regroup_inv[regroup] = torch.arange(total, device=flat.device)
        return RoutePlan(order, inv, in_splits, out_splits, recv_counts, regroup, regroup_inv,
                         recv_counts.sum(0).tolist())

    def grouped_experts(self, x: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """Run the local experts on expert-contiguous rows: counts[e] rows for expert e."""
        if x.shape[0] == 0:
            # keep the experts in the autograd graph so their (zero) gradients exist on every rank
            return x + 0.0 * sum(p.sum() for e in self.local_experts for p in e.parameters())
        if self._grouped_ok(x):
            layout = grouped_gemm.GroupLayout.from_counts([int(c) for c in counts], x.device)
            return layout.unpad(self._experts_on_layout(layout.pad(x), layout))
        outs, off = [], 0
        for e, n in enumerate(counts):
            outs.append(self.local_experts[e](x[off:off + n]))
            off += n
        return torch.cat(outs, dim=0)

    def experts_uniform(self, x: torch.Tensor) -> torch.Tensor:
        """Local experts on ``x[l]`` (``[L, rows, d]``, the same number of rows for every expert)."""
        L, R, d = x.shape
        if self._grouped_ok(x) and R > 0:
            key = (L, R, x.device)
            layout = self._uniform_layouts.get(key)
            if layout is None:
                layout = self._uniform_layouts[key] = grouped_gemm.GroupLayout.uniform(L, R, x.device)
            if layout.pad_index is None:
                return self._experts_on_layout(x.reshape(L * R, d), layout).view(L, R, -1)
            return layout.unpad(self._experts_on_layout(layout.pad(x.reshape(L * R, d)), layout)).view(L, R, -1)
        return torch.stack([self.local_experts[l](x[l]) for l in range(L)])

    def _grouped_ok(self, x: torch.Tensor) -> bool:
        if os.environ.get("PICO_GROUPED_EXPERTS", "1") == "0":     # A/B switch: per-expert GEMM launches
            return False
        e0 = self.local_experts[0]
        # the stacked weight-gradient blocks need output widths that are whole 128-row tiles
        return grouped_gemm.kernel_ok(x, self.expert_dim, e0.gate_proj.weight.shape[0]) and \
            self.expert_dim % 128 == 0 and e0.gate_proj.weight.dtype == torch.bfloat16

    def _experts_on_layout(self, xp: torch.Tensor, layout, rows_in_use=None) -> torch.Tensor:
        """SwiGLU feed-forward of every local expert over the padded expert-major rows ``xp``: two
        grouped GEMM launches around one SwiGLU kernel (the reference's fused-MoE composition,
        picotron/expert_parallel/megakernel.py:294-357)."""
        experts = list(self.local_experts)
        inter = experts[0].gate_proj.weight.shape[0]
        gu = grouped_gemm.grouped_linear(xp, [m for e in experts for m in (e.gate_proj, e.up_proj)], layout, 2 * inter)
        # rows_in_use: device-side fill level of a buffer sized for the worst case (dropless exchange)
        return grouped_gemm.grouped_linear(swiglu_ops.swiglu(gu, rows_in_use), [e.down_proj for e in experts], layout,
                                           experts[0].down_proj.weight.shape[0])

    def _dispatch(self, rows_sorted, plan: RoutePlan):
        if self.ep_fp8_dispatch:
            return epc.all_to_all_fp8(rows_sorted, plan.out_splits, plan.in_splits, self.ep_group,
                                      self.ep_fp8_granularity)
        return epc.all_to_all(rows_sorted, plan.out_splits, plan.in_splits, self.ep_group)

    def _routed_fused_var(self, routed, expert_idx):
        """Dropless exchange with the layout computed on the device (``ops.fused_ep_var``): no host
        synchronisation, rows stored straight into the owners' expert-major buffers, experts as grouped
        GEMMs over the padded segments, outputs returned into this rank's sorted order."""
        from ..ops import fused_ep_var as fv
        epv = self.fused_ep_var
        order, inv = _argsort_inv(expert_idx)
        from .capacity_moe import expert_counts
        counts = expert_counts(expert_idx, self.num_experts).to(torch.int32)
        plan = epv.plan(counts)
        recv = fv.var_dispatch(routed[order], plan, epv)
        y_pad = self._experts_on_layout(recv, plan.layout, rows_in_use=plan.seg_start[self.num_local_experts:])
        return fv.var_return(y_pad, plan, epv)[inv]

    def _routed_naive(self, routed, expert_idx):
        plan = self.plan(expert_idx)
        x = routed[plan.order]
        if self.ep_world_size == 1:
            y = self.grouped_experts(x, plan.expert_counts)
            return y[plan.inv_order]
        recv = self._dispatch(x, plan)
        y = self.grouped_experts(recv[plan.regroup], plan.expert_counts)
        back = epc.all_to_all(y[plan.regroup_inv], plan.in_splits, plan.out_splits, self.ep_group)
        return back[plan.inv_order]

    def _device_routed_ok(self, tokens) -> bool:
        """Capacity-limited dispatch through the peer-memory kernels with routing, slot assignment and
        the weighted combine on the device (``ops.moe_route``): bf16 CUDA tokens, one round (rows over
        capacity are dropped), a fused exchange context of matching capacity."""
        epf = self.fused_ep
        if epf is None or not tokens.is_cuda or tokens.dtype != torch.bfloat16 or self.ep_capacity_factor <= 0 \
                or self.ep_capacity_dropless or self.ep_world_size == 1 or self.num_experts > 256 or self.top_k > 8:
            return False
        if os.environ.get("PICO_MOE_DEVICE_ROUTING", "1") == "0":
            return False
        from .capacity_moe import compute_capacity
        return epf.C == compute_capacity(tokens.shape[0], self.top_k, self.num_experts, self.ep_capacity_factor) \
            and epf.d == self.expert_dim

    def _forward_device_routed(self, tokens):
        """router GEMM -> route kernel -> slot kernel -> dispatch (peer memory, fp8 optional) -> grouped
        experts -> combine exchange -> weighted-sum kernel: no eager sort / gather / index_add, nothing
        read on the host."""
        from ..ops import fused_ep
        from ..ops import moe_route as mr
        epf, T, k, E = self.fused_ep, tokens.shape[0], self.top_k, self.num_experts
        logits = self.gate(tokens)
        bias = self.expert_bias if self.use_loss_free else None
        probs, idx, w, counts = mr.route(logits, bias, k, self.norm_topk_prob)
        self._balance(probs, idx, counts)
        shared = self._shared_start(tokens)
        latent = self.down_proj_latent(tokens) if self.latent else tokens
        pos, table = mr.slots(idx, E, epf.C)
        x = fused_ep.dispatch(latent, table, k, epf, bool(self.ep_fp8_dispatch), idx, pos.view(T, k))  # [L, ep*C, d]
        out = self.experts_uniform(x)
        back = fused_ep.combine(out, epf)                                             # [E*C, d]
        y = mr.combine(back, idx, pos.view(T, k), w, table, epf.C)
        self.last_dropped_fraction = (pos >= epf.C).float().mean()
        return self._finalize(y, shared)

    # ------------------------------------------------------------------------------ forward
    def forward(self, x):
        shape = x.shape
        tokens = x.reshape(-1, self.hidden_size)
        if self._device_routed_ok(tokens):
            return self._forward_device_routed(tokens).view(shape)
        topk_idx, topk_w = self._route(tokens)
        return self._moe_given_routing(tokens, topk_idx, topk_w, self.ep_capacity_factor > 0).view(shape)

    def _moe_given_routing(self, tokens, topk_idx, topk_w, capped: bool, force_plain: bool = False):
        """``tokens`` [T, hidden] through the experts named by ``topk_idx`` [T, k] with weights ``topk_w``:
        the capacity-limited exchange when ``capped``, otherwise the variable-size one (peer-memory layout,
        tiled pipeline or plain all-to-all, whichever the layer is configured for; ``force_plain`` = the
        plain one). Returns [T, hidden]."""
        T = tokens.shape[0]
        shared = self._shared_start(tokens)
        latent = self.down_proj_latent(tokens) if self.latent else tokens
        token_idx = torch.arange(T, device=tokens.device).repeat_interleave(self.top_k, output_size=T * self.top_k)
        routed = latent[token_idx]                       # [T*k, d] token-major
        expert_idx = topk_idx.reshape(-1)
        weights = topk_w.reshape(-1)
        if capped:
            from .capacity_moe import capacity_moe, compute_capacity
            cap = compute_capacity(T, self.top_k, self.num_experts, self.ep_capacity_factor)
            y, dropped = capacity_moe(self, routed, expert_idx, weights, token_idx, T, cap,
                                      self.ep_capacity_dropless, self.ep_max_rounds, tokens=latent)
            self.last_dropped_fraction = dropped
        else:
            epv = self.fused_ep_var
            if not force_plain and epv is not None and routed.is_cuda and routed.dtype == torch.bfloat16 \
                    and routed.shape[0] == epv.rows_per_rank and self._grouped_ok(routed):
                y_rows = self._routed_fused_var(routed, expert_idx)
            elif not force_plain and self.ep_world_size > 1 and self.ep_num_tiles > 1:
                from .tiled_moe import tiled_moe
                y_rows = tiled_moe(self, routed, expert_idx, self.ep_num_tiles)
            else:
                y_rows = self._routed_naive(routed, expert_idx)
            y = (y_rows * weights.unsqueeze(-1)).view(T, self.top_k, self.expert_dim).sum(dim=1)
        return self._finalize(y, shared)

    # the reference's per-path methods (expert_parallel.py:271-341 there), which its benchmark and ablation
    # scripts call with a routing of their own
    def _moe_naive(self, tokens, topk_idx, topk_weights):
        return self._moe_given_routing(tokens, topk_idx, topk_weights, False, force_plain=True)

    def _moe_capped(self, tokens, topk_idx, topk_weights):
        return self._moe_given_routing(tokens, topk_idx, topk_weights, True)


def collect_aux_loss(model):
    """Sum and drain the auxiliary load-balancing loss of every MoE layer in ``model`` (a module
    or a list of modules). None when no layer produced one (expert_parallel.py:442-454)."""
    mods = model if isinstance(model, (list, tuple)) else [model]
    total = None
    for root in mods:
        for m in root.modules():
            if isinstance(m, MoELayer) and m.aux_loss is not None:
                total = m.aux_loss if total is None else total + m.aux_loss
                m.aux_loss = None
    return total
