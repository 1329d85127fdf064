"""Flat parameter and gradient storage.

``ParamStore(model)`` moves every parameter of a module tree into one contiguous buffer (per
dtype) and gives each an fp32 ``main_grad`` view into one contiguous gradient buffer:

* the optimizer is a single kernel launch over the flat buffers (``ops.adamw.FlatAdamW``)
* weight-gradient GEMMs accumulate directly into ``main_grad`` — the per-parameter
  ``main_grad.add_(grad)`` / ``grad_data.zero_()`` / cast of the reference's bucket manager
  (picotron/data_parallel/bucket.py:96-147, data_parallel.py:134-180) disappears
* data-parallel reduction and ZeRO sharding operate on slices of one buffer
* projections that consume the same input (q/k/v, gate/up) are laid out back to back, so one
  GEMM over the fused ``[sum(out_i), in]`` view replaces several — while the state dict keeps
  the reference's separate ``q_proj`` / ``k_proj`` / ``v_proj`` / ``gate_proj`` / ``up_proj``
  entries, each parameter being a view of the fused block.

Parameter offsets are padded to 128 elements so every view is 256-byte aligned.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

ALIGN = 128


@dataclass
class FusedGroup:
    """Several bias-free linears with the same input, stored back to back."""
    mods: list
    weight: torch.Tensor                 # [sum(out_i), in] view of the flat parameter buffer
    main_grad: Optional[torch.Tensor]    # matching view of the flat fp32 gradient buffer
    splits: List[int]


def _fusion_groups(model: nn.Module):
    """Lists of modules whose weights should be adjacent: q/k/v and gate/up of each block."""
    groups = []
    expert_mlps = set()
    for m in model.modules():
        # routed experts: gate/up of all local experts form one stacked block, the down projections
        # another, so one grouped GEMM covers every local expert
        if getattr(m, "is_moe", False) and hasattr(m, "local_experts"):
            experts = list(m.local_experts)
            if experts and all(hasattr(e, n) for e in experts for n in ("gate_proj", "up_proj", "down_proj")):
                groups.append([p for e in experts for p in (e.gate_proj, e.up_proj)])
                groups.append([e.down_proj for e in experts])
                expert_mlps.update(id(e) for e in experts)
    for m in model.modules():
        if all(hasattr(m, n) for n in ("q_proj", "k_proj", "v_proj")):
            groups.append([m.q_proj, m.k_proj, m.v_proj])
        if all(hasattr(m, n) for n in ("gate_proj", "up_proj")) and not getattr(m, "is_moe", False) \
                and id(m) not in expert_mlps:
            groups.append([m.gate_proj, m.up_proj])
    return groups


class ParamStore:
    def __init__(self, model: nn.Module, with_grads: bool = True, grad_dtype: torch.dtype = torch.float32,
                 pad_to_multiple: int = 1, allocator=None, param_filter=None):
        """``allocator(numel, dtype) -> 1-D tensor`` lets the caller place the flat buffers in special
        memory (symmetric memory for the fused data-parallel optimizer); default: ordinary tensors."""
        params = [p for n, p in model.named_parameters()
                  if p.requires_grad and (param_filter is None or param_filter(n, p))]
        assert params, "no trainable parameters selected"
        selected = {id(p) for p in params}
        dtype, device = params[0].dtype, params[0].device
        assert all(p.dtype == dtype and p.device == device for p in params), \
            "ParamStore needs a single parameter dtype/device (cast the model first)"
        groups = _fusion_groups(model)
        in_group = {}
        for g in groups:
            ws = [m.weight for m in g]
            if any(w.dim() != 2 or w.shape[1] != ws[0].shape[1] or id(w) not in selected for w in ws):
                continue
            for w in ws:
                in_group[id(w)] = g
        order: List[nn.Parameter] = []
        seen = set()
        starts_group: Dict[int, list] = {}
        for p in params:
            if id(p) in seen:
                continue
            g = in_group.get(id(p))
            if g is None:
                order.append(p)
                seen.add(id(p))
            else:
                starts_group[id(g[0].weight)] = g
                for m in g:
                    if id(m.weight) not in seen:
                        order.append(m.weight)
                        seen.add(id(m.weight))
        # offsets: members of a fused group are packed without padding between them
        offsets, off = {}, 0
        grouped_follow = set()
        for g in starts_group.values():
            for m in g[1:]:
                grouped_follow.add(id(m.weight))
        for p in order:
            if id(p) not in grouped_follow:
                off = (off + ALIGN - 1) // ALIGN * ALIGN
            offsets[id(p)] = off
            off += p.numel()
        total = (off + ALIGN - 1) // ALIGN * ALIGN
        if pad_to_multiple > 1:
            total = (total + pad_to_multiple * ALIGN - 1) // (pad_to_multiple * ALIGN) * (pad_to_multiple * ALIGN)
        self.numel = total
        self.params = order
        self.offsets = offsets
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat_params = alloc(total, dtype)
        self.flat_grads = alloc(total, grad_dtype) if with_grads else None
        if allocator is not None:
            self.flat_params.zero_()
            if self.flat_grads is not None:
                self.flat_grads.zero_()
        with torch.no_grad():
            for p in order:
                o = offsets[id(p)]
                view = self.flat_params[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                if with_grads:
                    p.main_grad = self.flat_grads[o:o + p.numel()].view(p.shape)
                    p.grad = None
        self.fused_groups: List[FusedGroup] = []
        for g in starts_group.values():
            ws = [m.weight for m in g]
            o = offsets[id(ws[0])]
            rows = sum(w.shape[0] for w in ws)
            k = ws[0].shape[1]
            fw = self.flat_params[o:o + rows * k].view(rows, k)
            fg = self.flat_grads[o:o + rows * k].view(rows, k) if with_grads else None
            fused = FusedGroup(mods=list(g), weight=fw, main_grad=fg, splits=[w.shape[0] for w in ws])
            for m in g:
                m._fused_group = fused
            self.fused_groups.append(fused)

    def param_slice(self, p: nn.Parameter):
        o = self.offsets[id(p)]
        return o, o + p.numel()

    def zero_grads(self):
        if self.flat_grads is not None:
            self.flat_grads.zero_()
