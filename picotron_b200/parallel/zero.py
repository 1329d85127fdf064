"""ZeRO stages 1, 2 and 3 over autograd gradients, with whole-parameter ownership.

Same contract as picotron/data_parallel/zero.py:48-242: ``assign_param_owners`` balances
parameters over the ranks greedily (largest first); stage 1/2 average every gradient over the
group (stage 2 drops it on non-owners); stage 3 additionally keeps parameter storage only on
the owner and broadcasts it just-in-time around each module's forward and backward.
``ShardedOptimizer`` steps only the owned parameters and re-broadcasts them (stage 1/2).

Gradients are averaged with an all-reduce rather than a reduce-scatter so that results are
bit-identical to plain data parallelism, which is what the tests assert.
"""
from __future__ import annotations

import contextlib
from typing import Dict, List

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import process_group_manager as pgm
from .dist_utils import group_rank, group_size


def assign_param_owners(params: List[torch.nn.Parameter], world_size: int) -> Dict[torch.nn.Parameter, int]:
    """Greedy balance: visit parameters from largest to smallest, give each to the lightest rank
    (ties: lowest rank). Deterministic, so every rank computes the same map."""
    load = [0] * world_size
    owners = {}
    order = sorted(range(len(params)), key=lambda i: (-params[i].numel(), i))
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        owners[params[i]] = r
        load[r] += params[i].numel()
    return owners


class DataParallelZero(nn.Module):
    def __init__(self, module: nn.Module, stage: int = 1, group=None):
        super().__init__()
        assert stage in (1, 2, 3)
        self.module, self.stage = module, stage
        self.group = group if group is not None else pgm.get_pgm().cp_dp_group
        self.world_size = group_size(self.group)
        self.rank = group_rank(self.group)
        self.require_backward_grad_sync = True
        params = [p for p in module.parameters() if p.requires_grad]
        self.owners = assign_param_owners(params, self.world_size)
        self.owned_params = [p for p in params if self.owners[p] == self.rank]
        for p in params:
            p.register_post_accumulate_grad_hook(self._grad_hook)
        if stage == 3:
            self._setup_param_sharding()

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def backward(self, *args, **kwargs):
        return self.module.backward(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """No gradient reduction inside the block (micro-batches before the last one of a step)."""
        prev = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = prev

    def owns(self, p) -> bool:
        return self.owners[p] == self.rank

    def owner_global_rank(self, p) -> int:
        r = self.owners[p]
        return dist.get_global_rank(self.group, r) if (self.group is not None and dist.is_initialized()) else r

    def reset(self):
        pass

    def sync_all(self):
        for p in self.module.parameters():
            if p.requires_grad and p.grad is not None:
                if self.world_size > 1:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group)
                    p.grad /= self.world_size
                if self.stage >= 2 and not self.owns(p):
                    p.grad = None

    # --- gradients ---------------------------------------------------------------------------
    def _grad_hook(self, p):
        if self.stage == 3:
            self._free(p)
        if not self.require_backward_grad_sync:
            return
        if self.world_size > 1:
            dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group)
            p.grad /= self.world_size
        if self.stage >= 2 and not self.owns(p):
            p.grad = None

    # --- stage 3: parameter storage only on the owner ------------------------------------------
    def _setup_param_sharding(self):
        self._full_nbytes = {}
        for p in self.module.parameters():
            if not p.requires_grad:
                continue
            self._full_nbytes[p] = p.data.untyped_storage().nbytes()
            if not self.owns(p):
                p.data.untyped_storage().resize_(0)
        for unit in self._units(self.module):
            own = [p for p in unit.parameters() if p.requires_grad]
            if not own:
                continue
            unit.register_forward_pre_hook(lambda m, a, ps=own: self._gather(ps))
            unit.register_forward_hook(lambda m, a, out, ps=own: self._after_forward(ps, out))

    @staticmethod
    def _units(root):
        """Gather/free granularity: the children of the root (the elements of list/dict containers
        individually) — for a Llama: embedding, each decoder layer, final norm, lm head. A unit's
        parameters are materialised together because inner modules may read each other's weights
        without going through ``__call__`` (fused q/k/v and gate/up projections)."""
        units = []
        for child in root.children():
            if isinstance(child, (nn.ModuleList, nn.ModuleDict, nn.Sequential)):
                units.extend(child.children())
            else:
                units.append(child)
        if any(True for _ in root.parameters(recurse=False)) or not units:
            units = [root]
        return units

    def _gather(self, ps):
        for p in ps:
            st = p.data.untyped_storage()
            if st.nbytes() == 0:
                st.resize_(self._full_nbytes[p])
            if self.world_size > 1:
                dist.broadcast(p.data, src=self.owner_global_rank(p), group=self.group)

    def _free(self, p):
        if not self.owns(p):
            p.data.untyped_storage().resize_(0)

    def _after_forward(self, ps, out):
        for p in ps:
            self._free(p)
        # re-gather right before this module's backward needs the weights
        tensors = [t for t in (out if isinstance(out, (tuple, list)) else (out,)) if torch.is_tensor(t)]
        for t in tensors:
            if t.requires_grad:
                t.register_hook(lambda g, ps=ps: (self._gather(ps), g)[1])
                break

    def full_parameters(self):
        """Gather and return copies of all parameters (for tests and checkpoints)."""
        out = []
        for p in self.module.parameters():
            if not p.requires_grad:
                continue
            if self.stage == 3:
                self._gather([p])
                out.append(p.data.clone())
                self._free(p)
            else:
                out.append(p.data.clone())
        return out


class ShardedOptimizer:
    def __init__(self, dp_zero: DataParallelZero, optimizer_cls=torch.optim.AdamW, **opt_kwargs):
        self.dp = dp_zero
        self.stage = dp_zero.stage
        self.optimizer = optimizer_cls(dp_zero.owned_params, **opt_kwargs)

    def zero_grad(self, set_to_none: bool = True):
        for p in self.dp.module.parameters():
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    @torch.no_grad()
    def step(self, *args, **kwargs):
        loss = self.optimizer.step(*args, **kwargs)
        if self.stage in (1, 2) and self.dp.world_size > 1:
            for p in self.dp.module.parameters():
                if p.requires_grad:
                    dist.broadcast(p.data, src=self.dp.owner_global_rank(p), group=self.dp.group)
        return loss

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd)
