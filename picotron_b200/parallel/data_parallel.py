"""Data parallelism over autograd gradients: the naive per-parameter all-reduce and the bucketed,
overlapped variant. Public behaviour as picotron/data_parallel/data_parallel.py:12-186:

* ``require_backward_grad_sync`` / ``no_sync()`` suppress communication while gradients
  accumulate over micro-batches
* ``DataParallelBucket`` accumulates in fp32 ``main_grad`` buffers, fires one async all-reduce
  per bucket as soon as the bucket is complete, and hands ``p.grad = main_grad`` (cast to the
  parameter dtype) to the optimizer after the backward; ``reset()`` clears the buckets
* gradients are averaged over the group — by default CP x DP, since context-parallel ranks hold
  different tokens of the same batch
* ``backward(...)`` is forwarded to a wrapped pipeline stage

(The CUDA training path does not use these wrappers: there gradients are accumulated by the
GEMM epilogues into a flat buffer that is reduced in one piece; see ``engine.FlatOptimizer``.)
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import process_group_manager as pgm
from .bucket import BucketManager
from .dist_utils import group_size


class _DataParallelBase(nn.Module):
    def __init__(self, module: nn.Module, group=None):
        super().__init__()
        self.module = module
        self.group = group if group is not None else pgm.get_pgm().cp_dp_group
        self.world_size = group_size(self.group)
        self.require_backward_grad_sync = True

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def backward(self, *args, **kwargs):
        return self.module.backward(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)

    @contextlib.contextmanager
    def no_sync(self):
        prev = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = prev


    def sync_all(self):
        """Average every gradient over the group now. Used when gradients were produced outside
        the hooks' view (deferred weight gradients of the zero-bubble schedules)."""
        for p in self.module.parameters():
            if p.requires_grad and p.grad is not None and self.world_size > 1:
                dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group)
                p.grad /= self.world_size


class DataParallelNaive(_DataParallelBase):
    """All-reduce every gradient as soon as it has been accumulated, then divide by the group size."""

    def __init__(self, module: nn.Module, group=None):
        super().__init__(module, group)
        for p in self.module.parameters():
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._hook)

    def _hook(self, p):
        if self.require_backward_grad_sync and self.world_size > 1:
            dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group)
            p.grad /= self.world_size

    def reset(self):
        pass


class DataParallelBucket(_DataParallelBase):
    def __init__(self, module: nn.Module, bucket_cap_mb: float = 25, grad_type: torch.dtype = torch.float32,
                 group=None):
        super().__init__(module, group)
        elem = torch.tensor([], dtype=grad_type).element_size()
        bucket_size = int(bucket_cap_mb * 1024 * 1024 // elem)
        self.bucket_manager = BucketManager(list(module.parameters()), self.group, bucket_size, grad_type)
        self._post_backward_queued = False
        self._grad_accs = []
        for p in module.parameters():
            if p.requires_grad:
                # hook the AccumulateGrad node: it runs when the full gradient of p is known
                acc = p.expand_as(p).grad_fn.next_functions[0][0]
                acc.register_hook(self._make_hook(p))
                self._grad_accs.append(acc)

    def _make_hook(self, p):
        def hook(*unused):
            if p.grad is None:
                return
            p.main_grad.add_(p.grad.data)
            p.grad = None
            if self.require_backward_grad_sync:
                if not self._post_backward_queued:
                    torch.autograd.Variable._execution_engine.queue_callback(self._post_backward)
                    self._post_backward_queued = True
                self.bucket_manager.mark_param_as_ready(p)
        return hook

    def _post_backward(self):
        self.bucket_manager.wait()
        self._post_backward_queued = False
        for p in self.bucket_manager.params:
            p.grad = p.main_grad.to(p.dtype)

    def reset(self):
        self.bucket_manager.reset()

    def sync_all(self):
        bm = self.bucket_manager
        for p in bm.params:
            if p.grad is not None:      # late gradients that bypassed the accumulation hook
                p.main_grad.add_(p.grad.data)
                p.grad = None
        if self.world_size > 1:
            dist.all_reduce(bm.grad_data, group=self.group)
            bm.grad_data /= self.world_size
        for p in bm.params:
            p.grad = p.main_grad.to(p.dtype)


class DataParallelExpertAware(_DataParallelBase):
    """Gradient averaging when expert parallelism doubles as data parallelism (every EP rank holds
    different tokens): dense parameters are replicated over CP x EP x DP and averaged over that
    whole group; an expert lives on one EP rank only, so its gradient — which already contains the
    contributions of every EP rank's tokens through the backward of the dispatch — is summed over
    CP x DP and divided by the size of the whole group."""

    def __init__(self, module: nn.Module, dense_group, expert_group, is_expert=None):
        super().__init__(module, dense_group)
        self.expert_group = expert_group
        self.expert_world = group_size(expert_group)
        is_expert = is_expert or (lambda name: ".local_experts." in name)
        self._expert_ids = {id(p) for n, p in module.named_parameters() if is_expert(n)}
        for p in self.module.parameters():
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._hook)

    def _hook(self, p):
        if not self.require_backward_grad_sync:
            return
        if id(p) in self._expert_ids:
            if self.expert_world > 1:
                dist.all_reduce(p.grad, group=self.expert_group)
            p.grad /= self.world_size
        elif self.world_size > 1:
            dist.all_reduce(p.grad, group=self.group)
            p.grad /= self.world_size

    def reset(self):
        pass
