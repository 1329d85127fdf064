"""Gradient buckets for bucketed data parallelism.

A ``Bucket`` is a slice of one flat gradient buffer; parameters registered in it get a
``main_grad`` view. When every parameter of a bucket has accumulated its gradient the bucket is
averaged over the group with one asynchronous all-reduce. ``BucketManager`` assigns parameters
to buckets of at most ``bucket_size`` elements in reverse registration order (the order in
which the backward produces gradients), so early buckets reduce while later layers are still
in backward. Behaviour follows picotron/data_parallel/bucket.py:9-180; the layout differs: one
allocation for all buckets, so the same buffer can be handed to a flat optimizer.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.distributed as dist

from .dist_utils import group_size


class Bucket:
    def __init__(self, params: List[torch.nn.Parameter], grad_data: torch.Tensor, process_group):
        self.params = set(params)
        self.params_with_grad_ready = set()
        self.grad_data = grad_data
        self.process_group = process_group
        self.process_group_size = group_size(process_group)
        self.handle = None
        self.reset()

    def sync_gradient(self) -> None:
        """Average this bucket over the group (asynchronously)."""
        assert self.handle is None
        self.grad_data /= self.process_group_size
        if self.process_group_size > 1:
            self.handle = dist.all_reduce(self.grad_data, group=self.process_group, async_op=True)

    def reset(self) -> None:
        self.handle = None
        self.params_with_grad_ready.clear()
        self.grad_data.zero_()

    def wait(self) -> None:
        if self.handle is not None:
            self.handle.wait()
            self.handle = None

    def mark_param_as_ready(self, param) -> None:
        assert param in self.params and param not in self.params_with_grad_ready
        self.params_with_grad_ready.add(param)
        if len(self.params_with_grad_ready) == len(self.params):
            self.sync_gradient()


class BucketManager:
    def __init__(self, params: List[torch.nn.Parameter], process_group, bucket_size: int,
                 grad_type: torch.dtype = torch.float32):
        self.params = [p for p in params if p.requires_grad]
        self.device = self.params[0].device if self.params else torch.device("cpu")
        self.process_group = process_group
        self.bucket_size = bucket_size
        self.grad_type = grad_type
        self.buckets: List[Bucket] = []
        self.params_to_bucket_location: Dict[torch.nn.Parameter, tuple] = {}
        self._build()

    def _build(self) -> None:
        # greedy packing in reverse order; a parameter larger than the cap gets its own bucket
        assignments: List[List[torch.nn.Parameter]] = [[]]
        fill = 0
        for p in reversed(self.params):
            n = p.numel()
            if assignments[-1] and fill + n > self.bucket_size:
                assignments.append([])
                fill = 0
            assignments[-1].append(p)
            fill += n
        total = sum(p.numel() for p in self.params)
        self.grad_data = torch.zeros(total, dtype=self.grad_type, device=self.device)
        off = 0
        for idx, plist in enumerate(assignments):
            start = off
            for p in plist:
                self.params_to_bucket_location[p] = (off, off + p.numel(), idx)
                p.main_grad = self.grad_data[off:off + p.numel()].view(p.shape)
                off += p.numel()
            self.buckets.append(Bucket(plist, self.grad_data[start:off], self.process_group))

    def reset(self) -> None:
        for b in self.buckets:
            b.reset()

    def wait(self) -> None:
        for b in self.buckets:
            b.wait()

    def mark_param_as_ready(self, param) -> None:
        self.buckets[self.params_to_bucket_location[param][2]].mark_param_as_ready(param)
