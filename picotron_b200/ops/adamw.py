"""AdamW over flat buffers: one kernel launch per optimizer step per buffer.

``FlatAdamW`` owns fp32 ``exp_avg`` / ``exp_avg_sq`` (and optionally fp32 master weights) for a
flat bf16 parameter buffer whose gradients live in a flat fp32 buffer, applies the gradient
scale (1 / data-parallel size, 1 / accumulation steps), the decoupled weight decay of
``torch.optim.AdamW`` and zeroes the gradient buffer in the same pass — the work the reference
spreads over ``grad_data /= n`` (picotron/data_parallel/bucket.py:34), the foreach AdamW of
train.py:289 and ``grad_data.zero_()`` (bucket.py:43).
"""
from __future__ import annotations

import torch

from . import count_launch, ext, use_kernels


def adamw_ref_(p, g, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale=1.0, master=None):
    """In-place reference update with the same arithmetic as the kernel."""
    gf = g.float() * grad_scale
    pf = master if master is not None else p.float()
    pf = pf * (1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gf, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = v.sqrt() / (bc2 ** 0.5) + eps
    pf = pf - (lr / bc1) * m / denom
    if master is not None:
        master.copy_(pf)
    p.copy_(pf.to(p.dtype))


class FlatAdamW:
    """AdamW on a flat parameter / gradient buffer pair (optionally a shard of them)."""

    def __init__(self, params: torch.Tensor, grads: torch.Tensor, lr=3e-4, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.01, master_weights: bool = False):
        assert params.numel() == grads.numel() and grads.dtype == torch.float32
        self.params, self.grads = params, grads
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.exp_avg = torch.zeros_like(grads)
        self.exp_avg_sq = torch.zeros_like(grads)
        self.master = params.float() if (master_weights and params.dtype != torch.float32) else None
        self.step_count = 0

    def step(self, grad_scale: float = 1.0, zero_grad: bool = True):
        self.step_count += 1
        b1, b2 = self.betas
        bc1 = 1.0 - b1 ** self.step_count
        bc2 = 1.0 - b2 ** self.step_count
        if use_kernels(self.params):
            ext().adamw(self.params, self.master, self.grads, self.exp_avg, self.exp_avg_sq,
                        self.params.numel(), self.lr, b1, b2, self.eps, self.weight_decay, bc1, bc2,
                        grad_scale, zero_grad)
            count_launch()
        else:
            adamw_ref_(self.params, self.grads, self.exp_avg, self.exp_avg_sq, self.step_count, self.lr,
                       b1, b2, self.eps, self.weight_decay, grad_scale, self.master)
            if zero_grad:
                self.grads.zero_()

    def state_dict(self):
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "master": self.master, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])
