"""Token-tiled MoE pipeline: the routed rows are cut into ``num_tiles`` contiguous tiles and
dispatch / expert FFN / combine of neighbouring tiles overlap, in the forward and in the
backward pass (MegaScale-style; picotron/expert_parallel/tiled_moe.py:61-185).

  forward :  dispatch(i+1)  ||  experts(i)            ||  combine(i-1)
  backward:  combine_rev(i+1) || experts_backward(i)  ||  dispatch_rev(i-1)

One autograd Function owns both schedules. The exchanges are asynchronous single-buffer
all-to-alls; each tile's expert FFN is recorded as its own small autograd graph in the forward
and replayed in the backward, which accumulates the expert weight gradients directly. The tile
count is fixed, so ranks whose tiles are empty still take part in every collective. With FP8
dispatch enabled the forward payload of every tile is quantised as well (the reference leaves
the tiled path in bf16).
"""
from __future__ import annotations

import torch

from ..ops import quant
from . import ep_communications as epc


class _TiledMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, routed, layer, expert_idx, num_tiles, *expert_params):
        R, d = routed.shape
        group = layer.ep_group
        bounds = [(i * R) // num_tiles for i in range(num_tiles + 1)]
        plans = [layer.plan(expert_idx[bounds[i]:bounds[i + 1]]) for i in range(num_tiles)]
        fp8 = layer.ep_fp8_dispatch
        gran = layer.ep_fp8_granularity

        def launch_dispatch(i):
            p = plans[i]
            x = routed[bounds[i]:bounds[i + 1]][p.order]
            if fp8:
                payload, scales = quant.quantize_fp8(x, gran)
                a = epc.all_to_all_no_grad_async(payload, p.out_splits, p.in_splits, group)
                b = epc.all_to_all_no_grad_async(scales, p.out_splits, p.in_splits, group)
                return ("fp8", a, b)
            return ("raw", epc.all_to_all_no_grad_async(x, p.out_splits, p.in_splits, group))

        def finish_dispatch(h):
            if h[0] == "fp8":
                (pay, w1), (sc, w2) = h[1], h[2]
                w1.wait()
                w2.wait()
                return quant.dequantize_fp8(pay, sc, routed.dtype, gran)
            out, w = h[1]
            w.wait()
            return out

        out_rows = torch.empty_like(routed)
        graphs = []
        pending_combine = []
        nxt = launch_dispatch(0)
        for i in range(num_tiles):
            cur, nxt = nxt, (launch_dispatch(i + 1) if i + 1 < num_tiles else None)
            p = plans[i]
            recv = finish_dispatch(cur)
            with torch.enable_grad():
                xin = recv[p.regroup].detach().requires_grad_(True)
                yout = layer.grouped_experts(xin, p.expert_counts)
            graphs.append((xin, yout))
            pending_combine.append(epc.all_to_all_no_grad_async(yout.detach()[p.regroup_inv], p.in_splits,
                                                                p.out_splits, group))
            if i >= 1:   # complete the combine of the previous tile while this one is in flight
                back, w = pending_combine[i - 1]
                w.wait()
                out_rows[bounds[i - 1]:bounds[i]] = back[plans[i - 1].inv_order]
        back, w = pending_combine[-1]
        w.wait()
        out_rows[bounds[-2]:bounds[-1]] = back[plans[-1].inv_order]
        ctx.plans, ctx.bounds, ctx.graphs, ctx.group = plans, bounds, graphs, group
        return out_rows

    @staticmethod
    def backward(ctx, dy):
        plans, bounds, graphs, group = ctx.plans, ctx.bounds, ctx.graphs, ctx.group
        n = len(plans)
        d_routed = torch.empty_like(dy)

        def launch_combine_rev(i):
            p = plans[i]
            g = dy[bounds[i]:bounds[i + 1]][p.order]
            return epc.all_to_all_no_grad_async(g, p.out_splits, p.in_splits, group)

        pending = []
        nxt = launch_combine_rev(0)
        for i in range(n):
            cur, nxt = nxt, (launch_combine_rev(i + 1) if i + 1 < n else None)
            p = plans[i]
            g_recv, w = cur
            w.wait()
            xin, yout = graphs[i]
            torch.autograd.backward(yout, g_recv[p.regroup])
            dx = xin.grad if xin.grad is not None else torch.zeros_like(xin)
            pending.append(epc.all_to_all_no_grad_async(dx[p.regroup_inv], p.in_splits, p.out_splits, group))
            if i >= 1:
                back, w = pending[i - 1]
                w.wait()
                d_routed[bounds[i - 1]:bounds[i]] = back[plans[i - 1].inv_order]
        back, w = pending[-1]
        w.wait()
        d_routed[bounds[-2]:bounds[-1]] = back[plans[-1].inv_order]
        ctx.graphs = None
        return (d_routed, None, None, None) + (None,) * (len(ctx.needs_input_grad) - 4)


def tiled_moe(layer, routed: torch.Tensor, expert_idx: torch.Tensor, num_tiles: int) -> torch.Tensor:
    """Expert outputs for the routed rows, in routed order, computed tile by tile."""
    params = [p for e in layer.local_experts for p in e.parameters()]
    return _TiledMoE.apply(routed, layer, expert_idx, max(1, num_tiles), *params)
