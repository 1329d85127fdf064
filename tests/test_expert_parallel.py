"""MoE layer: every execution path against a loop-over-tokens reference (the oracle of the
reference's tests/test_expert_parallel.py:32-48), on one rank and on two gloo ranks; capacity
and load-balancing behaviour; FP8 dispatch accuracy."""
import types

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def moe_config(**kw):
    cfg = dict(hidden_size=32, intermediate_size=48, num_experts=4, num_experts_per_tok=2, num_shared_experts=1,
               norm_topk_prob=True, ep_num_tiles=1, ep_fp8_dispatch=False, moe_latent_dim=0, ep_capacity_factor=0.0,
               ep_capacity_dropless=True, ep_max_rounds=8, router_aux_loss_coef=0.0, router_bias_update_rate=0.0,
               ep_overlap=True)
    cfg.update(kw)
    return types.SimpleNamespace(**cfg)


def reference_moe(x, gate_w, experts, shared, top_k, norm):
    """Token-by-token mixture with all experts available. experts: list of (gate, up, down)."""
    def mlp(w, t):
        g, u, dn = w
        return torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(t, g)) *
                                          torch.nn.functional.linear(t, u), dn)
    tokens = x.reshape(-1, x.shape[-1])
    probs = torch.softmax(tokens @ gate_w.t(), dim=-1, dtype=torch.float32)
    out = torch.zeros_like(tokens)
    for t in range(tokens.shape[0]):
        w, idx = torch.topk(probs[t], top_k)
        if norm and top_k > 1:
            w = w / w.sum()
        for wi, ei in zip(w, idx):
            out[t] += wi.to(tokens.dtype) * mlp(experts[int(ei)], tokens[t:t + 1])[0]
        if shared is not None:
            out[t] += mlp(shared, tokens[t:t + 1])[0]
    return out.view_as(x)


def _gather_experts(layer, world):
    local = [(e.gate_proj.weight.detach(), e.up_proj.weight.detach(), e.down_proj.weight.detach())
             for e in layer.local_experts]
    if world == 1:
        return local
    allw = [None] * world
    dist.all_gather_object(allw, local)
    return [w for rank_list in allw for w in rank_list]


def _moe_worker(rank, world, overrides):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer

    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    cfg = moe_config(**overrides)
    torch.manual_seed(21)
    layer = MoELayer(cfg)
    with torch.no_grad():  # distinct experts per rank (the shared RNG stream makes them equal)
        for e in layer.local_experts:
            for p in e.parameters():
                p.add_(0.05 * (rank + 1) * torch.randn_like(p))
    torch.manual_seed(5)
    x = torch.randn(2, 12, cfg.hidden_size, requires_grad=True)
    y = layer(x)
    experts = _gather_experts(layer, world)
    sh = layer.shared_expert
    shared = (sh.gate_proj.weight.detach(), sh.up_proj.weight.detach(), sh.down_proj.weight.detach()) if sh else None
    xr = x.detach().clone().requires_grad_(True)
    yr = reference_moe(xr, layer.gate.weight.detach(), experts, shared, cfg.num_experts_per_tok, True)
    assert (y - yr).abs().max().item() < 1e-5, overrides
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert (x.grad - xr.grad).abs().max().item() < 1e-5, overrides


PATHS = [dict(), dict(ep_num_tiles=3), dict(ep_capacity_factor=8.0), dict(ep_capacity_factor=0.5, ep_capacity_dropless=True),
         dict(num_shared_experts=0), dict(num_experts_per_tok=1)]


@pytest.mark.parametrize("overrides", PATHS)
def test_moe_single_rank(overrides):
    run_distributed(_moe_worker, 1, overrides)


@pytest.mark.parametrize("overrides", PATHS + [dict(ep_num_tiles=7)])
def test_moe_ep2(overrides):
    run_distributed(_moe_worker, 2, overrides)


def _paths_agree_worker(rank, world):
    """naive == tiled == dropless-capacity, outputs and expert gradients (1e-5)."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    results = []
    for ov in (dict(), dict(ep_num_tiles=4), dict(ep_capacity_factor=0.25, ep_max_rounds=64), dict(moe_latent_dim=16)):
        torch.manual_seed(9)
        layer = MoELayer(moe_config(**ov))
        torch.manual_seed(100 + rank)
        x = torch.randn(3, 10, 32, requires_grad=True)
        y = layer(x)
        y.square().sum().backward()
        results.append((ov, y.detach(), [p.grad.clone() for p in layer.local_experts.parameters()], x.grad.clone()))
    base = results[0]
    for ov, y, grads, xg in results[1:3]:
        assert (y - base[1]).abs().max().item() < 1e-5, ov
        assert (xg - base[3]).abs().max().item() < 1e-4, ov
        for a, b in zip(grads, base[2]):
            assert (a - b).abs().max().item() < 1e-4, ov
    assert torch.isfinite(results[3][1]).all()


def test_paths_agree_ep2():
    run_distributed(_paths_agree_worker, 2)


def _capped_drop_worker(rank, world):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    torch.manual_seed(1)
    layer = MoELayer(moe_config(ep_capacity_factor=0.5, ep_capacity_dropless=False))
    x = torch.randn(2, 16, 32, requires_grad=True)
    y = layer(x)
    assert torch.isfinite(y).all() and layer.last_dropped_fraction.item() > 0
    y.sum().backward()
    assert torch.isfinite(x.grad).all()


def test_capped_drop_is_finite():
    run_distributed(_capped_drop_worker, 2)


def _fp8_worker(rank, world, gran):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    outs = []
    for fp8 in (False, True):
        torch.manual_seed(2)
        layer = MoELayer(moe_config(hidden_size=256, intermediate_size=64, ep_fp8_dispatch=fp8))
        layer.ep_fp8_granularity = gran
        torch.manual_seed(50 + rank)
        x = torch.randn(2, 32, 256, requires_grad=True)
        y = layer(x)
        y.sum().backward()
        outs.append((y.detach(), x.grad.clone()))
    rel = (outs[1][0] - outs[0][0]).norm() / outs[0][0].norm()
    assert 0 < rel.item() < 0.05, rel.item()      # the bound of the reference's tests/test_fp8_dispatch.py:85
    assert torch.isfinite(outs[1][1]).all()


@pytest.mark.parametrize("gran", ["block", "row"])
def test_fp8_dispatch_ep2(gran):
    run_distributed(_fp8_worker, 2, gran)


def test_quant_roundtrip_block_scales():
    from picotron_b200.ops import quant
    torch.manual_seed(0)
    x = torch.randn(64, 300) * torch.logspace(-2, 2, 300)
    for gran in ("block", "row"):
        p, s = quant.quantize_fp8(x, gran)
        assert p.dtype == torch.uint8 and p.shape == x.shape
        assert s.shape == (64, 3 if gran == "block" else 1)
        back = quant.dequantize_fp8(p, s, torch.float32, gran)
        rel = (back - x).norm() / x.norm()
        assert rel < 0.05
    # block scales adapt to the column-wise dynamic range, row scales cannot
    pb, sb = quant.quantize_fp8(x, "block")
    pr, sr = quant.quantize_fp8(x, "row")
    eb = (quant.dequantize_fp8(pb, sb, torch.float32, "block") - x)[:, :128].abs().mean()
    er = (quant.dequantize_fp8(pr, sr, torch.float32, "row") - x)[:, :128].abs().mean()
    assert eb < er


def test_aux_loss_and_bias_controller():
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer, collect_aux_loss
    pgm.process_group_manager = None
    torch.manual_seed(0)
    layer = MoELayer(moe_config(num_experts=8, router_aux_loss_coef=0.01, router_bias_update_rate=0.01))
    layer.train()
    x = torch.randn(4, 64, 32)
    layer(x)
    aux = collect_aux_loss(layer)
    assert aux is not None and aux.item() > 0
    aux.backward()
    assert layer.gate.weight.grad.abs().sum().item() > 0
    assert collect_aux_loss(layer) is None           # drained
    # the controller raises the bias of under-loaded experts and lowers over-loaded ones
    with torch.no_grad():
        layer.expert_bias.zero_()
        tokens = x.reshape(-1, 32)
        probs = torch.softmax(layer.gate(tokens), -1)
        idx = torch.topk(probs, 2).indices
        load = torch.bincount(idx.reshape(-1), minlength=8).float()
    layer(x)
    assert torch.equal(torch.sign(layer.expert_bias), torch.sign(load.mean() - load))


def test_loss_free_bias_reduces_imbalance():
    """The sign controller oscillates step to step, but the load accumulated over many steps is
    far more uniform with it than without (the criterion of the reference's
    tests/test_load_balance.py:78-95: time-averaged load std at least halves)."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.expert_parallel import MoELayer
    pgm.process_group_manager = None
    torch.manual_seed(2)
    x = torch.randn(8, 16, 32)

    def cumulative_load(rate):
        torch.manual_seed(0)
        layer = MoELayer(moe_config(num_experts=8, num_shared_experts=0, router_bias_update_rate=rate))
        layer.train()
        total = torch.zeros(8)
        with torch.no_grad():
            for _ in range(300):
                layer(x)
                probs = torch.softmax(layer.gate(x.reshape(-1, 32)), -1) + layer.expert_bias
                total += torch.bincount(torch.topk(probs, 2).indices.reshape(-1), minlength=8).float()
        return total

    off, on = cumulative_load(0.0), cumulative_load(0.01)
    assert on.std() < 0.5 * off.std(), (off.std().item(), on.std().item())


def test_group_layout_pads_expert_segments_to_tiles():
    """The padded expert-major layout of the grouped expert GEMM: segment starts are multiples of 128,
    pad/unpad round-trip, padding rows are zero, and the per-expert restatement on the padded rows
    equals the per-expert loop on the unpadded ones."""
    from picotron_b200.ops.grouped_gemm import GroupLayout, grouped_linear_ref
    counts = [5, 0, 300, 129, 128]
    layout = GroupLayout.from_counts(counts, "cpu")
    seg = layout.seg_start.tolist()
    assert seg == [0, 128, 128, 512, 768, 896] and layout.rows == 896
    assert layout.tile_group.tolist() == [0, 2, 2, 2, 3, 3, 4]
    torch.manual_seed(0)
    x = torch.randn(sum(counts), 16)
    xp = layout.pad(x)
    assert xp.shape == (896, 16) and torch.equal(layout.unpad(xp), x)
    assert xp.abs().sum().item() == pytest.approx(x.abs().sum().item(), rel=1e-6)
    ws = [torch.randn(24, 16) for _ in counts]
    y = layout.unpad(grouped_linear_ref(xp, ws, layout))
    ref, off = [], 0
    for c, w in zip(counts, ws):
        ref.append(x[off:off + c] @ w.t())
        off += c
    assert torch.allclose(y, torch.cat(ref), atol=1e-5)
    uniform = GroupLayout.uniform(3, 256, "cpu")
    assert uniform.pad_index is None and uniform.seg_start.tolist() == [0, 256, 512, 768]


def test_dropless_layout_reference_is_consistent_across_ranks():
    """Invariants of the dropless exchange layout (the Python restatement that the layout kernel is
    tested against): every sender's block for an expert lands inside that expert's segment at the
    receiver without overlapping another sender's block, segments are 128-aligned and cover exactly
    the rows sent, and the return blocks of the receiver are the inverse of the senders' blocks."""
    from picotron_b200.ops.fused_ep_var import var_layout_ref
    ep, L = 4, 3
    E = ep * L
    g = torch.Generator().manual_seed(11)
    table = torch.randint(0, 400, (ep, E), generator=g).tolist()
    for s in range(ep):
        table[s][4] = 0
    max_rows = 128 * 64
    layouts = [var_layout_ref(table, L, r, max_rows) for r in range(ep)]
    for recv in range(ep):
        _, ret, seg_start, seg_len, tiles = layouts[recv]
        assert all(x % 128 == 0 for x in seg_start)
        for l in range(L):
            e = recv * L + l
            total = sum(table[s][e] for s in range(ep))
            assert seg_len[l] == total and seg_start[l + 1] - seg_start[l] == (total + 127) // 128 * 128
            covered = []
            for s in range(ep):
                cnt, src_row, dst_rank, dst_row = layouts[s][0][e]        # sender s's block for expert e
                assert dst_rank == recv and cnt == table[s][e]
                assert src_row == sum(table[s][:e])
                covered.append((dst_row, dst_row + cnt))
                # the receiver sends the block back to where it came from
                rc, r_src, r_rank, r_dst = ret[s * L + l]
                assert (rc, r_src, r_rank, r_dst) == (cnt, dst_row, s, src_row)
            covered.sort()
            assert covered[0][0] == seg_start[l] and covered[-1][1] == seg_start[l] + total
            assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
        used = seg_start[L] // 128
        assert all(t >= 0 for t in tiles[:used]) and all(t == -1 for t in tiles[used:])


def test_fused_capacity_routing_matches_plain_path(monkeypatch):
    """The bookkeeping around the peer-memory exchange kernels of the capacity path (slot table
    without boolean-mask indexing, masked weighted sum) against the plain path, with the two exchange
    kernels emulated by their definition on one rank: outputs, dropped fraction and gradients."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.ops import fused_ep
    from picotron_b200.parallel import capacity_moe as cm
    from picotron_b200.parallel.expert_parallel import MoELayer

    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=1)
    for dropless in (False, True):
        cfg = moe_config(ep_capacity_factor=0.5, ep_capacity_dropless=dropless, num_shared_experts=0)
        torch.manual_seed(4)
        layer = MoELayer(cfg)
        T, k, E, d = 24, cfg.num_experts_per_tok, cfg.num_experts, cfg.hidden_size
        C = cm.compute_capacity(T, k, E, cfg.ep_capacity_factor)
        tokens = torch.randn(T, d, requires_grad=True)
        expert_idx = torch.randint(0, E, (T * k,))
        weights = torch.rand(T * k, requires_grad=True)
        token_idx = torch.arange(T).repeat_interleave(k)
        slot = cm.slot_assignment(expert_idx, E)
        rounds = int(((cm.expert_counts(expert_idx, E).max() + C - 1) // C).item()) if dropless else 1

        def fake_dispatch(tok, row_of_slot, top_k, epf, quant, *routing):  # [E*C] rows -> [L, C, d] on one rank
            valid = (row_of_slot >= 0).unsqueeze(-1)
            src = tok[(row_of_slot.clamp_min(0) // top_k).long()]
            return torch.where(valid, src, torch.zeros_like(src)).view(E, C, d)

        monkeypatch.setattr(fused_ep, "dispatch", fake_dispatch)
        monkeypatch.setattr(fused_ep, "combine", lambda out, epf: out.reshape(E * C, d))
        epf = types.SimpleNamespace(C=C, d=d)
        y1, drop1 = cm._capacity_moe_fused(layer, epf, tokens, expert_idx, weights, token_idx, T, slot, rounds)
        g1 = torch.autograd.grad(y1.square().sum(), [tokens, weights])
        y2, drop2 = cm.capacity_moe(layer, tokens[token_idx], expert_idx, weights, token_idx, T, C, dropless,
                                    cfg.ep_max_rounds)
        g2 = torch.autograd.grad(y2.square().sum(), [tokens, weights])
        assert torch.allclose(y1, y2, atol=1e-5), (y1 - y2).abs().max()
        assert abs(float(drop1) - float(drop2)) < 1e-6
        for a, b in zip(g1, g2):
            assert torch.allclose(a, b, atol=1e-4), (a - b).abs().max()
