"""Routing ops of the mixture-of-experts layer (``ops.moe_route``): the PyTorch restatements against
the layer's own eager routing code on CPU, and the kernels against the restatements on the GPU
(router forward / backward, slot assignment, weighted combine forward / backward)."""
import pytest
import torch


def _routing_case(T=96, E=16, k=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g) * 2.0
    bias = torch.randn(E, generator=g) * 0.1
    return logits, bias


def test_reference_router_matches_the_layer_code():
    from picotron_b200.ops import moe_route as mr
    logits, bias = _routing_case()
    for b in (None, bias):
        for renorm in (True, False):
            probs, idx, w, counts = mr.route_ref(logits, b, 3, renorm)
            p = torch.softmax(logits, -1, dtype=torch.float32)
            sc = p + b if b is not None else p
            want_idx = torch.topk(sc, 3, dim=-1).indices
            assert torch.equal(idx, want_idx)
            ww = p.gather(-1, want_idx)
            if renorm:
                ww = ww / ww.sum(-1, keepdim=True)
            assert torch.allclose(w, ww) and torch.allclose(probs, p)
            assert counts.sum().item() == idx.numel() and torch.equal(counts, torch.bincount(idx.reshape(-1), minlength=16))


def test_reference_slots_and_combine_match_the_capacity_path():
    from picotron_b200.ops import moe_route as mr
    from picotron_b200.parallel.capacity_moe import slot_assignment
    g = torch.Generator().manual_seed(1)
    T, E, k, C, d = 64, 8, 2, 10, 16
    idx = torch.randint(0, E, (T, k), generator=g)
    pos, table = mr.slots_ref(idx, E, C)
    assert torch.equal(pos, slot_assignment(idx.reshape(-1), E))
    rows = torch.arange(T * k)
    for r in rows.tolist():
        e, ps = idx.reshape(-1)[r].item(), pos[r].item()
        if ps < C:
            assert table[e * C + ps].item() == r
    assert (table >= 0).sum().item() == (pos < C).sum().item()
    out = torch.randn(E * C, d, generator=g)
    w = torch.rand(T, k, generator=g)
    y = mr.combine_ref(out, idx, pos.view(T, k), w, C)
    want = torch.zeros(T, d)
    for t in range(T):
        for j in range(k):
            ps = pos.view(T, k)[t, j].item()
            if ps < C:
                want[t] += w[t, j] * out[idx[t, j].item() * C + ps]
    assert torch.allclose(y, want, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("E,k,renorm,use_bias", [(64, 6, True, True), (8, 2, True, False), (16, 1, False, True),
                                                (200, 8, False, False)])
def test_route_kernel_matches_reference(E, k, renorm, use_bias):
    from picotron_b200 import ops
    from picotron_b200.ops import moe_route as mr
    torch.manual_seed(E + k)
    T = 777
    # every row is a random permutation of E distinct values that bf16 represents exactly: no ties, so the
    # selection is unambiguous (which of two equal scores wins is not part of the contract)
    step = 1.0 / 32 if E > 64 else 1.0 / 8
    perm = torch.rand(T, E, device="cuda").argsort(dim=-1).float()
    logits = ((perm - E / 2) * step).to(torch.bfloat16).requires_grad_(True)
    assert torch.equal(logits.detach().float(), (perm - E / 2) * step)
    bias = (torch.randn(E, device="cuda") * 0.001) if use_bias else None
    probs, idx, w, counts = mr.route(logits, bias, k, renorm)
    ref_logits = logits.detach().float().requires_grad_(True)
    rp, ri, rw, rc = mr.route_ref(ref_logits, bias, k, renorm)
    assert idx.dtype == torch.int32 and torch.equal(idx.long(), ri), "selected experts differ"
    assert torch.allclose(probs, rp, atol=1e-6, rtol=1e-4) and torch.allclose(w, rw, atol=1e-6, rtol=1e-4)
    assert torch.equal(counts.long(), rc)
    # backward: gradient through the weights and a dense gradient w.r.t. the probabilities (aux loss)
    gw = torch.randn_like(rw)
    gp = torch.randn_like(rp) * 0.1
    ((w * gw).sum() + (probs * gp).sum()).backward()
    ((rw * gw).sum() + (rp * gp).sum()).backward()
    err = (logits.grad.float() - ref_logits.grad).abs().max().item()
    scale = ref_logits.grad.abs().max().item()
    assert err <= 1e-2 * scale + 1e-6, (err, scale)      # bf16 rounding of the returned gradient
    ops.check_status("moe route")


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,C", [(512, 8, 2, 100), (4096, 64, 6, 300), (100, 4, 1, 1000)])
def test_slots_kernel_matches_reference(T, E, k, C):
    from picotron_b200.ops import moe_route as mr
    g = torch.Generator(device="cuda").manual_seed(T)
    idx = torch.randint(0, E, (T, k), device="cuda", generator=g, dtype=torch.int32)
    pos, table = mr.slots(idx, E, C)
    rpos, rtable = mr.slots_ref(idx.long(), E, C)
    assert torch.equal(pos.long(), rpos) and torch.equal(table, rtable)


@pytest.mark.gpu
def test_combine_kernel_matches_reference():
    from picotron_b200 import ops
    from picotron_b200.ops import moe_route as mr
    torch.manual_seed(3)
    T, E, k, C, d = 600, 16, 4, 120, 256
    idx = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
    pos, table = mr.slots(idx, E, C)
    out = torch.randn(E * C, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = torch.rand(T, k, device="cuda").requires_grad_(True)
    y = mr.combine(out, idx, pos.view(T, k), w, table, C)
    ro, rw = out.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
    ry = mr.combine_ref(ro, idx.long(), pos.view(T, k).long(), rw, C)
    assert (y.float() - ry).abs().max().item() <= 2e-2 * ry.abs().max().item()
    g = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    y.backward(g)
    ry.backward(g.float())
    assert (out.grad.float() - ro.grad).abs().max().item() <= 2e-2 * ro.grad.abs().max().item() + 1e-6
    assert (w.grad - rw.grad).abs().max().item() <= 2e-2 * rw.grad.abs().max().item() + 1e-6
    assert (pos >= C).any(), "the case should contain rows over capacity"
    ops.check_status("moe combine")
