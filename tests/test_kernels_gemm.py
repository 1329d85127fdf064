"""tcgen05 GEMM against an fp32 torch reference: all operand layouts, output modes, ragged
shapes (M, N, K not multiples of the tile) and strided views."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from picotron_b200 import ops
    from picotron_b200.ops import gemm
    return ops, gemm


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


SHAPES = [(128, 256, 64), (256, 512, 128), (1024, 2048, 512), (200, 264, 72), (8, 64, 2048),
          (4096, 1536, 2048), (136, 136, 200), (384, 128, 4096), (64, 8192, 256)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nt(M, N, K):
    ops, gemm = _ops()
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = gemm.gemm_nt(a, b)
    ref = a.float() @ b.float().t()
    ops.check_status()
    assert _rel_err(out, ref) < 1e-2
    out32 = gemm.gemm_nt(a, b, out_dtype=torch.float32)
    ops.check_status()
    assert _rel_err(out32, ref) < 1e-5


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nn(M, N, K):
    ops, gemm = _ops()
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    out = gemm.gemm_nn(a, b)
    ops.check_status()
    assert _rel_err(out, a.float() @ b.float()) < 1e-2


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tn_and_accumulate(M, N, K):
    ops, gemm = _ops()
    torch.manual_seed(2)
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float().t() @ b.float()
    out = gemm.gemm_tn(a, b)
    ops.check_status()
    assert _rel_err(out, ref) < 1e-2
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    base = acc.clone()
    gemm.gemm_tn(a, b, out=acc, accumulate=True)
    gemm.gemm_tn(a, b, out=acc, accumulate=True)
    ops.check_status()
    assert _rel_err(acc, base + 2 * ref) < 1e-5


def test_gemm_strided_views():
    ops, gemm = _ops()
    torch.manual_seed(3)
    big = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    a = big[:, 256:768]                      # row stride 1024, K = 512
    w = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    outbuf = torch.zeros(512, 1024, device="cuda", dtype=torch.bfloat16)
    out = outbuf[:, 128:512]
    gemm.gemm_nt(a, w, out=out)
    ops.check_status()
    assert _rel_err(out, a.float() @ w.float().t()) < 1e-2
    assert outbuf[:, :128].abs().sum().item() == 0 and outbuf[:, 512:].abs().sum().item() == 0


def test_linear_autograd_matches_torch():
    ops, gemm = _ops()
    torch.manual_seed(4)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gemm.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    ops.check_status()
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


def test_linear_main_grad_accumulation():
    ops, gemm = _ops()
    torch.manual_seed(5)
    x = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(64, 128, device="cuda", dtype=torch.bfloat16))
    w.main_grad = torch.zeros(64, 128, device="cuda", dtype=torch.float32)
    for _ in range(3):
        gemm.linear(x, w).sum().backward()
    ops.check_status()
    assert w.grad is None
    ref = 3 * torch.ones(256, 64, device="cuda").t() @ x.detach().float()
    assert _rel_err(w.main_grad, ref) < 1e-5


# ---------------------------------------------------------------------------------------------
# grouped GEMM over the local experts of a mixture-of-experts layer
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("counts,d_in,d_out", [([128, 256, 128], 128, 256), ([5, 0, 300, 129], 256, 384),
                                                ([1000, 17, 64, 512, 3, 250, 0, 77], 512, 1024)])
def test_grouped_gemm_forward_dgrad_wgrad(counts, d_in, d_out):
    ops, _ = _ops()
    from picotron_b200.ops import grouped_gemm as gg
    torch.manual_seed(3)
    G = len(counts)
    n = sum(counts)
    layout = gg.GroupLayout.from_counts(counts, "cuda")
    assert layout.rows % 128 == 0 and layout.tile_group.numel() == max(layout.rows // 128, 1)
    x = torch.randn(n, d_in, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(G * d_out, d_in, device="cuda", dtype=torch.bfloat16) * 0.1
    xp = layout.pad(x)
    # forward
    y = layout.unpad(gg.grouped_gemm_nt(xp, w, layout, d_out))
    ops.check_status()
    ref, off = [], 0
    for e, c in enumerate(counts):
        ref.append(x[off:off + c].float() @ w[e * d_out:(e + 1) * d_out].float().t())
        off += c
    ref = torch.cat(ref)
    assert _rel_err(y, ref) < 1e-2
    # input gradient
    dy = torch.randn(n, d_out, device="cuda", dtype=torch.bfloat16)
    dyp = layout.pad(dy)
    dx = layout.unpad(gg.grouped_gemm_nn(dyp, w, layout, d_out))
    ops.check_status()
    ref, off = [], 0
    for e, c in enumerate(counts):
        ref.append(dy[off:off + c].float() @ w[e * d_out:(e + 1) * d_out].float())
        off += c
    assert _rel_err(dx, torch.cat(ref)) < 1e-2
    # weight gradient, accumulated into fp32; experts without rows keep their old values
    acc = torch.randn(G * d_out, d_in, device="cuda", dtype=torch.float32)
    base = acc.clone()
    gg.grouped_gemm_tn(dyp, xp, layout, acc, accumulate=True)
    ops.check_status()
    off = 0
    for e, c in enumerate(counts):
        want = base[e * d_out:(e + 1) * d_out] + dy[off:off + c].float().t() @ x[off:off + c].float()
        got = acc[e * d_out:(e + 1) * d_out]
        assert _rel_err(got, want) < 1e-4, (e, c)
        off += c


def test_moe_layer_grouped_experts_match_per_expert_loop():
    """The MoE layer on the grouped-GEMM path (stacked expert weights in a ParamStore, gradients
    accumulated into main_grad) against the same layer run expert by expert in plain PyTorch."""
    import copy
    import types
    ops, _ = _ops()
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.param_store import ParamStore
    from picotron_b200.parallel.expert_parallel import MoELayer
    pgm.process_group_manager = None
    cfg = types.SimpleNamespace(hidden_size=256, intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                                init_std=0.05, num_shared_experts=1)
    torch.manual_seed(0)
    layer = MoELayer(cfg, ep_group=False).to("cuda", torch.bfloat16)
    ref = copy.deepcopy(layer)
    store = ParamStore(layer)
    assert any(len(g.mods) == 16 for g in store.fused_groups) and any(len(g.mods) == 8 for g in store.fused_groups)
    x = torch.randn(2, 192, 256, device="cuda", dtype=torch.bfloat16)
    xr = x.clone().requires_grad_(True)
    x.requires_grad_(True)
    before = ops.launches()
    y = layer(x)
    y.float().square().mean().backward()
    ops.check_status()
    assert ops.launches() - before > 0
    import os
    os.environ["PICO_REFERENCE_OPS"] = "1"
    try:
        yr = ref(xr)
        yr.float().square().mean().backward()
    finally:
        os.environ["PICO_REFERENCE_OPS"] = "0"
    assert _rel_err(y, yr) < 2e-2
    assert _rel_err(x.grad, xr.grad) < 3e-2
    for (n, p), (_, q) in zip(layer.named_parameters(), ref.named_parameters()):
        g = p.main_grad if getattr(p, "main_grad", None) is not None and p.grad is None else p.grad
        assert _rel_err(g, q.grad) < 5e-2, n


@pytest.mark.parametrize("my_rank", [0, 1, 3])
def test_dropless_ep_layout_kernel_matches_reference(my_rank):
    """The device-side layout of the dropless expert-parallel exchange (offsets of outgoing blocks,
    padded expert segments, tile -> expert array, return blocks) against its Python restatement, with
    empty experts, experts that are exact multiples of the tile, and a table that does not fit."""
    ops, _ = _ops()
    from picotron_b200.ops.fused_ep_var import var_layout_ref
    ep, L = 4, 3
    E = ep * L
    g = torch.Generator().manual_seed(7)
    table = torch.randint(0, 300, (ep, E), generator=g, dtype=torch.int32)
    table[:, 2] = 0                  # an expert nobody routes to
    table[:, 5] = 32                 # 4 x 32 = exactly one tile
    for max_rows in (128 * 40, 128 * 6):      # roomy, and too small for some experts
        dev = table.cuda()
        send = torch.empty((E, 4), device="cuda", dtype=torch.int32)
        ret = torch.empty((ep * L, 4), device="cuda", dtype=torch.int32)
        seg_start = torch.empty(L + 1, device="cuda", dtype=torch.int32)
        seg_len = torch.empty(L, device="cuda", dtype=torch.int32)
        tiles = torch.empty(max_rows // 128, device="cuda", dtype=torch.int32)
        ops.ext().ep_var_layout(dev, ep, L, my_rank, max_rows, send, ret, seg_start, seg_len, tiles)
        r_send, r_ret, r_seg, r_len, r_tiles = var_layout_ref(table.tolist(), L, my_rank, max_rows)
        assert send.cpu().tolist() == r_send
        got_ret, want_ret = ret.cpu().tolist(), r_ret
        for a, b in zip(got_ret, want_ret):
            assert a[0] == b[0] and a[2:] == b[2:] and (a[0] == 0 or a[1] == b[1]), (a, b)
        assert seg_start.cpu().tolist() == r_seg and seg_len.cpu().tolist() == r_len
        assert tiles.cpu().tolist() == r_tiles
        words = ops.ext().status_fetch()       # the small table reports the rows it could not place
        assert (words[0] != 0) == (max_rows == 128 * 6)
