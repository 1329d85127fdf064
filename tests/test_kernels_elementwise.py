"""Memory-bound kernels against fp32 torch restatements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("rows,H", [(64, 256), (1000, 2048), (33, 4096), (7, 8192), (5, 520)])
def test_rmsnorm_fwd_bwd(rows, H):
    from picotron_b200 import ops
    from picotron_b200.ops import norm
    torch.manual_seed(0)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y = norm.rmsnorm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = norm.rmsnorm_ref(xr, wr, 1e-5)
    yr.backward(g.float())
    ops.check_status()
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 2e-2


def test_add_rmsnorm_and_main_grad():
    from picotron_b200.ops import norm
    torch.manual_seed(1)
    rows, H = 300, 2048
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter((1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16))
    w.main_grad = torch.zeros(H, device="cuda", dtype=torch.float32)
    y, h = norm.add_rmsnorm(x, r, w, 1e-5)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [gy, gh])
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    # the kernel rounds the summed stream to bf16 before normalising (straight-through here)
    hr = (xr + rr) + ((xr + rr).to(torch.bfloat16).float() - (xr + rr)).detach()
    yr = norm.rmsnorm_ref(hr, wr, 1e-5)
    torch.autograd.backward([yr, hr], [gy.float(), gh.float()])
    assert _rel(y, yr) < 1e-2 and _rel(h, hr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(r.grad, rr.grad) < 1e-2
    assert w.grad is None and _rel(w.main_grad, wr.grad) < 2e-2


@pytest.mark.parametrize("d", [64, 128])
def test_rope(d):
    from picotron_b200.ops import rope
    torch.manual_seed(2)
    b, s, nh = 2, 48, 6
    cos, sin = rope.get_cos_sin(128, d, base=10000.0, device="cuda")
    x = torch.randn(b, s, nh, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = rope.apply_rope(x, cos, sin, pos_offset=16)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    yr = rope.apply_rope_ref(xr, cos, sin, pos_offset=16)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2


def test_swiglu():
    from picotron_b200.ops import swiglu
    torch.manual_seed(3)
    gu = torch.randn(5, 37, 2 * 688, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = swiglu.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_(True)
    yr = swiglu.swiglu_ref(gr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(gu.grad, gr.grad) < 1e-2


def test_swiglu_with_device_side_row_count():
    """Rows at or past a fill level that lives on the device are skipped, forward and backward."""
    from picotron_b200.ops import swiglu
    torch.manual_seed(5)
    gu = torch.randn(300, 2 * 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    n = torch.tensor([129], device="cuda", dtype=torch.int32)
    y = swiglu.swiglu(gu, rows_in_use=n)
    g = torch.randn_like(y)
    y[:129].backward(g[:129])
    gr = gu.detach().float().requires_grad_(True)
    yr = swiglu.swiglu_ref(gr)
    yr[:129].backward(g[:129].float())
    assert _rel(y[:129], yr[:129]) < 1e-2 and _rel(gu.grad[:129], gr.grad[:129]) < 1e-2


@pytest.mark.parametrize("rows,V", [(64, 4096), (300, 49152), (17, 32000)])
def test_cross_entropy(rows, V):
    from picotron_b200.ops import cross_entropy as ce
    torch.manual_seed(4)
    logits = (3 * torch.randn(rows, V, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    t = torch.randint(0, V, (rows,), device="cuda")
    lr = logits.detach().float().requires_grad_(True)
    loss_r = ce.cross_entropy_ref(lr, t)
    loss_r.mean().backward()
    loss = ce.cross_entropy(logits * 1.0, t, inplace=True)
    loss.mean().backward()
    assert torch.allclose(loss, loss_r, atol=2e-3, rtol=2e-3)
    assert _rel(logits.grad, lr.grad) < 2e-2


def test_cross_entropy_vocab_shards_combine():
    """Two column shards evaluated separately and merged by hand equal the dense loss."""
    from picotron_b200 import ops
    torch.manual_seed(5)
    rows, V = 50, 1024
    logits = (2 * torch.randn(rows, V, device="cuda")).to(torch.bfloat16)
    t = torch.randint(0, V, (rows,), device="cuda")
    e = ops.ext()
    stats = []
    for r in range(2):
        sh = logits[:, r * 512:(r + 1) * 512].contiguous()
        st = torch.empty(rows, 3, device="cuda")
        e.ce_stats(sh, 512, t, st, rows, 512, r * 512)
        stats.append(st)
    g = torch.stack(stats)
    m = g[..., 0].max(0).values
    s = (g[..., 1] * torch.exp(g[..., 0] - m)).sum(0)
    tl = g[..., 2].sum(0)
    loss = s.log() + m - tl
    ref = torch.nn.functional.cross_entropy(logits.float(), t, reduction="none")
    assert torch.allclose(loss, ref, atol=2e-3, rtol=2e-3)


def test_adamw_matches_torch():
    from picotron_b200.ops.adamw import FlatAdamW
    torch.manual_seed(6)
    n = 100_003
    p = torch.randn(n, device="cuda").to(torch.bfloat16)
    g = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.float().clone())
    opt_ref = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = FlatAdamW(p, g.clone(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, master_weights=True)
    for i in range(3):
        opt.grads.copy_(g * (i + 1))
        ref_p.grad = (g * (i + 1)) * 0.5
        opt.step(grad_scale=0.5, zero_grad=True)
        opt_ref.step()
    assert opt.grads.abs().sum().item() == 0
    assert torch.allclose(opt.master, ref_p.detach(), atol=1e-5, rtol=1e-5)
    assert _rel(p, ref_p.detach()) < 1e-2


def test_embedding():
    from picotron_b200.ops import embedding as emb
    torch.manual_seed(7)
    V, H = 1000, 256
    w = torch.nn.Parameter(torch.randn(V, H, device="cuda", dtype=torch.bfloat16))
    ids = torch.randint(0, 2 * V, (4, 33), device="cuda")
    out = emb.embedding(ids, w, vocab_start=500)
    ref = emb.embedding_ref(ids, w.detach().float(), vocab_start=500)
    assert _rel(out, ref) < 1e-3
    g = torch.randn_like(out)
    out.backward(g)
    wr = w.detach().float().requires_grad_(True)
    emb.embedding_ref(ids, wr, vocab_start=500).backward(g.float())
    assert _rel(w.grad, wr.grad) < 1e-2
