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
