"""The allocation-free RMSNorm backward, called through its exported C symbol.

Callers that cannot allocate device memory when they launch work (a host that gave the whole
device to its own arena, code holding the allocator lock, paths where cudaMalloc's implicit
synchronisation is unacceptable) use ``pico_rmsnorm_bwd_noalloc``, whose weight-gradient
scratch is a fixed array inside the library. This test drives that symbol with raw pointers,
twice in a row with different data (the second call reuses the scratch the first one dirtied),
and checks each result against the regular entry point ``pico_rmsnorm_bwd`` that takes
caller-provided scratch. It also checks that an oversized hidden dimension is refused.

Collected last on purpose: a failure here cannot mask any other test in a ``-x`` run.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "picotron_b200", "_C.so")


def _lib():
    lib = ctypes.CDLL(SO)
    vp, i, fp = ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p
    lib.pico_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, fp, vp, vp, fp, vp, i, i, i, vp]
    lib.pico_rmsnorm_bwd_noalloc.restype = i
    lib.pico_rmsnorm_bwd.argtypes = [vp, vp, vp, fp, vp, vp, fp, fp, vp, i, i, i, vp]
    lib.pico_rmsnorm_bwd.restype = i
    lib.pico_rmsnorm_bwd_num_partials.restype = i
    lib.pico_last_error.restype = ctypes.c_char_p
    return lib


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _case(lib, rows, H, seed, with_residual_grad):
    torch.manual_seed(seed)
    dev = "cuda"
    h = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device=dev)).to(torch.bfloat16)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5).contiguous()
    dres = torch.randn(rows, H, device=dev, dtype=torch.bfloat16) if with_residual_grad else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dres_p = ctypes.c_void_p(dres.data_ptr()) if dres is not None else None

    dh_new = torch.empty_like(h)
    dw_new = torch.full((H,), 7.0, device=dev, dtype=torch.float32)  # must be overwritten, not added to
    rc = lib.pico_rmsnorm_bwd_noalloc(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres_p,
                                      dh_new.data_ptr(), dw_new.data_ptr(), None, 0, rows, H, stream)
    assert rc == 0, lib.pico_last_error()

    dh_old = torch.empty_like(h)
    dw_old = torch.empty(H, device=dev, dtype=torch.float32)
    scratch = torch.empty(lib.pico_rmsnorm_bwd_num_partials() * H, device=dev, dtype=torch.float32)
    rc = lib.pico_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres_p,
                              dh_old.data_ptr(), scratch.data_ptr(), dw_old.data_ptr(), None, 0, rows, H, stream)
    assert rc == 0, lib.pico_last_error()
    torch.cuda.synchronize()
    assert _rel(dh_new, dh_old) < 1e-2
    assert _rel(dw_new, dw_old) < 2e-2
    # and both agree with the fp32 restatement of the op
    g = dy.float() * w.float()
    c = (g * h.float()).mean(-1, keepdim=True) * rstd[:, None] ** 3
    dh_ref = rstd[:, None] * g - h.float() * c + (dres.float() if dres is not None else 0)
    dw_ref = (dy.float() * h.float() * rstd[:, None]).sum(0)
    assert _rel(dh_new, dh_ref) < 1e-2
    assert _rel(dw_new, dw_ref) < 2e-2


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    _case(lib, rows=777, H=2048, seed=0, with_residual_grad=True)
    # second call right after the first: different shape and data, same built-in scratch
    _case(lib, rows=300, H=4096, seed=1, with_residual_grad=False)


def test_noalloc_rejects_oversized_hidden():
    lib = _lib()
    H = 16384
    t = torch.zeros(8, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(8, device="cuda", dtype=torch.float32)
    dw = torch.zeros(H, device="cuda", dtype=torch.float32)
    rc = lib.pico_rmsnorm_bwd_noalloc(t.data_ptr(), t.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                      t.data_ptr(), dw.data_ptr(), None, 0, 8, H,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    assert b"exceeds" in lib.pico_last_error()
