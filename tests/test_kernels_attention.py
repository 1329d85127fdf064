"""tcgen05 flash attention against the fp32 torch restatement (``ops.attention.attention_block``):
causal and full, grouped-query heads, ragged sequence lengths, strided q/k/v views of a fused
projection, and the position-offset form that ring attention uses."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _run_fwd(q, k, v, causal, q_pos0=0, k_pos0=0):
    from picotron_b200 import ops
    b, sq, H, d = q.shape
    out = torch.empty((b, sq, H, d), device=q.device, dtype=q.dtype)
    lse = torch.empty((b, H, sq), device=q.device, dtype=torch.float32)
    ops.ext().attention_fwd(q, k, v, out, lse, d ** -0.5, causal, q_pos0, k_pos0, None)
    ops.check_status("attention fwd")
    return out, lse


CASES = [  # b, sq, sk, H, Hkv, d, causal
    (2, 128, 128, 4, 4, 64, True), (1, 256, 256, 4, 2, 64, True), (2, 384, 384, 8, 8, 64, False),
    (1, 200, 200, 4, 4, 64, True), (1, 1000, 1000, 2, 1, 64, True), (1, 256, 256, 2, 2, 128, True),
    (2, 130, 130, 4, 2, 128, False), (1, 2048, 2048, 4, 4, 64, True),
]


@pytest.mark.parametrize("b,sq,sk,H,Hkv,d,causal", CASES)
def test_attention_fwd(b, sq, sk, H, Hkv, d, causal):
    from picotron_b200.ops import attention as A
    torch.manual_seed(0)
    q = torch.randn(b, sq, H, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, sk, Hkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, sk, Hkv, d, device="cuda", dtype=torch.bfloat16)
    out, lse = _run_fwd(q, k, v, causal)
    ref, ref_lse = A.attention_block(q.float(), k.float(), v.float(), causal)
    assert _rel(out, ref) < 1e-2
    assert torch.allclose(lse, ref_lse, atol=2e-2, rtol=1e-3)


def test_attention_fwd_strided_views_of_fused_qkv():
    from picotron_b200.ops import attention as A
    torch.manual_seed(1)
    b, s, H, Hkv, d = 2, 256, 8, 4, 64
    qkv = torch.randn(b, s, (H + 2 * Hkv) * d, device="cuda", dtype=torch.bfloat16)
    q = qkv[..., :H * d].view(b, s, H, d)
    k = qkv[..., H * d:(H + Hkv) * d].view(b, s, Hkv, d)
    v = qkv[..., (H + Hkv) * d:].view(b, s, Hkv, d)
    out, _ = _run_fwd(q, k, v, True)
    ref, _ = A.attention_block(q.float(), k.float(), v.float(), True)
    assert _rel(out, ref) < 1e-2


@pytest.mark.parametrize("q_pos0,k_pos0", [(256, 0), (256, 256), (0, 256), (128, 256)])
def test_attention_fwd_block_offsets(q_pos0, k_pos0):
    """A ring-attention step: queries at global positions q_pos0.., keys at k_pos0..; rows that see
    no key return 0 with lse = -inf."""
    from picotron_b200.ops import attention as A
    torch.manual_seed(2)
    b, s, H, d = 1, 256, 2, 64
    q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    out, lse = _run_fwd(q, k, v, True, q_pos0, k_pos0)
    ref, ref_lse = A.attention_block(q.float(), k.float(), v.float(), True, None, q_offset=q_pos0, k_offset=k_pos0)
    dead = torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(lse), dead)
    assert _rel(out, ref) < 1e-2 if ref.abs().sum() > 0 else out.abs().sum() == 0
    assert torch.allclose(lse[~dead], ref_lse[~dead], atol=2e-2, rtol=1e-3)


BWD_CASES = [  # b, s, H, Hkv, d, causal
    (2, 128, 2, 2, 64, True), (1, 256, 4, 2, 64, True), (1, 384, 4, 4, 64, False), (1, 200, 2, 1, 64, True),
    (1, 256, 2, 2, 128, True), (1, 300, 4, 2, 128, False), (1, 1024, 4, 4, 64, True),
]


@pytest.mark.parametrize("b,s,H,Hkv,d,causal", BWD_CASES)
def test_attention_autograd(b, s, H, Hkv, d, causal):
    from picotron_b200 import ops
    from picotron_b200.ops import attention as A
    torch.manual_seed(3)
    q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    out = A.attention(q, k, v, causal)
    out.backward(go)
    ops.check_status("attention bwd")
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, causal)
    ref.backward(go.float())
    assert _rel(out, ref) < 1e-2
    assert _rel(q.grad, qr.grad) < 2e-2
    assert _rel(k.grad, kr.grad) < 2e-2
    assert _rel(v.grad, vr.grad) < 2e-2


def test_attention_backward_block_offsets():
    """Backward of one ring step given the merged out / lse of the whole row."""
    from picotron_b200.ops import attention as A
    torch.manual_seed(4)
    b, s, H, d = 1, 256, 2, 64
    q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, 2 * s, H, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, 2 * s, H, d, device="cuda", dtype=torch.bfloat16)
    go = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    # queries are the second half of a 2*s sequence; full causal attention over both key blocks
    out, lse = A.attention_block(q.float(), k.float(), v.float(), True, None, q_offset=s, k_offset=0)
    out = out.to(torch.bfloat16)
    for blk in range(2):
        kb, vb = k[:, blk * s:(blk + 1) * s].contiguous(), v[:, blk * s:(blk + 1) * s].contiguous()
        dq, dk, dv = A.flash_attention_backward(go, q, kb, vb, out, lse, True, None, q_pos0=s, k_pos0=blk * s)
        rq, rk, rv = A.attention_block_backward(go, q, kb, vb, out, lse, True, None, q_offset=s, k_offset=blk * s)
        assert _rel(dq, rq) < 2e-2 and _rel(dk, rk) < 2e-2 and _rel(dv, rv) < 2e-2


@pytest.mark.parametrize("acc_dtype", [torch.float32, torch.bfloat16])
def test_merge_kernel_matches_eager_merge(acc_dtype):
    """Online-softmax merge of two partial results: the kernel against the eager formula, including
    rows that have seen no key on one side or on both (lse = -inf)."""
    from picotron_b200 import ops
    from picotron_b200.ops import attention as A
    torch.manual_seed(0)
    b, s, H, d = 2, 300, 6, 64
    out_a = torch.randn(b, s, H, d, device="cuda").to(acc_dtype)
    out_b = torch.randn(b, s, H, d, device="cuda").to(torch.bfloat16)
    lse_a = torch.randn(b, H, s, device="cuda") * 3
    lse_b = torch.randn(b, H, s, device="cuda") * 3
    lse_a[0, 0, :10] = float("-inf")
    lse_b[0, 1, :10] = float("-inf")
    lse_a[1, 2, 5:9] = float("-inf")
    lse_b[1, 2, 5:9] = float("-inf")
    with torch.enable_grad():       # the eager formula is what runs when gradients are recorded
        want_out, want_lse = A.merge_attention_blocks(out_a.clone().requires_grad_(True), lse_a, out_b, lse_b)
    with torch.no_grad():
        got_out, got_lse = A.merge_attention_blocks(out_a.clone(), lse_a.clone(), out_b, lse_b)
    ops.check_status("attn merge")
    assert got_out.dtype == torch.float32
    assert torch.equal(torch.isinf(got_lse), torch.isinf(want_lse))
    fin = ~torch.isinf(want_lse)
    assert torch.allclose(got_lse[fin], want_lse[fin], atol=1e-5, rtol=1e-5)
    assert torch.allclose(got_out, want_out.detach(), atol=2e-3, rtol=1e-3)
    assert got_out[1, 5:9, 2].abs().max().item() == 0.0        # no key on either side: stays zero


def _close(a, b, atol, rtol):
    """Per-element check next to the norm ratio: |a - b| <= atol + rtol * |b| everywhere."""
    return bool(((a.float() - b.float()).abs() <= atol + rtol * b.float().abs()).all())


def test_attention_head_dim_128_at_2048_tokens():
    """head_dim 128 at a training-size sequence (forward and backward), norm ratio and per-element bounds."""
    from picotron_b200 import ops
    from picotron_b200.ops import attention as A
    torch.manual_seed(11)
    b, s, H, Hkv, d = 1, 2048, 4, 2, 128
    q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    out = A.attention(q, k, v, True)
    out.backward(go)
    ops.check_status("attention d128 s2048")
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, True)
    ref.backward(go.float())
    assert _rel(out, ref) < 1e-2 and _close(out, ref, atol=2e-2, rtol=2e-2)
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _rel(got, want) < 2e-2
        assert _close(got, want, atol=0.05 * want.abs().max().item(), rtol=5e-2)


def test_attention_long_context_shape_against_library_attention():
    """The long-context benchmark's per-rank shape (16384 tokens, 32 query / 8 KV heads, head_dim 64,
    causal). The fp32 restatement would need a 16384 x 16384 score matrix per head, so the oracle here
    is PyTorch's library attention on the same bf16 inputs (K/V heads repeated for it); forward and
    backward."""
    import torch.nn.functional as F
    from picotron_b200 import ops
    from picotron_b200.ops import attention as A
    torch.manual_seed(12)
    b, s, H, Hkv, d = 1, 16384, 32, 8, 64
    q = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, s, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(b, s, H, d, device="cuda", dtype=torch.bfloat16)
    out = A.attention(q, k, v, True)
    out.backward(go)
    ops.check_status("attention long context")
    qr, kr, vr = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    rep = H // Hkv
    ref = F.scaled_dot_product_attention(qr.transpose(1, 2), kr.repeat_interleave(rep, dim=2).transpose(1, 2),
                                         vr.repeat_interleave(rep, dim=2).transpose(1, 2), is_causal=True)
    ref = ref.transpose(1, 2)
    ref.backward(go)
    assert _rel(out, ref) < 2e-2
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _rel(got, want) < 3e-2
