"""Ring and Ulysses context parallelism on CPU/gloo against single-process full-sequence
attention and a full-sequence model (the oracle of the reference's tests/test_cp_ulysses.py and
tests/test_cp_ring_flash.py, here in fp32 with tolerance 2e-4)."""
import types

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def _attn_worker(rank, world, kind, causal, kv_heads):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.ops import attention as A
    from picotron_b200.parallel.context_parallel import ring_attention_bshd
    from picotron_b200.parallel.ulysses import ulysses_attention_bshd

    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    torch.manual_seed(5)
    b, s, H, d = 2, 8 * world, 4, 16
    q = torch.randn(b, s, H, d)
    k = torch.randn(b, s, kv_heads, d)
    v = torch.randn(b, s, kv_heads, d)
    go = torch.randn(b, s, H, d)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, causal)
    ref.backward(go)
    sl = slice(rank * s // world, (rank + 1) * s // world)
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    fn = ring_attention_bshd if kind == "ring" else ulysses_attention_bshd
    out = fn(ql, kl, vl, causal)
    out.backward(go[:, sl])
    assert (out - ref[:, sl]).abs().max().item() < 2e-4
    for got, want in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
        assert (got - want[:, sl]).abs().max().item() < 2e-4, kind


@pytest.mark.parametrize("kind", ["ring", "ulysses"])
@pytest.mark.parametrize("causal", [True, False])
def test_cp2_attention(kind, causal):
    run_distributed(_attn_worker, 2, kind, causal, 2)


def test_cp4_ring_gqa():
    run_distributed(_attn_worker, 4, "ring", True, 2)


def test_cp4_ulysses_kv_heads_not_divisible():
    run_distributed(_attn_worker, 4, "ulysses", True, 2)


def _model_worker(rank, world, kind):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.context_parallel import apply_context_parallel

    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    cfg = types.SimpleNamespace(hidden_size=32, num_attention_heads=4, num_key_value_heads=2, intermediate_size=64,
                                vocab_size=64, num_hidden_layers=2, max_position_embeddings=16, rms_norm_eps=1e-5,
                                rope_theta=10000.0)
    torch.manual_seed(3)
    ref = Llama(cfg)
    g = torch.Generator().manual_seed(1)
    rows = torch.randint(0, 64, (2, 17), generator=g)
    ids, tgt = rows[:, :-1], rows[:, 1:]
    loss_ref = torch.nn.functional.cross_entropy(ref(ids).view(-1, 64), tgt.reshape(-1))
    loss_ref.backward()
    torch.manual_seed(3)
    model = Llama(cfg)
    model.load_state_dict(ref.state_dict())
    apply_context_parallel(model, attention=kind)
    sl = slice(rank * 16 // world, (rank + 1) * 16 // world)
    loss = torch.nn.functional.cross_entropy(model(ids[:, sl]).view(-1, 64), tgt[:, sl].reshape(-1))
    loss.backward()
    tot = loss.detach().clone()
    dist.all_reduce(tot)
    assert abs(tot.item() / world - loss_ref.item()) < 2e-4
    for (n, p), (_, pr) in zip(model.named_parameters(), ref.named_parameters()):
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert (gsum / world - pr.grad).abs().max().item() < 2e-4, (kind, n)


@pytest.mark.parametrize("kind", ["ring", "ulysses"])
def test_cp2_model(kind):
    run_distributed(_model_worker, 2, kind)


def _zigzag_attn_worker(rank, world, kv_heads):
    """Ring attention on zigzag shards (rank r holds chunks r and 2n-1-r) against full attention."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.ops import attention as A
    from picotron_b200.parallel.context_parallel import ring_attention_bshd, shard_pieces

    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    torch.manual_seed(6)
    b, s, H, d = 2, 8 * world, 4, 16
    q = torch.randn(b, s, H, d)
    k = torch.randn(b, s, kv_heads, d)
    v = torch.randn(b, s, kv_heads, d)
    go = torch.randn(b, s, H, d)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, True)
    ref.backward(go)
    pieces = shard_pieces(rank, world, s // world, True)
    assert [p[2] for p in pieces] == [rank * 4, (2 * world - 1 - rank) * 4]

    def mine(t):
        return torch.cat([t[:, pos:pos + n] for _, n, pos in pieces], dim=1)

    ql, kl, vl = (mine(t).clone().requires_grad_(True) for t in (q, k, v))
    out = ring_attention_bshd(ql, kl, vl, True, zigzag=True)
    out.backward(mine(go))
    assert (out - mine(ref)).abs().max().item() < 2e-4
    for got, want in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
        assert (got - mine(want)).abs().max().item() < 2e-4


@pytest.mark.parametrize("world,kv_heads", [(2, 2), (4, 4), (4, 1)])
def test_zigzag_ring_attention(world, kv_heads):
    run_distributed(_zigzag_attn_worker, world, kv_heads)


def _zigzag_engine_worker(rank, world, out_path):
    """The trainer with cp_zigzag (loader slicing, rotary positions, ring attention) reproduces the
    losses of the contiguous layout: same tokens, same model, only the assignment to ranks differs."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    losses = {}
    for zz in (False, True):
        pgm.process_group_manager = None
        cfg = {"distributed": dict(cp_size=world, cp_attention="ring", cp_zigzag=zz, use_cpu=True),
               "model": dict(name="tiny-llama-test", init_std=0.02, dtype="float32", num_hidden_layers=2),
               "training": dict(seed=0, learning_rate=1e-3, seq_length=64, micro_batch_size=2,
                                gradient_accumulation_steps=1, num_samples=256),
               "dataset": dict(name="synthetic")}
        eng = TrainEngine(cfg, device=torch.device("cpu"))
        assert eng.data_loader.cp_zigzag == zz
        losses[zz] = [eng.average_loss(eng.train_step()) for _ in range(3)]
    for a, b in zip(losses[True], losses[False]):
        assert abs(a - b) < 2e-4, losses


def test_zigzag_trainer_matches_contiguous_layout(tmp_path):
    run_distributed(_zigzag_engine_worker, 2, str(tmp_path / "x"))
