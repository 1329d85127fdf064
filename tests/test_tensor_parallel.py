"""Tensor parallelism on CPU/gloo against the single-process model: every TP mode (plain,
async, sequence parallel, vocabulary-parallel CE, chunked overlap, parallel block) must give
the single-process loss and gradients (sliced the same way as the weights) within 2e-4 in fp32
— the tolerance of the reference's tests/test_tp_sequence_parallel.py:183."""
import types

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def tiny_config(**kw):
    cfg = dict(hidden_size=64, num_attention_heads=8, num_key_value_heads=4, intermediate_size=176,
               vocab_size=128, num_hidden_layers=2, max_position_embeddings=32, rms_norm_eps=1e-5,
               rope_theta=10000.0, parallel_block=False)
    cfg.update(kw)
    return types.SimpleNamespace(**cfg)


def shard_like(full: torch.Tensor, local_shape, rank: int, world: int) -> torch.Tensor:
    """Slice ``full`` along the (single) dimension in which the local tensor is smaller."""
    if tuple(full.shape) == tuple(local_shape):
        return full
    for d, (f, l) in enumerate(zip(full.shape, local_shape)):
        if f != l:
            assert f == l * world
            return full.narrow(d, rank * l, l)
    raise AssertionError


def _tp_worker(rank, world, mode, parallel_block):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.engine import loss_fn
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel

    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    cfg = tiny_config(parallel_block=parallel_block)
    torch.manual_seed(7)
    ref = Llama(cfg)
    ref_sd = {k: v.clone() for k, v in ref.state_dict().items()}
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
    ref_loss = torch.nn.functional.cross_entropy(ref(ids).view(-1, cfg.vocab_size), tgt.view(-1))
    ref_loss.backward()
    ref_grads = {n: p.grad.clone() for n, p in ref.named_parameters()}

    flags = dict(plain={}, async_tp=dict(async_tp=True), sp=dict(sequence_parallel=True),
                 vocab_ce=dict(vocab_parallel_ce=True), sp_vocab_ce=dict(sequence_parallel=True, vocab_parallel_ce=True),
                 sp_overlap=dict(sequence_parallel=True, overlap_comm=True))[mode]
    torch.manual_seed(7)
    model = Llama(cfg)
    apply_tensor_parallel(model, **flags)
    sd = model.state_dict()
    model.load_state_dict({k: shard_like(ref_sd[k], v.shape, rank, world).clone() for k, v in sd.items()})
    logits = model(ids)
    loss = loss_fn(model, logits, tgt)
    loss.backward()
    if flags.get("sequence_parallel"):
        for p in model.parameters():
            if getattr(p, "sequence_parallel_grad", False):
                dist.all_reduce(p.grad, group=pgm.get_pgm().tp_group)
    assert abs(loss.item() - ref_loss.item()) < 2e-4, (mode, loss.item(), ref_loss.item())
    for n, p in model.named_parameters():
        want = shard_like(ref_grads[n], p.shape, rank, world)
        err = (p.grad - want).abs().max().item()
        assert err < 2e-4, (mode, n, err)


@pytest.mark.parametrize("mode", ["plain", "async_tp", "sp", "vocab_ce", "sp_vocab_ce", "sp_overlap"])
def test_tp2_matches_single_process(mode):
    run_distributed(_tp_worker, 2, mode, False)


@pytest.mark.parametrize("mode", ["plain", "sp", "sp_overlap", "sp_vocab_ce"])
def test_tp2_parallel_block(mode):
    run_distributed(_tp_worker, 2, mode, True)


def test_tp4_sequence_parallel():
    run_distributed(_tp_worker, 4, "sp_vocab_ce", False)


def _collective_count_worker(rank, world):
    """Sequence-parallel collectives per forward + backward pass, counted at the two helpers every
    gather / reduce-scatter along the sequence goes through: the sequential block needs two gathers and
    two reduce-scatters per layer and direction, the parallel block one of each
    (the counting idea of the reference's tests/test_ptb_overlap.py:71-91)."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.engine import loss_fn
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel import sequence_parallel as sp
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel

    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    counts = {"gather": 0, "scatter": 0}
    gather, scatter = sp.all_gather_along_seq, sp.reduce_scatter_along_seq

    def counted_gather(x, group=None):
        counts["gather"] += 1
        return gather(x, group)

    def counted_scatter(x, group=None):
        counts["scatter"] += 1
        return scatter(x, group)

    sp.all_gather_along_seq, sp.reduce_scatter_along_seq = counted_gather, counted_scatter
    seen = {}
    for parallel_block in (False, True):
        cfg = tiny_config(parallel_block=parallel_block, num_hidden_layers=3)
        torch.manual_seed(7)
        model = Llama(cfg)
        apply_tensor_parallel(model, sequence_parallel=True, vocab_parallel_ce=True)
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        tgt = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        counts["gather"] = counts["scatter"] = 0
        loss_fn(model, model(ids), tgt).backward()
        seen[parallel_block] = dict(counts)
    layers = 3
    # per layer, forward + backward. Sequential block: 2 gathers + 2 reduce-scatters forward; backward, each of
    # the two column-parallel groups re-gathers its input and reduce-scatters dx, each row-parallel linear
    # gathers dy: 6 gathers + 4 reduce-scatters. Parallel block: one gather and one reduce-scatter forward and
    # their mirror images backward: 2 + 2.
    assert seen[False]["gather"] - seen[True]["gather"] == 4 * layers, seen
    assert seen[False]["scatter"] - seen[True]["scatter"] == 2 * layers, seen
    outside = (seen[True]["gather"] - 2 * layers, seen[True]["scatter"] - 2 * layers)     # embedding and lm-head
    assert (seen[False]["gather"], seen[False]["scatter"]) == (6 * layers + outside[0], 4 * layers + outside[1]), seen
    assert 0 <= outside[0] <= 4 and 0 <= outside[1] <= 4, seen


def test_parallel_block_needs_fewer_sequence_parallel_collectives():
    run_distributed(_collective_count_worker, 2)


def _vocab_ce_worker(rank, world):
    """Vocabulary-parallel cross entropy on logit shards against the dense loss on the full logits
    (the reference's tests/test_tp_vocab_ce.py: loss within 1e-5, gradient within 1e-6), including
    targets that all live on one rank's shard and a vocabulary that a shard splits unevenly in value."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.tp_communications import vocab_parallel_cross_entropy

    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    V, N = 32 * world, 24
    for case in ("spread", "one_shard", "large_logits"):
        g = torch.Generator().manual_seed(11)
        full = torch.randn(2, N // 2, V, generator=g, dtype=torch.float64) * (30.0 if case == "large_logits" else 1.0)
        tgt = torch.randint(0, V if case != "one_shard" else V // world, (2, N // 2), generator=g)
        ref_in = full.clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(ref_in.view(-1, V), tgt.view(-1), reduction="none").view(tgt.shape)
        ref.mean().backward()
        v_loc = V // world
        shard = full[..., rank * v_loc:(rank + 1) * v_loc].clone().requires_grad_(True)
        loss = vocab_parallel_cross_entropy(shard, tgt)
        assert loss.shape == tgt.shape
        assert (loss - ref).abs().max().item() < 1e-5, case
        loss.mean().backward()
        want = ref_in.grad[..., rank * v_loc:(rank + 1) * v_loc]
        assert (shard.grad - want).abs().max().item() < 1e-6, case


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_cross_entropy_matches_dense_loss(world):
    run_distributed(_vocab_ce_worker, world)
