"""All five pipeline schedules on CPU/gloo against full-model gradient accumulation over the
same micro-batches (the oracle of the reference's tests/test_pipeline_parallel.py:70-109,
tolerance 1e-5), plus offline checks of the schedule planner."""
import types

import pytest
import torch

from distributed_helpers import run_distributed


def tiny_config(layers=8):
    return types.SimpleNamespace(hidden_size=32, num_attention_heads=4, num_key_value_heads=2, intermediate_size=64,
                                 vocab_size=64, num_hidden_layers=layers, max_position_embeddings=16,
                                 rms_norm_eps=1e-5, rope_theta=10000.0)


class FakeDataLoader:
    """Seeded in-memory batches with the loader protocol the schedules need."""

    def __init__(self, vocab, mbs, seq, grad_acc, seed=0):
        self.micro_batch_size, self.seq_length_per_gpu, self.grad_acc_steps = mbs, seq, grad_acc
        self.seq_length = seq
        g = torch.Generator().manual_seed(seed)
        self.rows = [torch.randint(0, vocab, (mbs, seq + 1), generator=g) for _ in range(grad_acc)]
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        r = self.rows[self.i % len(self.rows)]
        self.i += 1
        return {"input_ids": r[:, :-1].contiguous(), "target_ids": r[:, 1:].contiguous(),
                "position_ids": None, "hidden_states": None}


def _pp_worker(rank, world, engine, m):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.pipeline_parallel import run_schedule, wrap_pipeline

    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=world, dp_size=1)
    cfg = tiny_config()
    torch.manual_seed(11)
    ref = Llama(cfg)
    loader = FakeDataLoader(cfg.vocab_size, 2, 8, m)
    ref_loss = 0.0
    for _ in range(m):
        b = next(loader)
        loss = torch.nn.functional.cross_entropy(ref(b["input_ids"]).view(-1, cfg.vocab_size),
                                                 b["target_ids"].view(-1)) / m
        loss.backward()
        ref_loss += loss.item()
    ref_grads = {n: p.grad.clone() for n, p in ref.named_parameters()}

    torch.manual_seed(11)
    full = Llama(cfg)
    full.load_state_dict(ref.state_dict())
    stage = wrap_pipeline(full, cfg, engine, 2)
    loader = FakeDataLoader(cfg.vocab_size, 2, 8, m)
    loss = run_schedule(engine, stage, loader, (2, 8, cfg.hidden_size), torch.device("cpu"), torch.float32)
    if stage.has_last:
        assert abs(loss.item() - ref_loss) < 1e-5, (engine, loss.item(), ref_loss)
    n_checked = 0
    for n, p in stage.named_parameters():
        assert p.grad is not None, (engine, n)
        err = (p.grad - ref_grads[n]).abs().max().item()
        assert err < 1e-5, (engine, n, err)
        n_checked += 1
    assert n_checked > 0


@pytest.mark.parametrize("engine", ["afab", "1f1b", "zb", "interleaved", "zbv"])
def test_pp2(engine):
    run_distributed(_pp_worker, 2, engine, 4)


@pytest.mark.parametrize("engine", ["1f1b", "zb", "interleaved", "zbv"])
def test_pp4(engine):
    run_distributed(_pp_worker, 4, engine, 8)


def _pp_dp_worker(rank, world, engine, dp_cls_name):
    """pp=2 x dp=2 on the hook-based data-parallel wrappers: every chunk's gradients must come out
    averaged over the two replicas (each replica sees different micro-batches), i.e. equal to the
    full model's gradient over all micro-batches of both replicas divided by 2."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel import data_parallel as dp_mod
    from picotron_b200.parallel.pipeline_parallel import run_schedule, wrap_pipeline

    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=2, dp_size=2)
    m_pg = pgm.get_pgm()
    cfg = tiny_config()
    m = 4
    torch.manual_seed(11)
    ref = Llama(cfg)
    for replica in range(2):
        loader = FakeDataLoader(cfg.vocab_size, 2, 8, m, seed=100 + replica)
        for _ in range(m):
            b = next(loader)
            loss = torch.nn.functional.cross_entropy(ref(b["input_ids"]).view(-1, cfg.vocab_size),
                                                     b["target_ids"].view(-1)) / (m * 2)
            loss.backward()
    ref_grads = {n: p.grad.clone() for n, p in ref.named_parameters()}

    torch.manual_seed(11)
    full = Llama(cfg)
    full.load_state_dict(ref.state_dict())
    stage = wrap_pipeline(full, cfg, engine, 2)
    model = getattr(dp_mod, dp_cls_name)(stage, group=m_pg.cp_dp_group)
    loader = FakeDataLoader(cfg.vocab_size, 2, 8, m, seed=100 + m_pg.dp_rank)
    run_schedule(engine, model, loader, (2, 8, cfg.hidden_size), torch.device("cpu"), torch.float32)
    n_checked = 0
    for n, p in stage.named_parameters():
        assert p.grad is not None, (engine, n)
        err = (p.grad - ref_grads[n]).abs().max().item()
        assert err < 1e-5, (engine, dp_cls_name, n, err)
        n_checked += 1
    assert n_checked > 0


@pytest.mark.parametrize("dp_cls", ["DataParallelNaive", "DataParallelBucket"])
@pytest.mark.parametrize("engine", ["interleaved", "1f1b"])
def test_pp2_dp2_every_chunk_is_reduced(engine, dp_cls):
    run_distributed(_pp_dp_worker, 4, engine, dp_cls)


def test_planner_places_every_action_once():
    from picotron_b200.parallel import pp_schedules as S
    for engine in S.SCHEDULES:
        for p in (2, 4, 8):
            for m in (p, 2 * p, 4 * p):
                plan, smap, split = S.build_plan(engine, p, m, 2)
                for r in range(p):
                    acts = [a for a in plan.timeline[r] if a]
                    assert len(acts) == len(set(acts)) == m * smap.v * (3 if split else 2)
                # every cross-rank message has exactly one producer round
                keys = [msg.key for rnd in plan.messages for msg in rnd]
                assert len(keys) == len(set(keys))


def test_one_f_one_b_warmup_counts():
    from picotron_b200.parallel import pp_schedules as S
    orders = S.one_f_one_b_order(4, 8)
    for rank, acts in enumerate(orders):
        warm = 0
        for a in acts:
            if a[0] != S.F:
                break
            warm += 1
        assert warm == min(4 - rank - 1, 8) + 1  # warm-up forwards plus the first steady forward
