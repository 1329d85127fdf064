"""End-to-end trainer plumbing on CPU/gloo: the tiny-Llama config (4 layers, hidden 256, 8 heads,
4 KV heads, FFN 688, vocab 4096, seq 256, micro-batch 2, 2 accumulation steps, N(0, 0.02) init)
run as TP=2 and as DP=2 with ZeRO-1 must reproduce the single-process losses; checkpoints resume
exactly; the command-line tools round-trip."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tiny_cfg(**dist_kw):
    d = dict(tp_size=1, dp_size=1, use_cpu=True)
    d.update(dist_kw)
    return {"distributed": d,
            "model": dict(name="tiny-llama-test", init_std=0.02, dtype="float32"),
            "training": dict(seed=0, learning_rate=1e-3, seq_length=256, micro_batch_size=2,
                             gradient_accumulation_steps=2, num_samples=4096),
            "dataset": dict(name="synthetic")}


def _engine_worker(rank, world, dist_kw, steps, out_path):
    from picotron_b200.engine import TrainEngine
    engine = TrainEngine(tiny_cfg(**dist_kw), device=torch.device("cpu"))
    losses = []
    for _ in range(steps):
        losses.append(engine.average_loss(engine.train_step()))
    if rank == 0:
        state = {k: v.clone() for k, v in engine.model.state_dict().items()}
        torch.save({"losses": losses, "state": state}, out_path)


def test_tp2_matches_single_process(tmp_path):
    a, b = str(tmp_path / "single.pt"), str(tmp_path / "tp2.pt")
    run_distributed(_engine_worker, 1, {}, 2, a)
    run_distributed(_engine_worker, 2, dict(tp_size=2, sequence_parallel=True, vocab_parallel_ce=True), 2, b)
    la, lb = torch.load(a)["losses"], torch.load(b)["losses"]
    for x, y in zip(la, lb):
        assert abs(x - y) < 1e-5, (la, lb)


def _dp_equiv_worker(rank, world, zero_stage, out_path):
    """DP=2 with grad-acc 2 consumes, per step, the samples a single process with grad-acc 4 sees
    (rank r takes samples r, r+2, ...), so losses and weights must agree."""
    from picotron_b200.engine import TrainEngine
    cfg = tiny_cfg(dp_size=world, zero_stage=zero_stage)
    engine = TrainEngine(cfg, device=torch.device("cpu"))
    losses = [engine.average_loss(engine.train_step()) for _ in range(2)]
    if rank == 0:
        # under ZeRO-3 non-owned parameters have no storage at rest, so only losses are compared
        state = {} if zero_stage == 3 else {k: v.clone() for k, v in engine.model.state_dict().items()}
        torch.save({"losses": losses, "state": state}, out_path)


def _single_equiv_worker(rank, world, out_path):
    from picotron_b200.engine import TrainEngine
    from picotron_b200.data import MicroBatchDataLoader
    cfg = tiny_cfg()
    cfg["training"]["gradient_accumulation_steps"] = 4
    engine = TrainEngine(cfg, device=torch.device("cpu"))

    class Interleave:
        """Feeds a 1-rank engine the micro-batches of a 2-way DP run: (r0 mb0, r1 mb0, r0 mb1, r1 mb1)."""
        def __init__(self):
            self.loaders = [MicroBatchDataLoader(2, 256, "synthetic", grad_acc_steps=2, vocab_size=4096, seed=0,
                                                 num_samples=4096, dp_world_size=2, dp_rank=r, cp_world_size=1,
                                                 cp_rank=0) for r in range(2)]
            self.grad_acc_steps, self.i = 4, 0
        def __iter__(self):
            return self
        def __next__(self):
            b = next(self.loaders[self.i % 2])
            self.i += 1
            return b
    engine.data_loader = Interleave()
    losses = [engine.average_loss(engine.train_step()) for _ in range(2)]
    torch.save({"losses": losses, "state": {k: v.clone() for k, v in engine.model.state_dict().items()}}, out_path)


@pytest.mark.parametrize("zero_stage", [0, 1, 2, 3])
def test_dp2_zero_matches_single_process(tmp_path, zero_stage):
    a, b = str(tmp_path / "single.pt"), str(tmp_path / "dp2.pt")
    run_distributed(_single_equiv_worker, 1, a)
    run_distributed(_dp_equiv_worker, 2, zero_stage, b)
    ra, rb = torch.load(a), torch.load(b)
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) < 1e-5, (ra["losses"], rb["losses"])
    if zero_stage < 3:
        for k in ra["state"]:
            assert (ra["state"][k] - rb["state"][k]).abs().max().item() < 1e-4, k  # Adam amplifies summation-order noise to ~lr


def _zero_bitexact_worker(rank, world):
    """ZeRO-1/2/3 equal plain (naive all-reduce) data parallelism bit for bit over 5 AdamW steps
    (the criterion of the reference's tests/test_data_parallel_zero.py:124)."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.parallel.data_parallel import DataParallelNaive
    from picotron_b200.parallel.zero import DataParallelZero, ShardedOptimizer
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=world)

    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 8))

    def run(wrap):
        model = make()
        dp, opt = wrap(model)
        for step in range(5):
            torch.manual_seed(100 * step + rank)
            x, y = torch.randn(4, 16), torch.randn(4, 8)
            torch.nn.functional.mse_loss(dp(x), y).backward()
            opt.step()
            opt.zero_grad()
        return dp.full_parameters() if hasattr(dp, "full_parameters") else [p.data.clone() for p in model.parameters()]

    base = run(lambda m: (DataParallelNaive(m), torch.optim.AdamW(m.parameters(), lr=1e-2)))
    for stage in (1, 2, 3):
        def wrap(m, stage=stage):
            dp = DataParallelZero(m, stage=stage)
            return dp, ShardedOptimizer(dp, torch.optim.AdamW, lr=1e-2)
        got = run(wrap)
        for a, b in zip(base, got):
            assert (a - b).abs().max().item() == 0.0, stage
        if stage == 3:
            dp, _ = wrap(make())
            held = sum(p.data.untyped_storage().nbytes() for p in dp.module.parameters())
            full = sum(p.numel() * 4 for p in dp.module.parameters())
            assert held < full


def test_zero_bit_exact_vs_plain_dp():
    run_distributed(_zero_bitexact_worker, 2)


def _ckpt_worker(rank, world, tmp):
    from picotron_b200.checkpoint import CheckpointManager
    from picotron_b200.engine import TrainEngine
    dist_kw = dict(tp_size=2, sequence_parallel=True, vocab_parallel_ce=True)
    engine = TrainEngine(tiny_cfg(**dist_kw), device=torch.device("cpu"))
    for _ in range(2):
        engine.train_step()
    ckpt = CheckpointManager()
    out = os.path.join(tmp, "2")
    ckpt.save_checkpoint(engine.model, engine.optimizer, engine.trained_steps, engine.trained_tokens, out,
                         data_loader=engine.data_loader)
    want = engine.average_loss(engine.train_step())
    engine2 = TrainEngine(tiny_cfg(**dist_kw), device=torch.device("cpu"))
    steps, tokens = ckpt.load_checkpoint(engine2.model, engine2.optimizer, out, data_loader=engine2.data_loader)
    assert (steps, tokens) == (2, 2 * engine.tokens_per_step)
    got = engine2.average_loss(engine2.train_step())
    assert abs(got - want) < 1e-6, (got, want)
    if rank == 0:
        names = sorted(os.listdir(out))
        assert "weights_tp_rank_world_size=0_2_pp_rank_world_size=0_1.pth" in names
        assert "weights_tp_rank_world_size=1_2_pp_rank_world_size=0_1.pth" in names and "manifest.json" in names
        sd = torch.load(os.path.join(out, names[1]), weights_only=False)
        assert set(sd) >= {"model", "optimizer", "trained_steps", "trained_tokens"}
        assert "decoder_layers.0.attention.q_proj.weight" in sd["model"] and "final_proj.weight" in sd["model"]


def test_checkpoint_resume_reproduces_next_loss(tmp_path):
    run_distributed(_ckpt_worker, 2, str(tmp_path))


def _ckpt_cp_zero_worker(rank, world, tmp):
    """cp=2 with ZeRO-1: the optimizer is sharded over the context-parallel ranks, so each of them
    owns different Adam state; a resume must restore every rank's own shard bit for bit."""
    from picotron_b200.checkpoint import CheckpointManager
    from picotron_b200.engine import TrainEngine
    dist_kw = dict(cp_size=2, zero_stage=1, cp_attention="ring")
    engine = TrainEngine(tiny_cfg(**dist_kw), device=torch.device("cpu"))
    assert engine.optimizer_is_sharded
    for _ in range(2):
        engine.train_step()
    ckpt = CheckpointManager()
    out = os.path.join(tmp, "2")
    ckpt.save_checkpoint(engine.model, engine.optimizer, engine.trained_steps, engine.trained_tokens, out,
                         data_loader=engine.data_loader, sharded_optimizer=True)
    saved_state = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in _flat_state(engine.optimizer).items()}
    want = [engine.average_loss(engine.train_step()) for _ in range(2)]
    engine2 = TrainEngine(tiny_cfg(**dist_kw), device=torch.device("cpu"))
    ckpt.load_checkpoint(engine2.model, engine2.optimizer, out, data_loader=engine2.data_loader,
                         sharded_optimizer=True)
    engine2.trained_steps, engine2.trained_tokens = 2, 2 * engine.tokens_per_step
    got_state = _flat_state(engine2.optimizer)
    assert saved_state.keys() == got_state.keys() and len(saved_state) > 0
    for k in saved_state:
        a, b = saved_state[k], got_state[k]
        assert torch.equal(a, b) if torch.is_tensor(a) else a == b, (rank, k)
    got = [engine2.average_loss(engine2.train_step()) for _ in range(2)]
    assert got == want, (got, want)
    dist.barrier()
    if rank == 0:
        names = sorted(os.listdir(out))
        manifest = json.load(open(os.path.join(out, "manifest.json")))
        for cp in range(2):
            n = f"optimizer_dp_rank=0_1_cp_rank={cp}_2_tp_rank_world_size=0_1_pp_rank_world_size=0_1.pth"
            assert n in names and n in manifest["files"], names
        # a missing shard makes the checkpoint incomplete
        os.remove(os.path.join(out, "optimizer_dp_rank=0_1_cp_rank=1_2_tp_rank_world_size=0_1_pp_rank_world_size=0_1.pth"))
    dist.barrier()
    try:
        ckpt.load_checkpoint(engine2.model, engine2.optimizer, out, sharded_optimizer=True)
        raise AssertionError("a checkpoint with a missing optimizer shard was accepted")
    except FileNotFoundError:
        pass


def _flat_state(optimizer):
    """{name: tensor or number} of every entry of an optimizer state dict, nested dicts flattened."""
    out = {}

    def walk(prefix, obj):
        if isinstance(obj, dict):
            for k, v in obj.items():
                walk(f"{prefix}.{k}", v)
        elif isinstance(obj, (list, tuple)):
            for i, v in enumerate(obj):
                walk(f"{prefix}[{i}]", v)
        elif torch.is_tensor(obj) or isinstance(obj, (int, float)):
            out[prefix] = obj
    walk("", optimizer.state_dict())
    return out


def test_checkpoint_resume_cp2_zero1_restores_every_shard(tmp_path):
    run_distributed(_ckpt_cp_zero_worker, 2, str(tmp_path))


def test_create_config_and_train_cli(tmp_path):
    out = subprocess.run([sys.executable, os.path.join(REPO, "create_config.py"), "--out_dir", str(tmp_path),
                          "--exp_name", "cli", "--model_name", "tiny-llama-test", "--use_cpu", "--dataset", "synthetic",
                          "--mbs", "2", "--seq_len", "64", "--grad_acc_steps", "2", "--dp", "2", "--zero_stage", "1",
                          "--total_train_steps", "2", "--init_std", "0.02"],
                         capture_output=True, text=True, cwd=REPO)
    assert out.returncode == 0, out.stderr
    cfg_path = tmp_path / "cli" / "config.json"
    cfg = json.load(open(cfg_path))
    assert cfg["distributed"]["dp_size"] == 2 and cfg["distributed"]["zero_stage"] == 1
    cfg["checkpoint"]["save_dir"] = str(tmp_path / "ckpt")
    cfg["checkpoint"]["save_frequency"] = 2
    cfg["logging"]["log_frequency"] = 2          # step 1 is neither synchronised nor printed
    json.dump(cfg, open(cfg_path, "w"))
    env = dict(os.environ, PICO_WATCHDOG_TIMEOUT="0")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29617", os.path.join(REPO, "train.py"),
                          "--config", str(cfg_path)], capture_output=True, text=True, cwd=REPO, env=env, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    log = tmp_path / "cli" / "train.log"
    log.write_text(run.stdout)
    assert "Step: 2" in run.stdout and "Tokens/s/GPU:" in run.stdout and "MFU:" in run.stdout
    assert "Step: 1 " not in run.stdout
    assert os.path.exists(tmp_path / "ckpt" / "2" / "manifest.json")
    ex = subprocess.run([sys.executable, os.path.join(REPO, "extract_metrics.py"), str(tmp_path)],
                        capture_output=True, text=True, cwd=REPO)
    assert ex.returncode == 0, ex.stderr
    assert os.path.exists(tmp_path / "global_metrics.csv")
    rows = open(tmp_path / "global_metrics.csv").read().strip().splitlines()
    assert rows[0].startswith("run_name,status,dp,tp,pp") and len(rows) == 2


def _ep_as_dp_worker(rank, world):
    """EP=2 used as data parallelism for the dense weights: every EP rank trains on different tokens;
    dense replicas must stay identical, experts (one owner each) must not be averaged away."""
    from picotron_b200.engine import TrainEngine
    cfg = tiny_cfg(ep_size=world, ep_as_dp=True)
    cfg["model"].update(num_experts=4, num_experts_per_tok=2, num_shared_experts=1, intermediate_size=128,
                        router_aux_loss_coef=0.01, num_hidden_layers=2)
    cfg["training"].update(seq_length=64)
    engine = TrainEngine(cfg, device=torch.device("cpu"))
    assert engine.data_loader.dp_world_size == world and engine.data_loader.dp_rank == rank
    losses = [engine.average_loss(engine.train_step()) for _ in range(3)]
    assert all(l == l for l in losses)
    for name, p in engine.model.named_parameters():
        mine = p.detach().clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        if ".local_experts." in name:
            continue
        assert torch.equal(mine, other), f"dense replica diverged: {name}"
    g = engine.model.decoder_layers[0].mlp.local_experts[0].down_proj.weight
    assert g.grad is None or torch.isfinite(g.grad).all()


def test_ep_as_dp_keeps_dense_replicas_in_sync():
    run_distributed(_ep_as_dp_worker, 2)
