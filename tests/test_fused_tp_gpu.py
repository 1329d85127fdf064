"""Fused tensor-parallel linears (push all-gather -> gated GEMM, GEMM -> peer-memory reduce-scatter)
on 2+ GPUs against an fp32 single-device restatement. Each rank is its own process on its own GPU
(spawned here); the test is skipped with fewer than two devices."""
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, errors):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", PICO_SYMM_CANARY="1")
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        fn(rank, world)
        torch.cuda.synchronize()
        dist.barrier()
        # every symmetric buffer of these tests sits between guard zones: no kernel of any rank may have
        # stored past an end of a buffer of this rank
        from picotron_b200.runtime.symm import check_all_canaries
        check_all_canaries()
    except Exception:
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


#: world sizes every multi-GPU test runs at (those the machine has; the rest are skipped)
WORLDS = [2, 4, 8]


def run_gpu_ranks(fn, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(360)         # several engines per test (symmetric-memory set-up, graph capture) on up to 8 ranks
    msgs = []
    while not errors.empty():
        r, tb = errors.get()
        msgs.append(f"--- rank {r} ---\n{tb}")
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    assert not msgs and not alive and all(p.exitcode == 0 for p in procs), "\n".join(msgs)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _fused_ops_worker(rank, world):
    from picotron_b200 import ops
    from picotron_b200.ops import fused_tp
    from picotron_b200.ops.gemm import WeightSet
    from picotron_b200.runtime.symm import SymmGroup

    dev = torch.device("cuda", rank)
    b, s_loc, K, N = 2, 256, 512, 768
    sg = SymmGroup(None)
    tp = fused_tp.TPFused(sg, b * s_loc, max(K, N), s_loc)
    torch.manual_seed(0)                               # same full tensors on every rank
    x_full = torch.randn(b, s_loc * world, K, device=dev).to(torch.bfloat16)
    w_col = (torch.randn(N * world, K, device=dev) / K ** 0.5).to(torch.bfloat16)     # column-parallel weight
    w_row = (torch.randn(K, N * world, device=dev) / N ** 0.5).to(torch.bfloat16)     # row-parallel weight
    g_full = torch.randn(b, s_loc * world, N * world, device=dev).to(torch.bfloat16)
    for it in range(3):                                # several rounds exercise buffer alternation
        # ---- column parallel: y[:, :, my columns] = x_full @ w_col[my rows].T
        x_sh = x_full[:, rank * s_loc:(rank + 1) * s_loc].clone().requires_grad_(True)
        w_loc = torch.nn.Parameter(w_col[rank * N:(rank + 1) * N].clone())

        class M:  # minimal module stand-in for WeightSet.of
            weight = w_loc
        y = fused_tp.ag_linear(x_sh, tp, [M])
        ref = x_full.float() @ w_loc.float().t()
        assert _rel(y, ref) < 1e-2, ("ag_linear fwd", it)
        gy = g_full[:, :, rank * N:(rank + 1) * N].contiguous()
        y.backward(gy)
        # dx shard = sum over ranks of (g[:, :, cols_r] @ w_col[rows_r]) restricted to my sequence chunk
        dx_ref = (g_full.float() @ w_col.float())[:, rank * s_loc:(rank + 1) * s_loc]
        assert _rel(x_sh.grad, dx_ref) < 1e-2, ("ag_linear dx", it)
        dw_ref = gy.float().reshape(-1, N).t() @ x_full.float().reshape(-1, K)
        assert _rel(w_loc.grad, dw_ref) < 1e-2, ("ag_linear dw", it)
        # ---- row parallel: y_shard = (x2 @ w_row[:, my cols].T summed over ranks)[my sequence chunk]
        xin_full = g_full                                  # [b, s, N*world] plays the role of the hidden activations
        xin = xin_full[:, :, rank * N:(rank + 1) * N].clone().requires_grad_(True)
        wr = torch.nn.Parameter(w_row[:, rank * N:(rank + 1) * N].clone())
        res = x_full[:, rank * s_loc:(rank + 1) * s_loc].clone().requires_grad_(True)
        out = fused_tp.linear_rs(xin, wr, tp, addend=res)
        ref_full = xin_full.float() @ w_row.float().t() + x_full.float()
        assert _rel(out, ref_full[:, rank * s_loc:(rank + 1) * s_loc]) < 1e-2, ("linear_rs fwd", it)
        go = x_full[:, rank * s_loc:(rank + 1) * s_loc].contiguous()
        out.backward(go)
        dxin_ref = x_full.float() @ wr.float()
        assert _rel(xin.grad, dxin_ref) < 1e-2, ("linear_rs dx", it)
        dwr_ref = x_full.float().reshape(-1, K).t() @ xin_full.float().reshape(-1, N * world)[:, rank * N:(rank + 1) * N]
        assert _rel(wr.grad, dwr_ref) < 1e-2, ("linear_rs dw", it)
        assert _rel(res.grad, go) < 1e-3
        # the fused reductions sum their slots in rank order: repeating an operation on the same inputs
        # gives bit-identical results (forward reduce-scatter and the dx reduce-scatter of ag_linear)
        if it == 0:
            first_out, first_dx = out.detach().clone(), x_sh.grad.detach().clone()
        else:
            assert torch.equal(out.detach(), first_out), "GEMM -> reduce-scatter is not deterministic"
            assert torch.equal(x_sh.grad, first_dx), "all-gather -> GEMM backward is not deterministic"
    ops.check_status("fused tp")


@pytest.mark.parametrize("world", WORLDS)
def test_fused_tp_ops(world):
    run_gpu_ranks(_fused_ops_worker, world)


def _timeout_worker(rank, world):
    """A flag that nobody raises: the bounded wait must give up, report, and leave the context usable."""
    from picotron_b200 import ops
    from picotron_b200.runtime.status import CommTimeoutError, raise_if_failed
    from picotron_b200.runtime.symm import SymmGroup
    sg = SymmGroup(None)
    sg.wait(slot=200, epoch=7, timeout_ms=300)      # slot 200 is never signalled
    try:
        raise_if_failed("expected")
        raise AssertionError("the wait did not report a timeout")
    except CommTimeoutError as e:
        assert e.code == 2
    # the context still works: a normal barrier over the group succeeds afterwards
    sg.barrier()
    ops.check_status("after timeout")
    t = torch.ones(4, device="cuda") * (rank + 1)
    dist.all_reduce(t)
    assert t[0].item() == sum(range(1, world + 1))


@pytest.mark.parametrize("world", WORLDS)
def test_bounded_wait_reports_timeout(world):
    run_gpu_ranks(_timeout_worker, world)


def _tp_engine_cfg(tp, dp, zero_stage=0, parallel_block=False):
    """Small Llama whose heads, KV heads and sequence divide by every tested TP size (head_dim 64, a
    sequence shard of 128 rows per rank)."""
    return {"distributed": dict(tp_size=tp, dp_size=dp, sequence_parallel=True, vocab_parallel_ce=True,
                                zero_stage=zero_stage),
            "model": dict(name="tiny-llama-test", init_std=0.02, dtype="bfloat16", num_hidden_layers=2,
                          hidden_size=1024, intermediate_size=2048, num_attention_heads=16, num_key_value_heads=8,
                          max_position_embeddings=128 * tp, parallel_block=parallel_block),
            "training": dict(seed=0, learning_rate=1e-3, seq_length=128 * tp, micro_batch_size=2,
                             gradient_accumulation_steps=2, num_samples=512),
            "dataset": dict(name="synthetic")}


def _engine_worker(rank, world):
    """Two optimizer steps of a small Llama with TP=2 + sequence parallelism + vocabulary-parallel
    loss: the fused-kernel path and the NCCL-collective path must agree to bf16 accuracy."""
    from picotron_b200 import ops
    from picotron_b200.engine import TrainEngine
    losses = {}
    for fused in ("1", "0"):
        os.environ["PICO_FUSED_TP"] = fused
        cfg = _tp_engine_cfg(world, 1)
        eng = TrainEngine(cfg, device=torch.device("cuda", rank))
        assert (eng.fused_tp is not None) == (fused == "1")
        losses[fused] = [eng.train_step().item() for _ in range(3)]
        ops.check_status("engine fused=" + fused)
    for a, b in zip(losses["1"], losses["0"]):
        assert abs(a - b) < 3e-2, losses
    assert all(x == x and x < 12.0 for x in losses["1"]), losses      # finite and sane (fresh random tokens every step)
    # the fused path replays its micro-batch from a CUDA graph (flag epochs advance on the device);
    # eager launches of the same kernels must give the same bits
    os.environ["PICO_FUSED_TP"] = "1"
    cfg["training"]["cuda_graph"] = False
    eng = TrainEngine(cfg, device=torch.device("cuda", rank))
    eager = [eng.train_step().item() for _ in range(3)]
    ops.check_status("engine eager")
    assert eager == losses["1"], (eager, losses["1"])


def _jitter_worker(rank, world):
    """Race check by double run: random per-rank delays before every communicating kernel must not
    change a single bit of three optimizer steps (eager launches, so the delays differ per step)."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    runs = {}
    for seed in ("", "7", "8"):
        os.environ["PICO_RACE_JITTER"] = seed
        pgm.process_group_manager = None
        cfg = _tp_engine_cfg(world, 1)
        cfg["training"]["cuda_graph"] = False
        eng = TrainEngine(cfg, device=torch.device("cuda", rank))
        losses = [eng.train_step().item() for _ in range(3)]
        ops.check_status("jitter seed=" + seed)
        runs[seed] = (losses, eng.store.flat_params.clone())
        eng.close()
    os.environ["PICO_RACE_JITTER"] = ""
    for seed in ("7", "8"):
        assert runs[seed][0] == runs[""][0], (seed, runs[seed][0], runs[""][0])
        assert torch.equal(runs[seed][1], runs[""][1]), f"parameters differ under launch delays (seed {seed})"


@pytest.mark.parametrize("world", WORLDS)
def test_engine_bits_survive_random_launch_delays(world):
    run_gpu_ranks(_jitter_worker, world)


@pytest.mark.parametrize("world", WORLDS)
def test_engine_fused_tp_matches_nccl_path(world):
    run_gpu_ranks(_engine_worker, world)


def _engine_ptb_worker(rank, world):
    """Parallel transformer block under TP + sequence parallelism: the peer-memory form (one pushed
    gather for q/k/v and gate/up, two scatter epilogues summed with the residual) against the same
    block on NCCL all-gather / reduce-scatter; losses over three steps and the parameters afterwards."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    from picotron_b200.ops import fused_tp
    calls = [0]
    plain = fused_tp.dual_linear_rs

    def counted(*a, **k):
        calls[0] += 1
        return plain(*a, **k)

    fused_tp.dual_linear_rs = counted
    out = {}
    for fused in ("1", "0"):
        os.environ["PICO_FUSED_TP"] = fused
        pgm.process_group_manager = None
        eng = TrainEngine(_tp_engine_cfg(world, 1, parallel_block=True), device=torch.device("cuda", rank))
        before = calls[0]
        losses = [eng.train_step().item() for _ in range(3)]
        ops.check_status("parallel block fused=" + fused)
        assert (calls[0] > before) == (fused == "1"), "the peer-memory block did not run" if fused == "1" else \
            "the NCCL arm took the peer-memory block"
        out[fused] = (losses, eng.store.flat_params.float().clone())
        eng.close()
    fused_tp.dual_linear_rs = plain
    os.environ["PICO_FUSED_TP"] = "1"
    for a, b in zip(out["1"][0], out["0"][0]):
        assert abs(a - b) < 3e-2, (out["1"][0], out["0"][0])
    rel = (out["1"][1] - out["0"][1]).norm() / out["0"][1].norm()
    assert rel < 1e-2, rel


@pytest.mark.parametrize("world", WORLDS)
def test_engine_parallel_block_on_peer_memory_matches_nccl_path(world):
    run_gpu_ranks(_engine_ptb_worker, world)


def _engine_dp_tp_worker(rank, world):
    """DP2 x TP(world/2) with sequence parallelism, vocabulary-parallel loss and ZeRO-1 — the layout of
    the 8-GPU headline run: every fused path on (peer-memory TP kernels, graph replay, one-launch
    ZeRO-1 optimizer) against the same layout on NCCL collectives; losses over three steps, the
    parameters afterwards, and identical replicas."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    out = {}
    for fused in ("1", "0"):
        os.environ["PICO_FUSED_TP"] = os.environ["PICO_FUSED_DP"] = fused
        pgm.process_group_manager = None
        eng = TrainEngine(_tp_engine_cfg(world // 2, 2, zero_stage=1), device=torch.device("cuda", rank))
        assert (eng.fused_tp is not None) == (fused == "1") and (eng.dp_symm is not None) == (fused == "1")
        losses = [eng.average_loss(eng.train_step()) for _ in range(3)]
        ops.check_status("dp x tp engine fused=" + fused)
        params = eng.store.flat_params.float().clone()
        other = params.clone()
        dist.broadcast(other, src=dist.get_global_rank(eng.pgm.dp_group, 0), group=eng.pgm.dp_group)
        assert torch.equal(other, params), "data-parallel replicas diverged"
        out[fused] = (losses, params)
        eng.close()
    for a, b in zip(out["1"][0], out["0"][0]):
        assert abs(a - b) < 3e-2, (out["1"][0], out["0"][0])
    rel = (out["1"][1] - out["0"][1]).norm() / out["0"][1].norm()
    assert rel < 1e-2, rel
    os.environ["PICO_FUSED_TP"] = os.environ["PICO_FUSED_DP"] = "1"


@pytest.mark.parametrize("world", [4, 8])
def test_engine_dp2_tp_zero1_matches_nccl_path(world):
    run_gpu_ranks(_engine_dp_tp_worker, world)


def _dp_engine_worker(rank, world):
    """DP=2 + ZeRO-1: the peer-memory optimizer kernel (reduce-scatter + AdamW + all-gather in one
    launch) against the NCCL reduce-scatter / all-gather path."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    results = {}
    for fused in ("1", "0"):
        os.environ["PICO_FUSED_DP"] = fused
        pgm.process_group_manager = None
        cfg = {"distributed": dict(tp_size=1, dp_size=world, zero_stage=1),
               "model": dict(name="tiny-llama-test", init_std=0.02, dtype="bfloat16", num_hidden_layers=2,
                             hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=4),
               "training": dict(seed=0, learning_rate=1e-3, seq_length=256, micro_batch_size=2,
                                gradient_accumulation_steps=2, num_samples=512),
               "dataset": dict(name="synthetic")}
        eng = TrainEngine(cfg, device=torch.device("cuda", rank))
        assert (eng.dp_symm is not None) == (fused == "1")
        losses = [eng.train_step().item() for _ in range(3)]
        ops.check_status("dp engine fused=" + fused)
        results[fused] = (losses, eng.store.flat_params.float().clone())
        # every replica must hold identical parameters after the step
        ref = results[fused][1].clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, results[fused][1]), "replicas diverged"
    for a, b in zip(results["1"][0], results["0"][0]):
        assert abs(a - b) < 2e-2, (results["1"][0], results["0"][0])
    rel = (results["1"][1] - results["0"][1]).norm() / results["0"][1].norm()
    assert rel < 1e-2, rel


@pytest.mark.parametrize("world", WORLDS)
def test_engine_fused_zero1_matches_nccl_path(world):
    run_gpu_ranks(_dp_engine_worker, world)


def _zero_stages_worker(rank, world):
    """ZeRO stages 2 and 3 on GPUs run on the per-parameter path (gradients dropped on non-owners,
    stage 3 also the parameters' storage); three steps of each against ZeRO-1 on the flat buffers."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    losses = {}
    for stage in (1, 2, 3):
        pgm.process_group_manager = None
        cfg = {"distributed": dict(tp_size=1, dp_size=world, zero_stage=stage),
               "model": dict(name="tiny-llama-test", init_std=0.02, dtype="bfloat16", num_hidden_layers=2,
                             hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=4),
               "training": dict(seed=0, learning_rate=1e-3, seq_length=256, micro_batch_size=2,
                                gradient_accumulation_steps=2, num_samples=512),
               "dataset": dict(name="synthetic")}
        eng = TrainEngine(cfg, device=torch.device("cuda", rank))
        assert eng.flat == (stage == 1)
        losses[stage] = [eng.average_loss(eng.train_step()) for _ in range(3)]
        ops.check_status(f"zero stage {stage}")
        if stage == 3:
            held = sum(p.untyped_storage().size() for p in eng.model.parameters())
            whole = sum(p.numel() * p.element_size() for p in eng.model.parameters())
            assert held < 0.75 * whole, (held, whole)          # the other rank's parameters are not resident
        eng.close()
    for stage in (2, 3):
        for a, b in zip(losses[stage], losses[1]):
            assert abs(a - b) < 5e-2, losses


def test_engine_zero_stages_2_and_3_shard_on_gpu():
    run_gpu_ranks(_zero_stages_worker, 2)


def _moe_engine_cfg(world, graph, dropless=False):
    return {"distributed": dict(ep_size=world, ep_as_dp=True),
            "model": dict(name="moe-graph-test", init_std=0.02, dtype="bfloat16", num_hidden_layers=2, hidden_size=512,
                          intermediate_size=256, num_attention_heads=8, num_key_value_heads=8, vocab_size=4096,
                          max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0, num_experts=8, num_experts_per_tok=2, num_shared_experts=0,
                          shared_expert_intermediate_size=512, router_aux_loss_coef=1e-3, router_bias_update_rate=1e-3,
                          ep_capacity_factor=0.0 if dropless else 1.25, ep_capacity_dropless=False,
                          ep_fp8_dispatch=True, ep_backend="fused" if dropless else "torch"),
            "training": dict(seed=1, learning_rate=1e-3, seq_length=512, micro_batch_size=2,
                             gradient_accumulation_steps=2, num_samples=512, cuda_graph=graph),
            "dataset": dict(name="synthetic")}


def _moe_graph_worker(rank, world, dropless=False):
    """MoE model on a peer-memory path (capacity-limited: routing, slot assignment, dispatch, experts,
    combine; dropless: layout computed on the device; the expert-load sum through peer memory in both):
    the micro-batch replayed from a CUDA graph against eager launches of the same kernels, four optimizer
    steps; the loss-free bias must have moved identically."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    from picotron_b200.parallel.expert_parallel import MoELayer
    out = {}
    for graph in (True, False):
        pgm.process_group_manager = None
        eng = TrainEngine(_moe_engine_cfg(world, graph, dropless), device=torch.device("cuda", rank))
        assert eng.fused_ep is not None
        losses = [eng.average_loss(eng.train_step()) for _ in range(4)]
        ops.check_status(f"moe engine graph={graph}")
        assert bool(eng._mb_graph) == graph, "the graph switch did not take"
        bias = torch.stack([m.expert_bias.float() for m in eng.model.modules() if isinstance(m, MoELayer)])
        out[graph] = (losses, bias.clone(), eng.store.flat_params.float().clone())
        eng.close()
    for a, b in zip(out[True][0], out[False][0]):
        assert abs(a - b) < 2e-2, (out[True][0], out[False][0])
    assert all(x == x and x < 10.0 for x in out[True][0]), out[True][0]
    assert torch.equal(out[True][1], out[False][1]), "expert bias differs between replay and eager launches"
    rel = (out[True][2] - out[False][2]).norm() / out[False][2].norm()
    assert rel < 1e-2, rel


@pytest.mark.parametrize("world", WORLDS)
def test_engine_moe_graph_replay_matches_eager(world):
    run_gpu_ranks(_moe_graph_worker, world)


def _moe_graph_dropless_worker(rank, world):
    _moe_graph_worker(rank, world, dropless=True)


@pytest.mark.parametrize("world", WORLDS)
def test_engine_dropless_moe_graph_replay_matches_eager(world):
    run_gpu_ranks(_moe_graph_dropless_worker, world)


def _ep_worker(rank, world):
    """Capacity-mode MoE layer on EP=2: exchanges through the peer-memory kernels (bf16 and FP8 block
    scaled dispatch) against the NCCL all-to-all path of the same layer; outputs and gradients."""
    import types
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.ops.fused_ep import EPFused
    from picotron_b200.parallel.capacity_moe import compute_capacity
    from picotron_b200.parallel.expert_parallel import MoELayer
    from picotron_b200.runtime.symm import SymmGroup
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    dev = torch.device("cuda", rank)
    sg = SymmGroup(pgm.get_pgm().ep_group, device=dev)
    for fp8 in (False, True):
        for dropless in (False, True):
            cfg = types.SimpleNamespace(hidden_size=512, intermediate_size=256, num_experts=8, num_experts_per_tok=2,
                                        num_shared_experts=1, norm_topk_prob=True, ep_fp8_dispatch=fp8,
                                        ep_capacity_factor=0.75, ep_capacity_dropless=dropless, ep_max_rounds=8,
                                        init_std=0.05, ep_overlap=False)
            torch.manual_seed(3)
            layer = MoELayer(cfg).to(dev).to(torch.bfloat16)
            torch.manual_seed(10 + rank)
            x = torch.randn(2, 256, 512, device=dev, dtype=torch.bfloat16)
            T = 512
            C = compute_capacity(T, 2, 8, 0.75)
            outs = []
            for fused in (False, True):
                layer.fused_ep = EPFused(sg, layer.num_local_experts, C, 512) if fused else None
                xi = x.clone().requires_grad_(True)
                layer.zero_grad()
                y = layer(xi)
                y.float().square().mean().backward()
                outs.append((y.detach().float(), xi.grad.float(),
                             layer.local_experts[0].down_proj.weight.grad.float().clone(),
                             layer.gate.weight.grad.float().clone()))
            ops.check_status(f"fused ep fp8={fp8} dropless={dropless}")
            names = ("output", "input grad", "expert weight grad", "router grad")
            for n, a, b in zip(names, outs[1], outs[0]):
                rel = ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
                assert rel < 3e-2, (n, fp8, dropless, rel)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_ep_capacity_moe(world):
    run_gpu_ranks(_ep_worker, world)


def _cp_worker(rank, world):
    """Ring (flash kernels per block, position offsets) and Ulysses attention on 2 GPUs in bf16 against
    single-device attention over the full sequence."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.ops import attention as A
    from picotron_b200.parallel.context_parallel import ring_attention_bshd
    from picotron_b200.parallel.ulysses import ulysses_attention_bshd
    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    b, s, H, Hkv, d = 1, 512 * world, 16, 8, 64      # Ulysses splits both head counts over the ranks
    q = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
    k = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
    v = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
    go = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, True)
    ref.backward(go.float())
    sl = slice(rank * s // world, (rank + 1) * s // world)
    for fn in (ring_attention_bshd, ulysses_attention_bshd):
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = fn(ql, kl, vl, True)
        out.backward(go[:, sl].contiguous())
        ops.check_status(fn.__name__)
        assert _rel(out, ref[:, sl]) < 2e-2, fn.__name__
        for got, want in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
            assert _rel(got, want[:, sl]) < 3e-2, fn.__name__


@pytest.mark.parametrize("world", WORLDS)
def test_context_parallel_attention(world):
    run_gpu_ranks(_cp_worker, world)


def _fused_cp_worker(rank, world):
    """Causal context-parallel attention with the K/V gather and dK/dV reduction through peer memory
    (``ops.fused_cp``) against single-device attention over the full sequence; several rounds so both
    copies of the double-buffered symmetric buffers are reused."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.ops import attention as A
    from picotron_b200.ops.fused_cp import CPFused
    from picotron_b200.parallel import context_parallel as cpar
    from picotron_b200.runtime.symm import SymmGroup
    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    group = pgm.get_pgm().cp_group
    dev = torch.device("cuda", rank)
    b, s_loc, H, Hkv, d = 2, 384, 8, 2, 64
    s = s_loc * world
    cp = CPFused(SymmGroup(group, device=dev), b, s_loc, Hkv * d)
    cpar.install_fused_cp(cp)
    try:
        for rnd in range(3):
            torch.manual_seed(rnd)
            q = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
            k = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
            v = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
            go = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
            qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
            ref = A.attention_ref(qr, kr, vr, True)
            ref.backward(go.float())
            sl = slice(rank * s_loc, (rank + 1) * s_loc)
            ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
            before = cp.n_gather
            out = cpar.ring_attention_bshd(ql, kl, vl, True)
            out.backward(go[:, sl].contiguous())
            ops.check_status("fused cp")
            assert cp.n_gather == before + 2, "the peer-memory path was not taken"
            assert _rel(out, ref[:, sl]) < 2e-2, rnd
            for name, got, want in (("dq", ql.grad, qr.grad), ("dk", kl.grad, kr.grad), ("dv", vl.grad, vr.grad)):
                assert _rel(got, want[:, sl]) < 3e-2, (name, rnd, _rel(got, want[:, sl]))
    finally:
        cpar.install_fused_cp(None)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_context_parallel_attention(world):
    run_gpu_ranks(_fused_cp_worker, world)


def _fused_ulysses_worker(rank, world):
    """Ulysses attention with the peer-memory all-to-all kernels (``ops.fused_ulysses``) against
    single-device attention over the full sequence, forward and backward, batch 2, GQA."""
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.ops import attention as A
    from picotron_b200.ops.fused_ulysses import UlyssesFused
    from picotron_b200.parallel import ulysses as uly
    from picotron_b200.runtime.symm import SymmGroup
    pgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    group = pgm.get_pgm().cp_group
    dev = torch.device("cuda", rank)
    b, s_loc, H, Hkv, d = 2, 256, 4 * world, 2 * world, 64
    s = s_loc * world
    u = UlyssesFused(SymmGroup(group, device=dev), b, s_loc, H * d)
    uly.install_fused_ulysses(u)
    try:
        for rnd in range(3):
            torch.manual_seed(10 + rnd)
            q = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
            k = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
            v = torch.randn(b, s, Hkv, d, device=dev, dtype=torch.bfloat16)
            go = torch.randn(b, s, H, d, device=dev, dtype=torch.bfloat16)
            qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
            ref = A.attention_ref(qr, kr, vr, True)
            ref.backward(go.float())
            sl = slice(rank * s_loc, (rank + 1) * s_loc)
            ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
            before = u.n_seq
            out = uly.ulysses_attention_bshd(ql, kl, vl, True)
            out.backward(go[:, sl].contiguous())
            ops.check_status("fused ulysses")
            assert u.n_seq == before + 4, "the peer-memory path was not taken"   # q, k, v forward + dout backward
            assert _rel(out, ref[:, sl]) < 2e-2, rnd
            for name, got, want in (("dq", ql.grad, qr.grad), ("dk", kl.grad, kr.grad), ("dv", vl.grad, vr.grad)):
                assert _rel(got, want[:, sl]) < 3e-2, (name, rnd, _rel(got, want[:, sl]))
    finally:
        uly.install_fused_ulysses(None)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_ulysses_attention(world):
    run_gpu_ranks(_fused_ulysses_worker, world)


def _ep_var_worker(rank, world):
    """Dropless MoE layer on EP=2 with the variable-size exchange laid out on the device and carried
    through peer memory (``ops.fused_ep_var``) against the NCCL variable-size all-to-all path of the
    same layer: outputs and gradients, several rounds with different (skewed) routings so both copies
    of every buffer are reused and experts with few or no rows occur."""
    import types
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.ops.fused_ep_var import EPVarFused
    from picotron_b200.parallel.expert_parallel import MoELayer
    from picotron_b200.runtime.symm import SymmGroup
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    dev = torch.device("cuda", rank)
    sg = SymmGroup(pgm.get_pgm().ep_group, device=dev)
    cfg = types.SimpleNamespace(hidden_size=512, intermediate_size=256, num_experts=8, num_experts_per_tok=2,
                                num_shared_experts=1, norm_topk_prob=True, ep_capacity_factor=0.0, init_std=0.05,
                                ep_overlap=False)
    torch.manual_seed(3)
    layer = MoELayer(cfg).to(dev).to(torch.bfloat16)
    T = 512
    # the router is skewed on purpose: with few experts per rank one rank can receive most rows
    slack = 2.0 if world == 2 else float(world)
    epv_bf16 = EPVarFused(sg, layer.num_local_experts, 512, T * 2, slack=slack)
    epv_fp8 = EPVarFused(sg, layer.num_local_experts, 512, T * 2, slack=slack, fp8_dispatch=True)
    assert epv_fp8.fp8
    for rnd in range(4):
        epv = epv_fp8 if rnd == 3 else epv_bf16      # last round: FP8 block-scaled forward dispatch
        torch.manual_seed(100 * rnd + rank)
        x = torch.randn(2, 256, 512, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():     # skew the router so that some experts get (almost) nothing
            layer.expert_bias.zero_()
            layer.gate.weight[rnd % 3].add_(0.5)
            layer.gate.weight[7 - rnd % 3].sub_(0.5)
        outs = []
        for fused in (False, True):
            layer.fused_ep_var = epv if fused else None
            xi = x.clone().requires_grad_(True)
            layer.zero_grad()
            before = epv.n["dispatch"]
            y = layer(xi)
            y.float().square().mean().backward()
            assert (epv.n["dispatch"] - before == 2) == fused, "wrong path taken"
            outs.append((y.detach().float(), xi.grad.float(),
                         layer.local_experts[0].down_proj.weight.grad.float().clone(),
                         layer.local_experts[-1].gate_proj.weight.grad.float().clone(),
                         layer.gate.weight.grad.float().clone()))
        ops.check_status(f"fused dropless ep round {rnd}")
        names = ("output", "input grad", "expert down grad", "expert gate grad", "router grad")
        for n, a, b in zip(names, outs[1], outs[0]):
            rel = ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
            assert rel < (6e-2 if rnd == 3 else 3e-2), (n, rnd, rel)
    layer.fused_ep_var = None


@pytest.mark.parametrize("world", WORLDS)
def test_fused_dropless_ep(world):
    run_gpu_ranks(_ep_var_worker, world)
