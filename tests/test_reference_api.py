"""Names that scripts written against the reference import besides the layer classes: block-level ring
attention helpers, functional sequence-parallel linears, the pipeline exchange helpers of the interleaved
and V-shaped schedules, the asynchronous all-to-all, the grouped-expert functions and small tensor helpers.
Each is checked against a dense single-process formula."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F

from distributed_helpers import run_distributed


def _dense_attention(q, k, v, causal):
    s = q.shape[2]
    scores = q @ k.transpose(-1, -2) / q.shape[-1] ** 0.5
    if causal:
        scores = scores.masked_fill(torch.triu(torch.ones(s, k.shape[2], dtype=torch.bool), 1), float("-inf"))
    return torch.softmax(scores, -1) @ v


def test_every_public_name_of_the_reference_modules_resolves():
    """The reference's public functions and classes, module by module (its per-tile dataclasses of the tiled
    MoE implementation are internals and have no counterpart)."""
    import importlib
    names = {
        "picotron.model": ["Llama", "DecoderLayer", "Attention", "MLP", "LlamaRMSNorm", "TritonRMSNorm", "get_cos_sin",
                           "apply_rotary_pos_emb", "flash_attention"],
        "picotron.tensor_parallel.tp_communications": ["merge_first_two_dims", "split_tensor_along_last_dim",
                                                       "vocab_parallel_cross_entropy", "linear_with_async_all_reduce"],
        "picotron.sequence_parallel.sequence_parallel": ["column_parallel_linear_sp", "GatherFromSequenceParallelRegion",
                                                         "ReduceScatterToSequenceParallelRegion"],
        "picotron.sequence_parallel.overlap": ["overlapped_column_parallel_linear_sp", "overlapped_row_parallel_linear_sp",
                                               "OverlappedColumnParallelLinearSP", "OverlappedRowParallelLinearSP"],
        "picotron.pipeline_parallel.pp_communications": ["pipeline_communicate", "bidirectional_pipeline_communicate",
                                                         "interleaved_pipeline_communicate", "vshape_pipeline_communicate"],
        "picotron.context_parallel.context_parallel": ["ring_attention", "RingAttentionFunc", "RingFlashAttentionFunc",
                                                       "ring_attention_forward", "ring_attention_backward",
                                                       "update_out_and_lse", "update_rope_for_context_parallel"],
        "picotron.expert_parallel.ep_communications": ["all_to_all", "all_to_all_async", "all_to_all_no_grad_async",
                                                       "exchange_split_sizes"],
        "picotron.expert_parallel.megakernel": ["fused_moe", "fused_moe_forward", "fused_moe_backward", "fused_moe_dgrad",
                                                "fused_moe_wgrad", "torch_fused_ffn", "torch_moe_backward",
                                                "cuda_available"],
        "picotron.expert_parallel.deepep_backend": ["deepep_available", "dispatch", "combine"],
    }
    for mod, wanted in names.items():
        m = importlib.import_module(mod)
        missing = [n for n in wanted if not hasattr(m, n)]
        assert not missing, (mod, missing)


def test_block_level_ring_helpers_reproduce_dense_attention():
    from picotron.context_parallel.context_parallel import (ring_attention_backward, ring_attention_forward,
                                                            update_out_and_lse)
    torch.manual_seed(0)
    b, h, s, d = 2, 3, 8, 16
    q, k, v = (torch.randn(b, h, s, d, dtype=torch.float64) for _ in range(3))
    scale = d ** -0.5
    # keys in two blocks, no mask: merging the blocks' results equals attention over all keys
    out = lse = None
    for lo in (0, s // 2):
        o_blk, l_blk = ring_attention_forward(q, k[:, :, lo:lo + s // 2], v[:, :, lo:lo + s // 2], scale, False)
        out, lse = update_out_and_lse(out, lse, o_blk, l_blk)
    assert lse.shape == (b, h, s, 1)
    want = _dense_attention(q, k, v, False)
    assert (out.double() - want).abs().max() < 1e-5
    # one causal block, forward and backward against autograd
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = _dense_attention(qa, ka, va, True)
    go = torch.randn_like(ref)
    ref.backward(go)
    o, l = ring_attention_forward(q, k, v, scale, True)
    assert (o - ref.detach()).abs().max() < 1e-6
    dq, dk, dv = ring_attention_backward(go, q, k, v, o, l, scale, True)
    for got, leaf in ((dq, qa), (dk, ka), (dv, va)):
        assert (got - leaf.grad).abs().max() < 1e-5


def test_model_level_helpers():
    os.environ.update(DEVICE="cpu", DTYPE="float32")
    from picotron.model import TritonRMSNorm, apply_rotary_pos_emb, flash_attention, get_cos_sin
    from picotron.tensor_parallel.tp_communications import merge_first_two_dims, split_tensor_along_last_dim
    torch.manual_seed(1)
    cos, sin = get_cos_sin(12, 8, base=10000.0)
    assert cos.shape == (12, 8) and torch.allclose(cos[:, :4], cos[:, 4:])
    x = torch.randn(2, 3, 12, 8)
    y = apply_rotary_pos_emb(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)          # a rotation
    assert torch.allclose(apply_rotary_pos_emb(y, cos, -sin), x, atol=1e-5)   # ... undone by the opposite angle
    out = flash_attention(x, x, x, causal=True)
    assert out.shape == (2, 12, 3, 8)
    assert torch.allclose(out.transpose(1, 2), _dense_attention(x, x, x, True), atol=1e-5)
    norm = TritonRMSNorm(8, eps=1e-5)
    h = torch.randn(2, 5, 8)
    assert torch.allclose(norm(h), h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5), atol=1e-5)
    res = torch.randn_like(h)
    assert torch.allclose(norm(h, residual=res), norm(h + res), atol=1e-5)
    a, c = merge_first_two_dims(torch.randn(2, 3, 4), torch.randn(2, 3, 5))
    assert a.shape == (6, 4) and c.shape == (6, 5)
    parts = split_tensor_along_last_dim(torch.arange(12.0).view(2, 6), 3)
    assert len(parts) == 3 and parts[1].tolist() == [[2.0, 3.0], [8.0, 9.0]]
    with pytest.raises(AssertionError):
        split_tensor_along_last_dim(torch.zeros(2, 5), 3)


def test_grouped_expert_functions_match_an_expert_loop():
    from picotron.expert_parallel import deepep_backend, megakernel as mk
    torch.manual_seed(2)
    counts = torch.tensor([5, 0, 9, 2])                         # an empty expert among ragged segments
    E, H, I = 4, 8, 12
    x = torch.randn(int(counts.sum()), H, dtype=torch.float64)
    gw, uw, dw = (torch.randn(E, I, H, dtype=torch.float64), torch.randn(E, I, H, dtype=torch.float64),
                  torch.randn(E, H, I, dtype=torch.float64))
    rw = torch.rand(x.shape[0], dtype=torch.float64)
    want, lo = [], 0
    for e, n in enumerate(counts.tolist()):
        seg = x[lo:lo + n]
        want.append((F.silu(seg @ gw[e].T) * (seg @ uw[e].T)) @ dw[e].T)
        lo += n
    want = torch.cat(want)
    assert torch.allclose(mk.fused_moe_forward(x, counts, gw, uw, dw), want)
    assert torch.allclose(mk.fused_moe(x, counts, gw, uw, dw, rw), want * rw[:, None])
    dy = torch.randn_like(want)
    got = mk.fused_moe_backward(x, counts, gw, uw, dw, dy)
    ref = mk.torch_moe_backward(x, counts, gw, uw, dw, dy)
    assert all(torch.allclose(a, b) for a, b in zip(got, ref)) and got[1][1].abs().max() == 0   # empty expert: zero grad
    dx, act, d13 = mk.fused_moe_dgrad(x, counts, gw, uw, dw, dy)              # the explicit two-step backward
    assert act.shape == (x.shape[0], I) and d13.shape == (x.shape[0], 2 * I)
    assert all(torch.allclose(a, b) for a, b in zip((dx, *mk.fused_moe_wgrad(x, counts, act, d13, dy)), ref))
    assert deepep_backend.deepep_available() is False
    with pytest.raises(RuntimeError):
        deepep_backend.dispatch(None, x, None, None, E)


def _sp_functional_worker(rank, world):
    """Functional sequence-parallel linears (plain and chunk-overlapped) against dense matmuls: outputs and
    gradients of the shard, the weight slice and the optional addend."""
    from picotron_b200 import process_group_manager as pgm
    from picotron.sequence_parallel.overlap import (OverlappedRowParallelLinearSP, overlapped_column_parallel_linear_sp,
                                                    overlapped_row_parallel_linear_sp)
    from picotron.sequence_parallel.sequence_parallel import column_parallel_linear_sp
    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    torch.manual_seed(3)
    b, s, h, n = 2, 8, 6, 10
    x_full = torch.randn(b, s, h, dtype=torch.float64)
    w_full = torch.randn(n, h, dtype=torch.float64)
    go_full = torch.randn(b, s, n // world, dtype=torch.float64)
    sl = slice(rank * s // world, (rank + 1) * s // world)
    w_col = w_full[rank * n // world:(rank + 1) * n // world]
    for fn in (column_parallel_linear_sp, overlapped_column_parallel_linear_sp):
        x = x_full[:, sl].clone().requires_grad_(True)
        w = w_col.clone().requires_grad_(True)
        y = fn(x, w, None)
        assert torch.allclose(y, x_full @ w_col.T), fn.__name__
        y.backward(go_full)
        assert torch.allclose(w.grad, go_full.flatten(0, 1).T @ x_full.flatten(0, 1)), fn.__name__
        dx = go_full @ w_col                                    # this rank's partial; the shard gets the sum over ranks
        dist.all_reduce(dx)
        assert torch.allclose(x.grad, dx[:, sl]), fn.__name__
    # row parallel: every rank multiplies its input slice, the sum is scattered along the sequence
    k = 4
    xr_all = [torch.randn(b, s, k, dtype=torch.float64) for _ in range(world)]
    wr_all = [torch.randn(h, k, dtype=torch.float64) for _ in range(world)]
    add_all = [torch.randn(b, s, h, dtype=torch.float64) for _ in range(world)]
    want = sum(xr @ wr.T + a for xr, wr, a in zip(xr_all, wr_all, add_all))[:, sl]
    xr = xr_all[rank].clone().requires_grad_(True)
    wr = wr_all[rank].clone().requires_grad_(True)
    add = add_all[rank].clone().requires_grad_(True)
    y = overlapped_row_parallel_linear_sp(xr, wr, add)
    assert torch.allclose(y, want)
    go = torch.randn(b, s, h, dtype=torch.float64)              # same on every rank (same seed)
    y.backward(go[:, sl])
    assert torch.allclose(xr.grad, go @ wr_all[rank]) and torch.allclose(add.grad, go)
    assert torch.allclose(wr.grad, go.flatten(0, 1).T @ xr_all[rank].flatten(0, 1))
    y2 = OverlappedRowParallelLinearSP.apply(xr_all[rank], wr_all[rank], None)
    assert torch.allclose(y2, sum(a @ c.T for a, c in zip(xr_all, wr_all))[:, sl])


def test_functional_sequence_parallel_linears():
    run_distributed(_sp_functional_worker, 2)


def _exchange_helpers_worker(rank, world):
    """Ring and arbitrary-peer pipeline exchanges, and the asynchronous differentiable all-to-all."""
    from picotron_b200 import process_group_manager as pgm
    from picotron.expert_parallel.ep_communications import all_to_all_async
    from picotron.pipeline_parallel.pp_communications import (interleaved_pipeline_communicate,
                                                              vshape_pipeline_communicate)
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=world, dp_size=1)
    dev, shape = torch.device("cpu"), (2, 3)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    fwd = torch.full(shape, 10.0 + rank)
    bwd = torch.full(shape, 20.0 + rank)
    got_f, got_b = interleaved_pipeline_communicate(dev, torch.float32, shape, send_forward_tensor=fwd,
                                                    send_backward_tensor=bwd, recv_forward=True, recv_backward=True)
    assert got_f.requires_grad and torch.equal(got_f.detach(), torch.full(shape, 10.0 + prv))
    assert torch.equal(got_b.detach(), torch.full(shape, 20.0 + nxt))
    only_f, none_b = interleaved_pipeline_communicate(dev, torch.float32, shape, send_forward_tensor=fwd, recv_forward=True)
    assert none_b is None and torch.equal(only_f.detach(), torch.full(shape, 10.0 + prv))
    # every rank sends two keyed tensors to every other rank
    sends = [(key, torch.full(shape, 100.0 * rank + 10 * peer + key), peer) for peer in range(world) if peer != rank
             for key in (1, 0)]
    recvs = [(key, peer) for peer in range(world) if peer != rank for key in (0, 1)]
    if world == 2:
        got = vshape_pipeline_communicate(dev, torch.float32, shape, sends, recvs)
        peer = 1 - rank
        assert sorted(got) == [0, 1]
        for key in (0, 1):
            assert torch.equal(got[key].detach(), torch.full(shape, 100.0 * peer + 10 * rank + key))
    assert vshape_pipeline_communicate(dev, torch.float32, shape, [], []) == {}
    # all-to-all: rank r sends r + 1 rows to every rank
    rows = rank + 1
    x = (torch.arange(world * rows * 2, dtype=torch.float64).view(world * rows, 2) + 1000 * rank).requires_grad_(True)
    out, work = all_to_all_async(x, [p + 1 for p in range(world)], [rows] * world, dist.group.WORLD)
    work.wait()
    assert out.shape[0] == sum(p + 1 for p in range(world))
    lo = 0
    for p in range(world):
        want = torch.arange(world * (p + 1) * 2, dtype=torch.float64).view(world * (p + 1), 2) + 1000 * p
        assert torch.equal(out.detach()[lo:lo + p + 1], want[rank * (p + 1):(rank + 1) * (p + 1)])
        lo += p + 1
    (out * (rank + 1)).sum().backward()                          # the gradient returns scaled by the receiver's factor
    for p in range(world):
        assert torch.equal(x.grad[p * rows:(p + 1) * rows], torch.full((rows, 2), float(p + 1), dtype=torch.float64))


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_exchange_helpers_and_async_all_to_all(world):
    run_distributed(_exchange_helpers_worker, world)


def test_call_signatures_accept_the_reference_parameter_names():
    """Parameter names of the reference's public entry points (read off its sources), so that calls by
    keyword keep working. ``capacity_moe.capacity_moe`` is the one deliberate exception: here it takes the
    layer instead of the reference's thirteen loose arguments."""
    import importlib
    import inspect
    table = {
        "picotron.model.FinalProjection": ["hidden_size", "vocab_size", "bias"],
        "picotron.model.Embedding": ["num_embeddings", "embedding_dim", "padding_idx"],
        "picotron.model.TritonRMSNorm": ["hidden_size", "eps", "device", "dtype"],
        "picotron.utils.get_mfu": ["tokens_per_second", "num_params", "model_config", "theoretical_flops"],
        "picotron.tensor_parallel.tensor_parallel.ColumnParallelLinear":
            ["in_features", "out_features", "bias", "gather_output", "async_all_reduce", "sequence_parallel",
             "overlap_comm", "ptb"],
        "picotron.tensor_parallel.tensor_parallel.RowParallelLinear":
            ["in_features", "out_features", "bias", "sequence_parallel", "overlap_comm", "ptb"],
        "picotron.tensor_parallel.tensor_parallel.VocabParallelEmbedding":
            ["num_embeddings", "embedding_dim", "padding_idx", "max_norm", "norm_type", "scale_grad_by_freq", "sparse",
             "sequence_parallel"],
        "picotron.tensor_parallel.tensor_parallel.apply_tensor_parallel":
            ["model", "async_tp", "sequence_parallel", "vocab_parallel_ce", "overlap_comm"],
        "picotron.context_parallel.ulysses.ulysses_attention": ["q", "k", "v", "causal"],
        "picotron.context_parallel.context_parallel.ring_attention": ["q", "k", "v", "sm_scale", "is_causal"],
        "picotron.context_parallel.context_parallel.update_out_and_lse": ["out", "lse", "block_out", "block_lse", "slice_"],
        "picotron.expert_parallel.capacity_moe.compute_capacity": ["num_tokens", "top_k", "num_experts", "capacity_factor"],
        "picotron.expert_parallel.ep_communications.all_to_all": ["x", "output_split_sizes", "input_split_sizes", "group"],
        "picotron.expert_parallel.ep_communications.all_to_all_fp8": ["x", "output_split_sizes", "input_split_sizes", "group"],
        "picotron.expert_parallel.ep_communications.all_to_all_no_grad_async":
            ["x", "output_split_sizes", "input_split_sizes", "group"],
        "picotron.expert_parallel.ep_communications.all_to_all_async":
            ["x", "output_split_sizes", "input_split_sizes", "group"],
        "picotron.sequence_parallel.sequence_parallel.column_parallel_linear_sp": ["x", "weight", "bias"],
        "picotron.sequence_parallel.overlap.overlapped_row_parallel_linear_sp": ["x", "weight", "addend"],
        "picotron.sequence_parallel.overlap.ring_all_gather_matmul": ["x_shard", "weight"],
        "picotron.sequence_parallel.overlap.pipelined_matmul_reduce_scatter": ["x_full", "weight", "addend_full"],
        "picotron.tensor_parallel.tp_communications.linear_with_all_reduce": ["x", "weight", "bias"],
        "picotron.tensor_parallel.tp_communications.linear_with_async_all_reduce": ["x", "weight", "bias"],
        "picotron.tensor_parallel.tp_communications.vocab_parallel_cross_entropy": ["vocab_parallel_logits", "target"],
        "picotron.expert_parallel.ep_communications.exchange_split_sizes": ["input_split_sizes", "group"],
        "picotron.pipeline_parallel.pp_communications.interleaved_pipeline_communicate":
            ["device", "dtype", "shapes", "send_forward_tensor", "send_backward_tensor", "recv_forward", "recv_backward"],
        "picotron.pipeline_parallel.pp_communications.vshape_pipeline_communicate":
            ["device", "dtype", "shape", "sends", "recvs"],
        "picotron.expert_parallel.megakernel.fused_moe":
            ["x_sorted", "counts", "gate_w", "up_w", "down_w", "row_weight"],
    }
    wrong = []
    for path, names in table.items():
        mod, _, attr = path.rpartition(".")
        params = inspect.signature(getattr(importlib.import_module(mod), attr)).parameters
        wrong += [f"{path}: {n}" for n in names if n not in params]
    assert not wrong, wrong


def test_class_members_named_by_the_reference():
    """Attributes and methods that reference scripts reach for on the grid manager, the pipeline stage
    wrapper, the ZeRO wrapper, the loader and the checkpoint initialiser."""
    from types import SimpleNamespace
    from picotron.checkpoint import InitializationManager
    from picotron.data import MicroBatchDataLoader
    from picotron.data_parallel.zero import DataParallelZero
    from picotron.pipeline_parallel.pipeline_parallel import PipelineParallel
    from picotron.process_group_manager import ProcessGroupManager
    m = ProcessGroupManager(1, 1, 1, 1, 1, create_groups=False)
    assert tuple(m.grid.shape) == (1, 1, 1, 1, 1) and int(m.grid.flatten()[0]) == 0
    for cls, names in ((PipelineParallel, ("distribute_layers", "backward", "backward_input", "backward_weight")),
                       (DataParallelZero, ("no_sync", "full_parameters")),
                       (MicroBatchDataLoader, ("collate_batch", "tokenizer_group_text", "tokenize_dataset")),
                       (InitializationManager, ("add_missing_params_as_zeros", "get_layer_names_in_sft_format"))):
        assert all(hasattr(cls, n) for n in names), (cls.__name__, names)

    class Tok:                                     # 'a b c' -> [1, 2, 3]
        def batch_encode_plus(self, texts, **kw):
            return {"input_ids": [[ord(ch) - 96 for ch in t.split()] for t in texts]}

    rows = MicroBatchDataLoader.tokenizer_group_text(["a b c d", "e f g"], Tok(), 3)["input_ids"]
    assert rows == [[1, 2, 3, 4], [4, 5, 6, 7]]                     # rows of 3 + 1 tokens sharing their boundary token
    assert MicroBatchDataLoader.tokenizer_group_text(["a b c"], Tok(), 3)["input_ids"] == []

    class Data:
        column_names = ["text"]

        def map(self, fn, input_columns, remove_columns, batched, num_proc, desc):
            assert input_columns == "text" and remove_columns == ["text"] and batched
            return fn(["a b c d e f g"])

    loader = MicroBatchDataLoader(micro_batch_size=2, seq_length=3, dataset_name="synthetic", vocab_size=32,
                                  num_samples=8, pin_memory=False)
    loader.tokenizer = Tok()
    assert loader.tokenize_dataset(Data(), "text", 3, 1)["input_ids"] == [[1, 2, 3, 4], [4, 5, 6, 7]]
    batch = loader.collate_batch([{"input_ids": [1, 2, 3, 4]}, {"input_ids": [4, 5, 6, 7]}])
    assert batch["input_ids"].tolist() == [[1, 2, 3], [4, 5, 6]] and batch["target_ids"].tolist() == [[2, 3, 4], [5, 6, 7]]
    assert batch["position_ids"].tolist() == [[0, 1, 2], [0, 1, 2]] and batch["hidden_states"] is None

    model = torch.nn.Linear(3, 2)
    sd = {"weight": torch.ones(2, 3)}
    InitializationManager(model, SimpleNamespace(num_experts=1), tp_rank=0, tp_world_size=1).add_missing_params_as_zeros(sd)
    assert set(sd) == {"weight", "bias"} and sd["bias"].abs().sum() == 0 and sd["weight"].sum() == 6


def _pp_split_backward_worker(rank, world):
    """``backward_input`` + ``backward_weight`` of a stage wrapper give what ``backward`` gives: the input
    gradient at once, the weight gradients of the linears when the queue is drained."""
    import types
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.models.llama import Llama
    from picotron_b200.ops import gemm as gemm_ops
    from picotron.pipeline_parallel.pipeline_parallel import PipelineParallel
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=world, dp_size=1)
    cfg = types.SimpleNamespace(hidden_size=32, num_attention_heads=4, num_key_value_heads=2, intermediate_size=64,
                                vocab_size=64, num_hidden_layers=2, max_position_embeddings=16, rms_norm_eps=1e-5,
                                rope_theta=10000.0, parallel_block=False)
    torch.manual_seed(0)
    stage = PipelineParallel(Llama(cfg), cfg)
    assert stage.distribute_layers(5) == [0, 1, 2, 3, 4]
    ids = torch.randint(0, 64, (2, 8))
    grads = {}
    for split in (False, True):
        stage.zero_grad()
        gemm_ops.set_zero_bubble(split)
        try:
            out = stage(input_ids=ids)
            go = torch.ones_like(out) / out.numel()
            if split:
                stage.backward_input(None, out, go)
                lin = stage.decoder_layers["0"].mlp.down_proj.weight
                assert lin.grad is None, "a linear's weight gradient must wait for the W pass"
                stage.backward_weight()
            else:
                stage.backward(None, out, go)
        finally:
            gemm_ops.set_zero_bubble(False)
        grads[split] = {n: p.grad.clone() for n, p in stage.named_parameters()}
    for n in grads[False]:
        assert torch.allclose(grads[True][n], grads[False][n], atol=1e-6), n
    # the multi-chunk wrappers answer the reference's questions about their chunks
    from picotron.pipeline_parallel.pp_schedules import InterleavedPipelineParallel, VShapePipelineParallel
    cfg4 = types.SimpleNamespace(**{**vars(cfg), "num_hidden_layers": 4})
    torch.manual_seed(0)
    inter = InterleavedPipelineParallel(Llama(cfg4), cfg4, num_virtual_stages=2)
    assert inter.chunk_global_id == [0, 1] and inter.num_global_stages == 2
    assert inter.is_first_stage(0) and not inter.is_first_stage(1) and inter.is_last_stage(1)
    hidden = inter(input_ids=ids, chunk_id=0)
    assert hidden.shape == (2, 8, 32) and inter(hidden_states=hidden, chunk_id=1).shape == (2, 8, 64)
    vee = VShapePipelineParallel(Llama(cfg4), cfg4)
    assert vee.dev(0) == 0 and vee.dev(1) == 0 and vee.is_first(0) and vee.is_last(1) and not vee.is_last(0)
    assert vee(1, hidden_states=vee(0, input_ids=ids)).shape == (2, 8, 64)


def test_pipeline_stage_split_backward():
    run_distributed(_pp_split_backward_worker, 1)


def test_the_reference_template_config_is_accepted():
    """A config file written for the reference (its ``template/base_config.json``, where a copy of the
    reference is at hand) validates here unchanged: this framework's schema is a superset."""
    import json
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    root = os.environ.get("PICOTRON_REFERENCE_ROOT", os.path.join(os.path.dirname(repo), "reference"))
    path = os.path.join(root, "template", "base_config.json")
    if not os.path.exists(path):
        pytest.skip("no copy of the reference on this machine")
    from picotron_b200.config import load_config
    theirs = json.load(open(path))
    ours = load_config(theirs)
    for section, keys in theirs.items():
        assert section in ours and not set(keys) - set(ours[section]), section
        assert all(ours[section][k] == v for k, v in keys.items() if v is not None), section
