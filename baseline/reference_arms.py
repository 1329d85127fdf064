"""Reference arms of ``bench.py`` for the configurations other than the headline one.

Every function here drives the *unmodified* reference package (installed under ``baseline/_ref``,
imported as ``picotron``) through its own public API and stock code paths; nothing of
``picotron_b200`` (models, kernels, engine) is on these paths. Each builder returns a dict

    device_step()   one optimizer step on micro-batches already resident on the GPU
    e2e_step()      the same step with every micro-batch copied from pinned host memory and the
                    loss read back to the host; returns the loss
    tokens_per_step, h2d_bytes_per_step, d2h_bytes_per_step, parallelism (label)

The step loops follow the reference's own drivers: ``tests/bench_ep_train_step.py`` (MoE train
step), ``tests/bench_cp.py`` (ring / Ulysses step) and ``tests/bench_pp_schedules.py`` (pipeline
schedules, fake loader protocol), plus the optimizer step and gradient synchronisation its
``train.py`` performs. Where the reference's trainer has no wiring for a layout (different tokens
per expert-parallel rank; gradients averaged over the context-parallel group when dp = 1) the
harness adds the one collective that makes the step a correct training step, using the reference's
own ``DataParallelBucket`` where it applies and one flat all-reduce otherwise.
"""
from __future__ import annotations

import os
import types

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _namespace(model: dict, seq: int, **extra):
    keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "vocab_size", "rms_norm_eps", "rope_theta")
    ns = types.SimpleNamespace(**{k: model[k] for k in keys}, max_position_embeddings=seq, num_experts=1,
                               num_experts_per_tok=1, num_shared_experts=0, norm_topk_prob=True)
    for k, v in extra.items():
        setattr(ns, k, v)
    return ns


def _init_like_ours(model):
    """N(0, 0.02) for every matrix, as the other arm (norm weights stay 1)."""
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.02)


def _env():
    os.environ["FLASH_ATTEN"] = "1"
    os.environ["DEVICE"] = "cuda"
    os.environ["DTYPE"] = "bfloat16"


def _flat_all_reduce(params, group, divide_by: float):
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    dist.all_reduce(flat, group=group)
    flat.div_(divide_by)
    for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(f)


class _HostBatches:
    """Seeded token batches in pinned host memory, shaped like the reference's collate output."""

    def __init__(self, vocab: int, mbs: int, seq: int, seed: int):
        self.g = torch.Generator().manual_seed(seed)
        self.vocab, self.mbs, self.seq = vocab, mbs, seq

    def next(self):
        rows = torch.randint(0, self.vocab, (self.mbs, self.seq + 1), generator=self.g)
        return rows[:, :-1].contiguous().pin_memory(), rows[:, 1:].contiguous().pin_memory()


# ------------------------------------------------------------------------------------------- MoE
def build_moe(spec: dict, device, world: int):
    """DeepSeek-style MoE Llama with expert parallelism over all ``world`` ranks, every rank on its
    own tokens: the reference's ``Llama`` + ``MoELayer`` (its Triton grouped-expert kernels on CUDA),
    aux loss via ``collect_aux_loss``, AdamW; the non-expert gradients are averaged over the
    expert-parallel group with one flat all-reduce and expert gradients divided by its size."""
    _env()
    import picotron.process_group_manager as rpgm
    from picotron.expert_parallel.expert_parallel import collect_aux_loss
    from picotron.model import Llama
    rpgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=world)
    pg = rpgm.process_group_manager
    m = spec["model"]
    shared = m.get("shared_expert_intermediate_size") or 0
    cfg = _namespace(m, spec["seq"], num_experts=m["num_experts"], num_experts_per_tok=m["num_experts_per_tok"],
                     num_shared_experts=(shared // m["intermediate_size"]) if shared else m.get("num_shared_experts", 0),
                     norm_topk_prob=True, ep_overlap=True, ep_num_tiles=m.get("ep_num_tiles", 1),
                     ep_fp8_dispatch=m.get("ep_fp8_dispatch", False), moe_latent_dim=0, ep_backend="torch",
                     ep_capacity_factor=m.get("ep_capacity_factor", 0.0),
                     ep_capacity_dropless=m.get("ep_capacity_dropless", True), ep_max_rounds=8,
                     router_aux_loss_coef=m.get("router_aux_loss_coef", 0.0),
                     router_bias_update_rate=m.get("router_bias_update_rate", 0.0))
    torch.manual_seed(1234)
    with torch.device(device):
        model = Llama(cfg)
    _init_like_ours(model)
    model.to(torch.bfloat16).to(device).train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=spec["lr"])
    dense = [p for n, p in model.named_parameters() if ".local_experts." not in n]
    experts = [p for n, p in model.named_parameters() if ".local_experts." in n]
    mbs, seq, ga, vocab = spec["mbs"], spec["seq"], spec["grad_acc"], m["vocab_size"]
    host = _HostBatches(vocab, mbs, seq, seed=99 + pg.ep_rank)
    resident = [tuple(t.to(device) for t in host.next()) for _ in range(ga)]

    def micro(inp, tgt):
        logits = model(input_ids=inp)
        loss = F.cross_entropy(logits.view(-1, logits.size(-1)).float(), tgt.reshape(-1)) / ga
        aux = collect_aux_loss(model)
        total = loss + aux / ga if aux is not None else loss
        total.backward()
        return loss

    def finish():
        if world > 1:
            _flat_all_reduce(dense, pg.ep_group, float(world))
            for p in experts:                      # every rank's tokens reached the expert through the dispatch
                if p.grad is not None:
                    p.grad.div_(world)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)

    def device_step():
        for inp, tgt in resident:
            micro(inp, tgt)
        finish()

    def e2e_step():
        acc = 0.0
        for _ in range(ga):
            inp, tgt = host.next()
            acc += micro(inp.to(device, non_blocking=True), tgt.to(device, non_blocking=True)).item()
        finish()
        return acc

    return dict(device_step=device_step, e2e_step=e2e_step, tokens_per_step=mbs * seq * ga * world,
                h2d_bytes_per_step=ga * 2 * mbs * seq * 8, d2h_bytes_per_step=ga * 4,
                parallelism=f"ep{world} (ep ranks on different tokens)")


# -------------------------------------------------------------------------------------------- CP
def build_cp(spec: dict, device, world: int):
    """Long-context Llama with the sequence sharded over all ranks (contiguous shards as in the
    reference's data loader): ``apply_context_parallel`` + ``CP_ATTENTION`` = ring | ulysses, flash
    attention for the blocks, ``DataParallelBucket`` for the gradient average over the CP group,
    AdamW."""
    _env()
    import picotron.process_group_manager as rpgm
    from picotron.context_parallel.context_parallel import apply_context_parallel
    from picotron.data_parallel.data_parallel import DataParallelBucket
    from picotron.model import Llama
    rpgm.setup_process_group_manager(tp_size=1, cp_size=world, pp_size=1, dp_size=1)
    pg = rpgm.process_group_manager
    m = spec["model"]
    seq, mbs, vocab = spec["seq"], spec["mbs"], m["vocab_size"]
    s_local = seq // world
    cfg = _namespace(m, seq)
    os.environ["CP_ATTENTION"] = spec["cp_attention"]
    torch.manual_seed(1234)
    with torch.device(device):
        model = Llama(cfg)
    _init_like_ours(model)
    model = apply_context_parallel(model)
    model.to(torch.bfloat16).to(device).train()
    dp_model = DataParallelBucket(model) if world > 1 else model
    optimizer = torch.optim.AdamW(model.parameters(), lr=spec["lr"])
    host = _HostBatches(vocab, mbs, seq, seed=99)            # the same sequence on every CP rank
    lo, hi = pg.cp_rank * s_local, (pg.cp_rank + 1) * s_local

    def shard(t):
        return t[:, lo:hi].contiguous()

    inp0, tgt0 = host.next()
    resident = (shard(inp0).to(device), shard(tgt0).to(device))

    def micro(inp, tgt):
        logits = dp_model(input_ids=inp)
        loss = F.cross_entropy(logits.reshape(mbs * s_local, -1).float(), tgt.reshape(-1))
        loss.backward()
        return loss

    def finish():
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        if world > 1:
            dp_model.reset()

    def device_step():
        micro(*resident)
        finish()

    def e2e_step():
        inp, tgt = host.next()
        loss = micro(shard(inp).pin_memory().to(device, non_blocking=True),
                     shard(tgt).pin_memory().to(device, non_blocking=True)).item()
        finish()
        return loss

    return dict(device_step=device_step, e2e_step=e2e_step, tokens_per_step=mbs * seq,
                h2d_bytes_per_step=2 * mbs * s_local * 8, d2h_bytes_per_step=4,
                parallelism=f"cp{world} {spec['cp_attention']}")


# -------------------------------------------------------------------------------------------- PP
class _Loader:
    """The loader protocol of the reference's pipeline schedules (tests/test_pipeline_parallel.py:43-69):
    ``grad_acc_steps``, ``seq_length_per_gpu``, ``micro_batch_size`` and ``__next__`` returning the
    collate dict. ``source`` yields (input_ids, target_ids) per micro-batch."""

    def __init__(self, source, grad_acc: int, mbs: int, seq: int):
        self.source, self.grad_acc_steps, self.micro_batch_size, self.seq_length_per_gpu = source, grad_acc, mbs, seq
        self.pos = torch.arange(seq).unsqueeze(0).repeat(mbs, 1)

    def __iter__(self):
        return self

    def __next__(self):
        inp, tgt = self.source()
        return {"input_ids": inp, "target_ids": tgt, "position_ids": self.pos, "hidden_states": None}


def build_pp(spec: dict, device, world: int):
    """Llama-2-7B-shaped model on TP x PP x DP with the reference's tensor-parallel layers
    (``apply_tensor_parallel`` as its trainer calls it), its pipeline stage wrappers and schedule
    functions (interleaved 1F1B with 2 virtual stages, zero-bubble, 1F1B, AFAB),
    ``DataParallelBucket`` and AdamW."""
    _env()
    import picotron.process_group_manager as rpgm
    from picotron.data_parallel.data_parallel import DataParallelBucket
    from picotron.model import Llama
    from picotron.pipeline_parallel.pipeline_parallel import (PipelineParallel, train_step_pipeline_1f1b,
                                                              train_step_pipeline_afab)
    from picotron.pipeline_parallel.pp_schedules import (InterleavedPipelineParallel, train_step_pipeline_interleaved,
                                                         train_step_pipeline_zb)
    from picotron.tensor_parallel.tensor_parallel import apply_tensor_parallel
    tp, pp, dp = spec["tp"], spec["pp"], spec["dp"]
    assert tp * pp * dp == world
    rpgm.setup_process_group_manager(tp_size=tp, cp_size=1, pp_size=pp, dp_size=dp)
    pg = rpgm.process_group_manager
    m = spec["model"]
    seq, mbs, ga, vocab = spec["seq"], spec["mbs"], spec["grad_acc"], m["vocab_size"]
    cfg = _namespace(m, seq)
    engine = spec["pp_engine"]
    torch.manual_seed(1234)
    with torch.device(device):
        model = Llama(cfg)
        if tp > 1:
            model = apply_tensor_parallel(model)
    _init_like_ours(model)
    if pp > 1:
        model = InterleavedPipelineParallel(model, cfg, num_virtual_stages=2) if engine == "interleaved" \
            else PipelineParallel(model, cfg)
    model.to(torch.bfloat16).to(device).train()
    dp_model = DataParallelBucket(model) if dp > 1 else model
    optimizer = torch.optim.AdamW(model.parameters(), lr=spec["lr"])
    fn = {"interleaved": train_step_pipeline_interleaved, "zb": train_step_pipeline_zb,
          "1f1b": train_step_pipeline_1f1b, "afab": train_step_pipeline_afab}[engine]
    shapes = (mbs, seq, m["hidden_size"])
    host = _HostBatches(vocab, mbs, seq, seed=99 + pg.dp_rank)
    resident = [tuple(t.to(device) for t in host.next()) for _ in range(ga)]
    cursor = {"i": 0}

    def from_resident():
        b = resident[cursor["i"] % ga]
        cursor["i"] += 1
        return b

    def from_host():
        inp, tgt = host.next()
        return inp.to(device, non_blocking=True), tgt.to(device, non_blocking=True)

    loaders = {"device": _Loader(from_resident, ga, mbs, seq), "e2e": _Loader(from_host, ga, mbs, seq)}
    for ld in loaders.values():
        ld.pos = ld.pos.to(device)

    def step(kind):
        cursor["i"] = 0
        if pp > 1:
            loss = fn(dp_model, loaders[kind], shapes, device, torch.bfloat16)
        else:
            loss = 0.0
            for i in range(ga):
                if dp > 1:
                    dp_model.require_backward_grad_sync = i == ga - 1
                b = next(loaders[kind])
                out = dp_model(input_ids=b["input_ids"])
                l = F.cross_entropy(out.flatten(0, 1).float(), b["target_ids"].flatten()) / ga
                l.backward()
                loss = loss + l.detach()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        if dp > 1:
            dp_model.reset()
        return loss

    def e2e_step():
        loss = step("e2e")
        return float(loss) if not torch.is_tensor(loss) else float(loss.item())

    return dict(device_step=lambda: step("device"), e2e_step=e2e_step, tokens_per_step=mbs * seq * ga * dp,
                h2d_bytes_per_step=ga * 2 * mbs * seq * 8, d2h_bytes_per_step=4,
                parallelism=f"tp{tp}xpp{pp}xdp{dp} {engine}")
