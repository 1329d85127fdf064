"""Pipeline-parallel stage wrappers and the schedule executor.

Wrappers (names and layer placement as in the reference):
* ``PipelineParallel(model, config)`` — one contiguous block of layers per rank; embedding on
  the first stage, final norm + lm head on the last, ``decoder_layers`` keyed by *global* layer
  index so checkpoints keep the reference's names (pipeline_parallel.py:87-143)
* ``InterleavedPipelineParallel(model, config, num_virtual_stages=2)`` — chunk c of rank r is
  global stage ``c*p + r`` (pp_schedules.py:160-207)
* ``VShapePipelineParallel(model, config)`` — rank r owns global stages r and 2p-1-r
  (pp_schedules.py:384-428)

All three are the same class with a different stage map. ``run_schedule`` executes any plan
from ``pp_schedules`` on such a wrapper: forward/backward per (chunk, micro-batch), loss (and
MoE auxiliary loss) on whichever stage produces it, deferred weight gradients for the
zero-bubble schedules, and one batched P2P group per round.

``train_step_pipeline_afab`` / ``train_step_pipeline_1f1b`` keep the reference signature.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn

from .. import process_group_manager as pgm
from ..ops import gemm as gemm_ops
from . import pp_schedules as sched
from .pp_communications import RoundCommunicator


def distribute_layers(num_layers: int, num_stages: int) -> List[List[int]]:
    """Contiguous split, the remainder going to the earliest stages (pipeline_parallel.py:57-69)."""
    base, extra = divmod(num_layers, num_stages)
    out, start = [], 0
    for s in range(num_stages):
        n = base + (1 if s < extra else 0)
        out.append(list(range(start, start + n)))
        start += n
    return out


def pp_autograd_backward(input_tensor, output_tensor, output_tensor_grad, extra_tensors=(), extra_grads=()):
    """Backward of one stage; returns the gradient w.r.t. the stage input (None on stage 0)."""
    if input_tensor is not None and input_tensor.requires_grad:
        input_tensor.retain_grad()
    if output_tensor_grad is None:
        output_tensor_grad = torch.ones_like(output_tensor, memory_format=torch.preserve_format)
    torch.autograd.backward([output_tensor, *extra_tensors], grad_tensors=[output_tensor_grad, *extra_grads])
    return input_tensor.grad if input_tensor is not None else None


class PipelineParallel(nn.Module):
    """This rank's share of a Llama: the layers of its stage(s) plus embedding / head where due."""

    def __init__(self, model, config, stage_map: Optional[sched.StageMap] = None, pp_rank: Optional[int] = None,
                 pp_size: Optional[int] = None):
        super().__init__()
        m = pgm.get_pgm()
        self.pp_rank = m.pp_rank if pp_rank is None else pp_rank
        self.pp_size = m.pp_world_size if pp_size is None else pp_size
        self.stage_map = stage_map or sched.StageMap(self.pp_size, 1)
        smap = self.stage_map
        per_stage = distribute_layers(config.num_hidden_layers, smap.num_stages)
        self.stages = [smap.stage_of(self.pp_rank, c) for c in range(smap.v)]
        self.chunk_layers = [per_stage[s] for s in self.stages]
        self.layer_distribution = [i for chunk in self.chunk_layers for i in chunk]
        self.has_first = 0 in self.stages
        self.has_last = (smap.num_stages - 1) in self.stages
        self.embedding = model.embedding if self.has_first else nn.Identity()
        self.decoder_layers = nn.ModuleDict({str(i): model.decoder_layers[i] for i in self.layer_distribution})
        self.final_norm = model.final_norm if self.has_last else nn.Identity()
        self.final_proj = model.final_proj if self.has_last else nn.Identity()
        self.rope = model.rope
        self.config = config
        self.sequence_parallel = getattr(model, "sequence_parallel", False)
        self.vocab_parallel_ce = getattr(model, "vocab_parallel_ce", False)
        self.tp_group = getattr(model, "tp_group", None)

    def decoder_layers_iter(self):
        return iter(self.decoder_layers.values())

    def reset_parameters(self):
        for mod in (self.embedding, self.final_norm, self.final_proj):
            if not isinstance(mod, nn.Identity):
                mod.reset_parameters()
        for layer in self.decoder_layers.values():
            layer.reset_parameters()

    def forward_chunk(self, chunk: int, input_ids=None, hidden_states=None):
        stage = self.stages[chunk]
        x = self.embedding(input_ids) if stage == 0 else hidden_states
        for i in self.chunk_layers[chunk]:
            x = self.decoder_layers[str(i)](x, self.rope)
        if stage == self.stage_map.num_stages - 1:
            from ..models.llama import lm_head
            x = lm_head(self, x)
        return x

    def forward(self, input_ids=None, position_ids=None, hidden_states=None):
        assert self.stage_map.v == 1, "multi-chunk wrappers are driven through forward_chunk"
        return self.forward_chunk(0, input_ids=input_ids, hidden_states=hidden_states)

    def backward(self, input_tensor, output_tensor, output_tensor_grad):
        return pp_autograd_backward(input_tensor, output_tensor, output_tensor_grad)

    def distribute_layers(self, num_layers: int) -> List[int]:
        """Layer indices of this rank's contiguous stage (the reference's method, pipeline_parallel.py:123-127)."""
        m = pgm.get_pgm()
        return distribute_layers(num_layers, m.pp_world_size)[m.pp_rank]

    # Zero-bubble split for callers that drive a stage by hand (the executor does the same per action):
    # B = input gradient now, weight-gradient GEMMs queued; W = run one micro-batch's queue. On the CPU
    # restatement the forward pass must have run under ``ops.gemm.set_zero_bubble(True)`` for its linears
    # to be deferrable; otherwise B computes everything and W finds an empty queue.
    def backward_input(self, input_tensor, output_tensor, output_tensor_grad):
        with gemm_ops.defer_wgrad() as queue:
            grad_in = pp_autograd_backward(input_tensor, output_tensor, output_tensor_grad)
        self.__dict__.setdefault("_zb_pending", []).append(list(queue))
        return grad_in

    def backward_weight(self, output_tensor=None, output_tensor_grad=None):
        gemm_ops.run_deferred(self.__dict__["_zb_pending"].pop(0))


class InterleavedPipelineParallel(PipelineParallel):
    def __init__(self, model, config, num_virtual_stages: int = 2, **kw):
        m = pgm.get_pgm()
        p = kw.get("pp_size") or m.pp_world_size
        super().__init__(model, config, stage_map=sched.StageMap(p, num_virtual_stages), **kw)
        self.num_virtual_stages = num_virtual_stages
        self.num_global_stages = self.stage_map.num_stages
        #: global stage of each local chunk (chunk c of rank r is stage c * p + r)
        self.chunk_global_id = list(self.stages)

    def is_first_stage(self, chunk_id: int) -> bool:
        return self.stages[chunk_id] == 0

    def is_last_stage(self, chunk_id: int) -> bool:
        return self.stages[chunk_id] == self.stage_map.num_stages - 1

    def forward(self, input_ids=None, position_ids=None, hidden_states=None, chunk_id: int = 0):
        """One local chunk (the reference's call: ``forward(input_ids, position_ids, hidden_states, chunk_id)``)."""
        return self.forward_chunk(chunk_id, input_ids=input_ids, hidden_states=hidden_states)


class VShapePipelineParallel(PipelineParallel):
    def __init__(self, model, config, **kw):
        m = pgm.get_pgm()
        p = kw.get("pp_size") or m.pp_world_size
        super().__init__(model, config, stage_map=sched.StageMap(p, 2, vshape=True), **kw)
        self.p = p
        self.num_global_stages = self.stage_map.num_stages

    def dev(self, g: int) -> int:
        """Pipeline rank that hosts global stage ``g``: ``g`` on the way down, ``2p - 1 - g`` on the way up."""
        return self.stage_map.rank_of(g)

    def is_first(self, g: int) -> bool:
        return g == 0

    def is_last(self, g: int) -> bool:
        return g == self.stage_map.num_stages - 1

    def forward(self, gid=None, input_ids=None, position_ids=None, hidden_states=None):
        """One of this rank's two stages by its global id (the reference's call: ``forward(gid, input_ids,
        position_ids, hidden_states)``)."""
        gid = self.stages[0] if gid is None else gid
        return self.forward_chunk(self.stages.index(gid), input_ids=input_ids, hidden_states=hidden_states)


def wrap_pipeline(model, config, engine: str, num_virtual_stages: int = 2):
    if engine == "interleaved":
        return InterleavedPipelineParallel(model, config, num_virtual_stages)
    if engine == "zbv":
        return VShapePipelineParallel(model, config)
    return PipelineParallel(model, config)


# ------------------------------------------------------------------------------------------
# executor
# ------------------------------------------------------------------------------------------
_PLAN_CACHE: Dict[tuple, tuple] = {}


def _unwrap(model):
    return model.module if hasattr(model, "module") and isinstance(model.module, PipelineParallel) else model


def run_schedule(engine: str, model, data_loader, tensor_shapes, device, dtype, device_batches=None,
                 loss_function=None):
    """One optimizer step's worth of micro-batches through the pipeline. Returns the summed
    (already 1/m-scaled) loss as a 0-d tensor on the last stage's device (zero elsewhere)."""
    from ..engine import loss_fn as default_loss
    loss_function = loss_function or default_loss
    stage_mod = _unwrap(model)
    m_pg = pgm.get_pgm()
    p, rank = stage_mod.pp_size, stage_mod.pp_rank
    m = data_loader.grad_acc_steps
    v = stage_mod.stage_map.v
    key = (engine, p, m, v, stage_mod.stage_map.vshape)
    if key not in _PLAN_CACHE:
        plan, smap, split_w = sched.build_plan(engine, p, m, v)
        assert smap == stage_mod.stage_map, f"pp_engine '{engine}' needs a {smap} wrapper, model has {stage_mod.stage_map}"
        _PLAN_CACHE[key] = (plan, smap, split_w)
    plan, smap, split_w = _PLAN_CACHE[key]
    S = smap.num_stages
    comm = RoundCommunicator(device, dtype)
    batches: Dict[int, dict] = {}

    def batch(i):
        # every rank advances its loader identically so replicas of a DP rank stay in step
        while len(batches) <= i:
            k = len(batches)
            if device_batches is not None:
                batches[k] = {"input_ids": device_batches[k][0], "target_ids": device_batches[k][1]}
            else:
                b = next(data_loader)
                batches[k] = {"input_ids": b["input_ids"].to(device, non_blocking=True),
                              "target_ids": b["target_ids"].to(device, non_blocking=True)}
        return batches[i]

    for i in range(m):
        batch(i)
    has_dp_hooks = hasattr(model, "require_backward_grad_sync")
    my_actions = [a for a in plan.timeline[rank] if a is not None]
    last_b = max(i for i, a in enumerate(my_actions) if a[0] == sched.B)
    if has_dp_hooks:
        model.require_backward_grad_sync = False
    # With one model chunk per rank the hooks reduce gradients during this rank's very last
    # backward. With several chunks (interleaved 1F1B) that last backward belongs to one chunk only;
    # the other chunks finished earlier with synchronisation off, so everything is reduced once at
    # the end instead (as for the schedules that split off weight gradients). The reference turns
    # synchronisation on for the last backward only (pp_schedules.py:347) and leaves the other
    # chunk's gradients un-reduced.
    sync_at_end = split_w or v > 1
    gemm_ops.set_zero_bubble(split_w)
    saved: Dict[tuple, tuple] = {}          # (chunk, mb) -> (input, output, aux)
    local_act: Dict[tuple, torch.Tensor] = {}   # hand-offs between chunks on the same rank
    local_grad: Dict[tuple, torch.Tensor] = {}
    deferred: Dict[tuple, list] = {}
    outgoing: Dict[tuple, torch.Tensor] = {}
    total_loss = torch.zeros((), device=device, dtype=torch.float32)
    n_done = 0
    try:
        for t in range(plan.num_rounds):
            act = plan.timeline[rank][t]
            if act is not None:
                kind, c, i = act
                s = smap.stage_of(rank, c)
                if kind == sched.F:
                    if s == 0:
                        inp = None
                        out = stage_mod.forward_chunk(c, input_ids=batch(i)["input_ids"])
                    else:
                        if smap.rank_of(s - 1) == rank:
                            inp = local_act.pop((s, i))
                        else:
                            inp = comm.take(("act", s, i))
                        inp = inp.detach().requires_grad_(True)
                        out = stage_mod.forward_chunk(c, hidden_states=inp)
                    aux = _collect_aux(stage_mod, c)
                    if s == S - 1:
                        if loss_function is default_loss:
                            out = loss_function(stage_mod, out, batch(i)["target_ids"], divisor=m)
                        else:
                            out = loss_function(stage_mod, out, batch(i)["target_ids"]) / m
                        total_loss += out.detach().float()
                    elif smap.rank_of(s + 1) == rank:
                        local_act[(s + 1, i)] = out
                    else:
                        outgoing[("act", s + 1, i)] = out.detach()
                    saved[(c, i)] = (inp, out, aux)
                elif kind == sched.B:
                    inp, out, aux = saved.pop((c, i))
                    if s == S - 1:
                        grad = None
                    elif smap.rank_of(s + 1) == rank:
                        grad = local_grad.pop((s, i))
                    else:
                        grad = comm.take(("grad", s, i))
                    if has_dp_hooks and not sync_at_end and n_done == last_b:
                        model.require_backward_grad_sync = True
                    extra_t = [aux] if aux is not None else []
                    extra_g = [torch.full_like(aux, 1.0 / m)] if aux is not None else []
                    if split_w:
                        with gemm_ops.defer_wgrad() as q:
                            gin = pp_autograd_backward(inp, out, grad, extra_t, extra_g)
                        deferred[(c, i)] = list(q)
                    else:
                        gin = pp_autograd_backward(inp, out, grad, extra_t, extra_g)
                    if s > 0:
                        if smap.rank_of(s - 1) == rank:
                            local_grad[(s - 1, i)] = gin
                        else:
                            outgoing[("grad", s - 1, i)] = gin
                else:  # W
                    gemm_ops.run_deferred(deferred.pop((c, i)))
                n_done += 1
            comm.post_round(plan.messages[t], rank, m_pg.pp_group_ids, outgoing, tensor_shapes)
        comm.finish()
    finally:
        gemm_ops.set_zero_bubble(False)
    assert not saved and not deferred
    if has_dp_hooks and sync_at_end and hasattr(model, "sync_all"):
        model.sync_all()
    return total_loss


def _collect_aux(stage_mod, chunk):
    if getattr(stage_mod.config, "num_experts", 1) and getattr(stage_mod.config, "num_experts", 1) > 1:
        from .expert_parallel import collect_aux_loss
        layers = [stage_mod.decoder_layers[str(i)] for i in stage_mod.chunk_layers[chunk]]
        return collect_aux_loss(layers)
    return None


def run_pipeline_step(engine, device_batches=None):
    """Pipeline step for ``TrainEngine``: picks the schedule and the P2P tensor shape."""
    cfg = engine.cfg
    t = cfg["training"]
    m = engine.pgm
    s_local = t["seq_length"] // m.cp_world_size
    if cfg["distributed"]["sequence_parallel"] and m.tp_world_size > 1:
        s_local //= m.tp_world_size
    shape = (t["micro_batch_size"], s_local, engine.model_config.hidden_size)
    return run_schedule(cfg["distributed"]["pp_engine"], engine.dp_model, engine.data_loader, shape, engine.device,
                        engine.dtype, device_batches)


def train_step_pipeline_afab(model, data_loader, tensor_shapes, device, dtype):
    return run_schedule("afab", model, data_loader, tensor_shapes, device, dtype)


def train_step_pipeline_1f1b(model, data_loader, tensor_shapes, device, dtype):
    return run_schedule("1f1b", model, data_loader, tensor_shapes, device, dtype)
