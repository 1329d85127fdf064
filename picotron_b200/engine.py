"""Training engine: builds the parallel model from a config and runs optimizer steps.

This is the programmatic form of ``train.py`` (and what ``bench.py`` times): topology ->
model -> tensor / pipeline / context / data parallel wrappers -> optimizer -> ``train_step``.
It follows the order of the reference trainer (train.py:254-289: TP, then PP, then CP, then
dtype/device, then DP) and wires in what the reference leaves as library code: sequence
parallelism, vocabulary-parallel cross entropy, ZeRO, interleaved 1F1B and ZB-V.

Two gradient paths exist, split by device exactly like the ops:

* CUDA/bf16 ("flat" path): parameters and fp32 gradients live in one flat buffer each
  (``ParamStore``); weight-gradient GEMMs accumulate into it, the data-parallel reduction is a
  reduce-scatter (ZeRO-1) or all-reduce of that buffer and AdamW is one kernel over this rank's
  shard followed by an all-gather of the updated parameters.
* CPU/fp32 (plumbing path, gloo): ordinary autograd ``.grad`` with the ``DataParallelBucket`` /
  ``DataParallelZero`` wrappers and ``torch.optim.AdamW``, as the reference does.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.distributed as dist

from . import process_group_manager as pgm
from .config import load_config, model_config_from
from .data import MicroBatchDataLoader
from .models.llama import Llama
from .ops import adamw as adamw_ops
from .ops import cross_entropy as ce_ops
from .param_store import ParamStore
from .parallel.dist_utils import group_rank, group_size


def _dtype_of(cfg, device) -> torch.dtype:
    if device.type != "cuda" or cfg["distributed"]["use_cpu"]:
        return torch.float32
    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg["model"].get("dtype", "bfloat16")]


def loss_fn(model, logits, targets, divisor: float = 1.0) -> torch.Tensor:
    """Mean token loss (divided by ``divisor``, the number of micro-batches) from the model output:
    dense logits, or vocabulary-sharded logits when the lm head keeps them sharded
    (``vocab_parallel_ce``). ``backward()`` must be called on the result (or a sum containing it)."""
    if getattr(model, "vocab_parallel_ce", False) and group_size(getattr(model, "tp_group", None)) > 1:
        g = model.tp_group
        start = group_rank(g) * logits.shape[-1]
        return ce_ops.mean_cross_entropy(logits, targets, vocab_start=start, group=g, divisor=divisor)
    return ce_ops.mean_cross_entropy(logits, targets, divisor=divisor)


class FlatOptimizer:
    """AdamW on the flat buffers of a ParamStore, optionally sharded over a data-parallel group
    (ZeRO-1: reduce-scatter gradients, update the local shard, all-gather parameters)."""

    def __init__(self, store: ParamStore, lr, weight_decay=0.01, betas=(0.9, 0.999), eps=1e-8, dp_group=None,
                 zero_stage: int = 0, sp_grad_params=None, tp_group=None, fused=None, extra_grad_scale: float = 1.0):
        """``fused``: (SymmGroup, params SymmBuffer, grads SymmBuffer) selects the kernel that does the
        gradient reduce-scatter, the sharded AdamW update and the parameter all-gather in one launch
        over NVLink peer memory; otherwise the two collectives are NCCL calls around the AdamW kernel."""
        self.store, self.dp_group, self.zero_stage = store, dp_group, zero_stage
        self.fused = fused
        self.extra_grad_scale = extra_grad_scale
        self.dp_size = group_size(dp_group)
        self.dp_rank = group_rank(dp_group)
        self.sp_grad_params = list(sp_grad_params or [])
        self.tp_group = tp_group
        n = store.numel
        if self.zero_stage >= 1 and self.dp_size > 1:
            assert n % self.dp_size == 0
            shard = n // self.dp_size
            lo = self.dp_rank * shard
            self.shard_params = store.flat_params[lo:lo + shard]
            self.shard_grads = store.flat_grads[lo:lo + shard]
        else:
            self.shard_params, self.shard_grads = store.flat_params, store.flat_grads
        self.adam = adamw_ops.FlatAdamW(self.shard_params, self.shard_grads, lr=lr, betas=betas, eps=eps,
                                        weight_decay=weight_decay)

    def reduce_sequence_parallel_grads(self):
        """Norm weights see only a sequence shard under sequence parallelism: sum their gradients
        over the TP group (the reference does this only in its tests,
        tests/test_tp_sequence_parallel.py:151-152)."""
        if not self.sp_grad_params or group_size(self.tp_group) == 1:
            return
        flat = torch.cat([p.main_grad.reshape(-1) for p in self.sp_grad_params])
        dist.all_reduce(flat, group=self.tp_group)
        off = 0
        for p in self.sp_grad_params:
            p.main_grad.copy_(flat[off:off + p.numel()].view_as(p.main_grad))
            off += p.numel()

    READY_SLOT, DONE_SLOT = 10, 11

    def _fused_step(self, grad_scale: float):
        from .ops import count_launch, ext
        sg, pbuf, gbuf = self.fused
        a = self.adam
        a.step_count += 1
        b1, b2 = a.betas
        shard = self.store.numel // self.dp_size
        ready = sg.next_epoch(self.READY_SLOT)
        sg.signal(self.READY_SLOT, ready)                      # my gradients are final
        ext().zero1_adamw(gbuf.ptrs, pbuf.ptrs, a.exp_avg, a.exp_avg_sq, a.master, self.dp_rank * shard, shard,
                          self.dp_size, self.dp_rank, a.lr, b1, b2, a.eps, a.weight_decay,
                          1.0 - b1 ** a.step_count, 1.0 - b2 ** a.step_count, grad_scale / self.dp_size,
                          sg.flags.local_ptr, self.READY_SLOT, ready, 60000)
        count_launch()
        done = sg.next_epoch(self.DONE_SLOT)
        sg.signal(self.DONE_SLOT, done)                        # my shard is written everywhere
        sg.wait(self.DONE_SLOT, done, 60000)                   # ... and so is everyone else's
        self.store.flat_grads.zero_()

    def step(self, grad_scale: float = 1.0):
        grad_scale = grad_scale * self.extra_grad_scale
        self.reduce_sequence_parallel_grads()
        st = self.store
        if self.fused is not None and self.dp_size > 1 and self.zero_stage >= 1:
            self._fused_step(grad_scale)
            return
        if self.dp_size > 1:
            if self.zero_stage >= 1:
                dist.reduce_scatter_tensor(self.shard_grads, st.flat_grads, group=self.dp_group)
            else:
                dist.all_reduce(st.flat_grads, group=self.dp_group)
        self.adam.step(grad_scale=grad_scale / self.dp_size, zero_grad=False)
        st.flat_grads.zero_()
        if self.dp_size > 1 and self.zero_stage >= 1:
            dist.all_gather_into_tensor(st.flat_params, self.shard_params, group=self.dp_group)

    def zero_grad(self):
        self.store.flat_grads.zero_()

    def state_dict(self):
        return self.adam.state_dict()

    def load_state_dict(self, sd):
        self.adam.load_state_dict(sd)


class MultiFlatOptimizer:
    """Several flat optimizers stepped together (dense and expert parameters reduce over different
    groups when expert parallelism doubles as data parallelism)."""

    def __init__(self, parts):
        self.parts = list(parts)
        self.zero_stage = self.parts[0].zero_stage
        self.dp_size = self.parts[0].dp_size

    def step(self, grad_scale: float = 1.0):
        for p in self.parts:
            p.step(grad_scale)

    def zero_grad(self):
        for p in self.parts:
            p.zero_grad()

    def state_dict(self):
        return {"parts": [p.state_dict() for p in self.parts]}

    def load_state_dict(self, sd):
        for p, s in zip(self.parts, sd["parts"]):
            p.load_state_dict(s)


class TrainEngine:
    def __init__(self, cfg, device: Optional[torch.device] = None):
        cfg = load_config(cfg)
        self.cfg = cfg
        d, t = cfg["distributed"], cfg["training"]
        if device is None:
            device = torch.device("cpu") if d["use_cpu"] or not torch.cuda.is_available() \
                else torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.dtype = _dtype_of(cfg, device)
        m = pgm.process_group_manager
        if m is None or (m.tp_world_size, m.cp_world_size, m.pp_world_size, m.dp_world_size, m.ep_world_size) != \
                (d["tp_size"], d["cp_size"], d["pp_size"], d["dp_size"], d["ep_size"]):
            m = pgm.setup_process_group_manager(d["tp_size"], d["cp_size"], d["pp_size"], d["dp_size"], d["ep_size"])
        self.pgm = m
        self.model_config = model_config_from(cfg)
        torch.manual_seed(t["seed"])
        self.data_loader = MicroBatchDataLoader(
            micro_batch_size=t["micro_batch_size"], seq_length=t["seq_length"], dataset_name=cfg["dataset"]["name"],
            tokenizer_name=cfg["model"]["name"], grad_acc_steps=t["gradient_accumulation_steps"],
            num_samples=t["num_samples"], vocab_size=self.model_config.vocab_size, seed=t["seed"],
            subset_name=cfg["dataset"].get("subset_name"), split=cfg["dataset"].get("split", "train"),
            num_proc=cfg["dataset"].get("num_proc", 1),
            dp_world_size=m.dp_world_size * (m.ep_world_size if d["ep_as_dp"] else 1),
            dp_rank=m.dp_rank * (m.ep_world_size if d["ep_as_dp"] else 1) + (m.ep_rank if d["ep_as_dp"] else 0),
            cp_zigzag=bool(d.get("cp_zigzag", False)) and d["cp_attention"] == "ring")
        self.tokens_per_step = self.data_loader.global_batch_size * t["seq_length"]
        self._build_model()
        self._build_optimizer()
        self.trained_steps = 0
        self.trained_tokens = 0
        #: optional ``runtime.timing.EventTimer``: when set, every step records the device time of its
        #: sections ("micro_batches" = forward + backward of all micro-batches, or "forward" /
        #: "backward" separately on the eager path, and "optimizer" = gradient reduction + update +
        #: parameter gather); ``timer.collect()`` returns the milliseconds, MAX over ranks
        self.timer = None

    def _section(self, name: str):
        return self.timer.section(name) if self.timer is not None else contextlib.nullcontext()

    # ------------------------------------------------------------------------------ build
    def _build_model(self):
        from .parallel.tensor_parallel import apply_tensor_parallel
        d = self.cfg["distributed"]
        m = self.pgm
        build_device = self.device if self.device.type == "cuda" else torch.device("cpu")
        with torch.device(build_device):
            model = Llama(self.model_config)
        if m.tp_world_size > 1:
            with torch.device(build_device):
                apply_tensor_parallel(model, async_tp=d["async_tp"], sequence_parallel=d["sequence_parallel"],
                                      vocab_parallel_ce=d["vocab_parallel_ce"], overlap_comm=d["overlap_comm"])
        if m.pp_world_size > 1:
            from .parallel.pipeline_parallel import wrap_pipeline
            model = wrap_pipeline(model, self.model_config, d["pp_engine"], d["num_virtual_stages"])
        if m.cp_world_size > 1:
            from .parallel.context_parallel import apply_context_parallel
            apply_context_parallel(model, attention=d["cp_attention"], seq_length=self.cfg["training"]["seq_length"],
                                   zigzag=bool(d.get("cp_zigzag", False)) and d["cp_attention"] == "ring")
        # (re-)initialise in canonical module order from the configured seed: tensor-parallel
        # layers draw the full master weight and keep their slice, so a TP run starts from
        # exactly the weights of the single-device run (reference: checkpoint.py:114-119)
        torch.manual_seed(self.cfg["training"]["seed"])
        with torch.no_grad():
            model.reset_parameters()
        model.to(self.dtype).to(self.device)
        self.model = model
        self.flat = self.device.type == "cuda" and self.dtype == torch.bfloat16 and self._flat_wanted()
        self._symm_groups = []         # symmetric-memory groups whose kernels run inside a micro-batch
        self._mb_graph = None
        self.dp_symm = None
        allocator = None
        if self.flat and self._use_fused_dp():
            # flat parameters and gradients live in symmetric memory so the optimizer kernel can
            # read every replica's gradients and write every replica's parameters directly
            from .runtime.symm import SymmGroup
            self.dp_symm = SymmGroup(self._grad_group(), device=self.device)
            self._symm_flat = []

            def allocator(numel, dtype):
                buf = self.dp_symm.alloc(numel * torch.tensor([], dtype=dtype).element_size())
                self._symm_flat.append(buf)
                return buf.view(dtype, (numel,))
        self.expert_store = None
        if self.flat and self._split_expert_params():
            is_expert = lambda n, p: ".local_experts." in n      # noqa: E731
            self.store = ParamStore(model, pad_to_multiple=max(1, self._grad_group_size()), allocator=allocator,
                                    param_filter=lambda n, p: not is_expert(n, p))
            self.expert_store = ParamStore(model, pad_to_multiple=max(1, self.pgm.cp_dp_world_size),
                                           param_filter=is_expert)
        else:
            self.store = ParamStore(model, pad_to_multiple=max(1, self._grad_group_size()),
                                    allocator=allocator) if self.flat else None
        self._maybe_install_fused_ep()
        self.fused_tp = None
        self._maybe_install_fused_tp()
        self._maybe_install_fused_cp()

    def _flat_wanted(self) -> bool:
        """``training.flat_params``. The flat buffers keep every gradient and parameter whole on every
        rank (the optimizer kernel shards the state and the update), so ZeRO stages 2 and 3, whose
        point is to hold only a shard of them, default to the per-parameter path of
        ``parallel/zero.py`` (picotron/data_parallel/zero.py:102-176)."""
        want = self.cfg["training"].get("flat_params")
        stage = self.cfg["distributed"]["zero_stage"]
        if want is None:
            return stage < 2
        if want and stage >= 2 and self.pgm.global_rank == 0:
            print(f"zero_stage={stage} on flat parameters: the optimizer state is sharded, gradients and "
                  "parameters stay whole on every rank (set training.flat_params=false for sharded ones)", flush=True)
        return bool(want)

    def _maybe_install_fused_cp(self):
        """Context parallelism through NVLink peer memory on the flat bf16 path: ring attention gathers
        K/V and reduces dK/dV with ``ops.fused_cp``, Ulysses does its all-to-alls with
        ``ops.fused_ulysses``; ``PICO_FUSED_CP=0`` keeps the NCCL point-to-point ring / all-to-all."""
        import os
        from .parallel import context_parallel as cpar
        d, t, m, mc = self.cfg["distributed"], self.cfg["training"], self.pgm, self.model_config
        from .parallel import ulysses as uly
        self.fused_cp = None
        cpar.install_fused_cp(None)
        uly.install_fused_ulysses(None)
        if not (self.flat and m.cp_world_size > 1 and os.environ.get("PICO_FUSED_CP", "1") != "0"):
            return
        from .runtime.symm import SymmGroup
        head_dim = mc.hidden_size // mc.num_attention_heads
        kv_heads = mc.num_key_value_heads // m.tp_world_size
        q_heads = mc.num_attention_heads // m.tp_world_size
        if head_dim not in (64, 128) or kv_heads < 1:
            return
        s_local = t["seq_length"] // m.cp_world_size
        sg = SymmGroup(m.cp_group, device=self.device)
        self._symm_groups.append(sg)
        if d["cp_attention"] == "ring":
            from .ops.fused_cp import CPFused
            self.fused_cp = CPFused(sg, t["micro_batch_size"], s_local, kv_heads * head_dim)
            cpar.install_fused_cp(self.fused_cp)
        elif q_heads % m.cp_world_size == 0:
            from .ops.fused_ulysses import UlyssesFused
            self.fused_cp = UlyssesFused(sg, t["micro_batch_size"], s_local, q_heads * head_dim)
            uly.install_fused_ulysses(self.fused_cp)

    def _split_expert_params(self) -> bool:
        return (self.cfg["distributed"]["ep_as_dp"] and self.pgm.ep_world_size > 1
                and getattr(self.model_config, "num_experts", 1) > 1)

    def _maybe_install_fused_ep(self):
        """Capacity-mode MoE layers exchange rows through NVLink peer memory (``ops.fused_ep``) on the
        flat bf16 path; ``PICO_FUSED_EP=0`` keeps the NCCL all-to-alls."""
        import os
        mc, m, t = self.model_config, self.pgm, self.cfg["training"]
        self.fused_ep = None
        if not (self.flat and m.ep_world_size > 1 and getattr(mc, "num_experts", 1) > 1
                and os.environ.get("PICO_FUSED_EP", "1") != "0"):
            return
        from .ops.fused_ep import EPFused
        from .parallel.capacity_moe import compute_capacity
        from .parallel.expert_parallel import MoELayer
        from .runtime.symm import SymmGroup
        tokens = t["micro_batch_size"] * (t["seq_length"] // m.cp_world_size)
        if self.cfg["distributed"]["sequence_parallel"] and m.tp_world_size > 1:
            tokens //= m.tp_world_size
        if (getattr(mc, "ep_capacity_factor", 0.0) or 0.0) <= 0:
            # dropless: ``ep_backend`` "fused" (or "deepep", whose role it takes here) selects the
            # peer-memory exchange with the layout computed on the device
            if getattr(mc, "ep_backend", "torch") not in ("fused", "deepep"):
                return
            from .ops.fused_ep_var import EPVarFused
            layers = [mod for mod in self.model.modules() if isinstance(mod, MoELayer)]
            if not layers or layers[0].expert_dim % 128 != 0:
                return
            sg = SymmGroup(m.ep_group, device=self.device)
            self._symm_groups.append(sg)
            # rows one rank may receive, as a multiple of the balanced load: an untrained router is
            # skewed (single experts at 3-5x, groups of 8 experts at up to ~1.7x the mean were measured)
            # ``ep_var_slack`` 0 = the worst case (every row of every rank routed to one rank: ep_size times
            # the balanced load), with which the overflow cannot happen; the buffers then take
            # 2 x ep_size x tokens x top_k x dim x 2 bytes (1.6 GB at 8192 tokens, top-6, dim 2048, EP 8)
            slack = os.environ.get("PICO_EP_VAR_SLACK", getattr(mc, "ep_var_slack", 3.0))
            slack = 3.0 if slack is None else float(slack)
            if slack <= 0:
                slack = float(m.ep_world_size)
            self.fused_ep = EPVarFused(sg, layers[0].num_local_experts, layers[0].expert_dim,
                                       tokens * mc.num_experts_per_tok, slack=min(slack, float(m.ep_world_size)),
                                       fp8_dispatch=bool(getattr(mc, "ep_fp8_dispatch", False)))
            for mod in layers:
                mod.fused_ep_var = self.fused_ep
            return
        cap = compute_capacity(tokens, mc.num_experts_per_tok, mc.num_experts, mc.ep_capacity_factor)
        layers = [mod for mod in self.model.modules() if isinstance(mod, MoELayer)]
        if not layers or layers[0].expert_dim % 8 != 0:
            return
        sg = SymmGroup(m.ep_group, device=self.device)
        self._symm_groups.append(sg)
        self.fused_ep = EPFused(sg, layers[0].num_local_experts, cap, layers[0].expert_dim)
        for mod in layers:
            mod.fused_ep = self.fused_ep

    def _maybe_install_fused_tp(self):
        """Switch the sequence-parallel linears to the kernels that carry their collectives through
        NVLink peer memory (``ops.fused_tp``). Needs the flat bf16 path, TP > 1 with sequence
        parallelism, and a micro-batch whose per-rank token count is a multiple of the GEMM tile;
        ``PICO_FUSED_TP=0`` keeps the NCCL collectives."""
        import os
        d, t, m = self.cfg["distributed"], self.cfg["training"], self.pgm
        ce_ops.install_peer_exchange(m.tp_group, None)
        if not (self.flat and m.tp_world_size > 1 and d["sequence_parallel"] and not d["overlap_comm"]):
            return
        if os.environ.get("PICO_FUSED_TP", "1") == "0":
            return
        from .ops.fused_tp import TPFused
        from .parallel.tensor_parallel import install_fused_tp
        from .runtime.symm import SymmGroup
        s_local = t["seq_length"] // m.cp_world_size // m.tp_world_size
        m_local = t["micro_batch_size"] * s_local
        if not TPFused.usable(m_local, s_local):
            return
        sg = SymmGroup(m.tp_group, device=self.device)
        self._symm_groups.append(sg)
        self.fused_tp = TPFused(sg, m_local, self.model_config.hidden_size, s_local)
        install_fused_tp(self.model, self.fused_tp)
        # one micro-batch in flight at a time: gathered inputs can stay in place for the backward pass
        self.fused_tp.keep_gathered = m.pp_world_size == 1 and os.environ.get("PICO_TP_KEEP_GATHERED", "1") != "0"
        ce_ops.install_peer_exchange(m.tp_group, self.fused_tp.ce_exchange)

    def _use_fused_dp(self) -> bool:
        """ZeRO-1 through the peer-memory optimizer kernel (``csrc/fused/dp_zero.cu``): needs the
        flat bf16 path, a gradient-reduction group of 2..8 GPUs and zero_stage >= 1;
        ``PICO_FUSED_DP=0`` keeps the NCCL reduce-scatter / all-gather."""
        import os
        n = self._grad_group_size()
        return (self.cfg["distributed"]["zero_stage"] >= 1 and 1 < n <= 8
                and os.environ.get("PICO_FUSED_DP", "1") != "0")

    def _grad_group(self):
        m = self.pgm
        if self.cfg["distributed"]["ep_as_dp"] and m.ep_world_size > 1:
            return m.dense_dp_group
        return m.cp_dp_group

    def _grad_group_size(self):
        m = self.pgm
        n = m.cp_dp_world_size
        if self.cfg["distributed"]["ep_as_dp"]:
            n *= m.ep_world_size
        return n

    def _build_optimizer(self):
        t, d = self.cfg["training"], self.cfg["distributed"]
        m = self.pgm
        if self.flat:
            sp_params = [p for p in self.model.parameters() if getattr(p, "sequence_parallel_grad", False)]
            self.optimizer = FlatOptimizer(self.store, lr=t["learning_rate"], weight_decay=t["weight_decay"],
                                           dp_group=self._grad_group() if self._grad_group_size() > 1 else None,
                                           zero_stage=d["zero_stage"], sp_grad_params=sp_params,
                                           tp_group=m.tp_group,
                                           fused=(self.dp_symm, self._symm_flat[0], self._symm_flat[1])
                                           if self.dp_symm is not None else None)
            if self.expert_store is not None:
                experts = FlatOptimizer(self.expert_store, lr=t["learning_rate"], weight_decay=t["weight_decay"],
                                        dp_group=m.cp_dp_group if m.cp_dp_world_size > 1 else None,
                                        zero_stage=d["zero_stage"], extra_grad_scale=1.0 / m.ep_world_size)
                self.optimizer = MultiFlatOptimizer([self.optimizer, experts])
            self.dp_model = self.model
            return
        from .parallel.data_parallel import DataParallelBucket, DataParallelExpertAware, DataParallelNaive
        from .parallel.zero import DataParallelZero, ShardedOptimizer
        self.dp_model = self.model
        if self._split_expert_params():
            self.dp_model = DataParallelExpertAware(self.model, m.dense_dp_group, m.cp_dp_group)
        elif self._grad_group_size() > 1:
            if d["zero_stage"] >= 1 or d["dp_engine"] == "zero":
                self.dp_model = DataParallelZero(self.model, stage=max(1, d["zero_stage"]), group=self._grad_group())
                self.optimizer = ShardedOptimizer(self.dp_model, torch.optim.AdamW, lr=t["learning_rate"],
                                                  weight_decay=t["weight_decay"])
                return
            cls = DataParallelNaive if d["dp_engine"] == "naive" else DataParallelBucket
            self.dp_model = cls(self.model, group=self._grad_group())
        self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=t["learning_rate"],
                                           weight_decay=t["weight_decay"])

    # ------------------------------------------------------------------------------ step
    def _sync_context(self, last: bool):
        dp = self.dp_model
        if hasattr(dp, "require_backward_grad_sync"):
            dp.require_backward_grad_sync = last
        return contextlib.nullcontext()

    def train_step(self, device_batches=None) -> torch.Tensor:
        """One optimizer step over ``gradient_accumulation_steps`` micro-batches. Returns the mean
        loss as a 0-d tensor on the device (no host sync).

        ``device_batches``: optional list of ``(input_ids, target_ids)`` already on the device,
        one per micro-batch, used instead of the data loader (kernel-only timing)."""
        m = self.pgm
        dl = self.data_loader
        ga = dl.grad_acc_steps
        if m.pp_world_size > 1:
            from .parallel.pipeline_parallel import run_pipeline_step
            with self._section("micro_batches"):
                loss = run_pipeline_step(self, device_batches)
        elif self._graph_wanted():
            with self._section("micro_batches"):
                loss = self._graphed_micro_batches(device_batches)
        else:
            loss = torch.zeros((), device=self.device, dtype=torch.float32)
            for i in range(ga):
                if device_batches is not None:
                    input_ids, target_ids = device_batches[i]
                else:
                    batch = next(dl)
                    input_ids = batch["input_ids"].to(self.device, non_blocking=True)
                    target_ids = batch["target_ids"].to(self.device, non_blocking=True)
                self._sync_context(i == ga - 1)
                loss += self._micro_batch(input_ids, target_ids, ga)
        with self._section("optimizer"):
            self._optimizer_step()
        self.trained_steps += 1
        self.trained_tokens += self.tokens_per_step
        return loss

    def _micro_batch(self, input_ids, target_ids, ga: int) -> torch.Tensor:
        """Forward + backward of one micro-batch; gradients accumulate; returns its detached loss / ga."""
        timed = self.timer is not None and not (self.device.type == "cuda"
                                                and torch.cuda.is_current_stream_capturing())
        if self.fused_tp is not None:
            self.fused_tp.begin_micro_batch()
        with (self.timer.section("forward") if timed else contextlib.nullcontext()):
            logits = self.dp_model(input_ids=input_ids)
            mb_loss = loss_fn(self.model, logits, target_ids, divisor=ga)
            aux = self._aux_loss()
            total = mb_loss + aux / ga if aux is not None else mb_loss
        with (self.timer.section("backward") if timed else contextlib.nullcontext()):
            total.backward()
        return mb_loss.detach().float()

    # ------------------------------------------------------------------------------ CUDA graph
    def _graph_wanted(self) -> bool:
        """The micro-batch (forward + backward) is replayed from a CUDA graph on the flat bf16 path:
        its few hundred to few thousand launches then cost the host one call, which is what keeps
        small per-rank kernels (tensor parallelism over 4 GPUs and more) from being bound by launch
        overhead. ``training.cuda_graph: false`` or ``PICO_CUDA_GRAPH=0`` keeps eager launches; so do
        the paths that synchronise with the host inside a micro-batch (tiled / NCCL expert exchange,
        NCCL context parallelism, the hook-based data-parallel wrappers)."""
        import os
        if self._mb_graph is False:
            return False
        if self._mb_graph is not None:
            return True
        t, m, mc = self.cfg["training"], self.pgm, self.model_config
        from .ops import reference_ops_forced
        ok = self.flat and t.get("cuda_graph", True) and os.environ.get("PICO_CUDA_GRAPH", "1") != "0" \
            and not reference_ops_forced()
        if ok and getattr(mc, "num_experts", 1) > 1:
            ok = self._moe_graph_safe()
        if ok and m.cp_world_size > 1:
            # ring attention on zigzag shards runs the step-by-step NCCL ring: no collective library
            # call is ever captured
            d = self.cfg["distributed"]
            zigzag = bool(d.get("cp_zigzag", False)) and d["cp_attention"] == "ring"
            ok = self.fused_cp is not None and not zigzag
        if ok and m.tp_world_size > 1:
            ok = self.fused_tp is not None
        if not ok:
            self._mb_graph = False
        return ok

    def _moe_graph_safe(self) -> bool:
        """Mixture-of-experts layers can be captured on the paths whose routing and exchange never read
        a device value on the host and never call a collective: capacity-limited dispatch
        (``MoELayer._forward_device_routed``) and the dropless exchange laid out on the device
        (``MoELayer._routed_fused_var``), both through the peer-memory kernels, with the expert-load sum
        of the bias controller through peer memory too. ``PICO_MOE_GRAPH=0`` keeps eager launches."""
        import os
        from .ops.fused_ep import EPFused
        from .ops.fused_ep_var import EPVarFused
        from .parallel.expert_parallel import MoELayer
        if os.environ.get("PICO_MOE_GRAPH", "1") == "0" or os.environ.get("PICO_MOE_DEVICE_ROUTING", "1") == "0":
            return False
        if self.fused_ep is None or self.pgm.pp_world_size > 1 or self.pgm.tp_world_size > 1:
            return False
        layers = [mod for mod in self.model.modules() if isinstance(mod, MoELayer)]
        if not layers or any(mod.num_experts > 256 or mod.num_experts % 4 or mod.top_k > 8 for mod in layers):
            return False
        if isinstance(self.fused_ep, EPFused):
            return all(mod.fused_ep is self.fused_ep and mod.ep_capacity_factor > 0 and not mod.ep_capacity_dropless
                       for mod in layers)
        if isinstance(self.fused_ep, EPVarFused):
            return all(mod.fused_ep_var is self.fused_ep and mod.ep_capacity_factor <= 0 for mod in layers)
        return False

    def _graphed_micro_batches(self, device_batches) -> torch.Tensor:
        from . import ops
        dl = self.data_loader
        ga = dl.grad_acc_steps
        if self._mb_graph is None and self.trained_steps < 1:
            # first step eagerly: lazily created buffers (scratch, tables, counters) must exist
            # before a capture, which may not allocate outside its pool
            loss = torch.zeros((), device=self.device, dtype=torch.float32)
            for i in range(ga):
                inp, tgt = self._fetch(device_batches, i)
                loss += self._micro_batch(inp.to(self.device, non_blocking=True),
                                          tgt.to(self.device, non_blocking=True), ga)
            return loss
        if self._mb_graph is None:
            self._capture_micro_batch(ga)
        g = self._mb_graph
        g["loss"].zero_()
        for i in range(ga):
            inp, tgt = self._fetch(device_batches, i)
            g["input_ids"].copy_(inp, non_blocking=True)
            g["target_ids"].copy_(tgt, non_blocking=True)
            for rec in g["epochs"]:
                rec.before_replay()
            g["graph"].replay()
            for rec in g["epochs"]:
                rec.after_replay()
            ops.count_launch(g["launches"])
        return g["loss"].clone()

    def _fetch(self, device_batches, i):
        """Micro-batch i of this step: the caller's device tensors, or the next (pinned host) batch
        of the data loader."""
        if device_batches is not None:
            return device_batches[i]
        batch = next(self.data_loader)
        return batch["input_ids"], batch["target_ids"]

    def _capture_micro_batch(self, ga: int):
        from . import ops
        dl = self.data_loader
        shape = (dl.micro_batch_size, dl.seq_length_per_gpu)
        inp = torch.zeros(shape, dtype=torch.long, device=self.device)
        tgt = torch.zeros(shape, dtype=torch.long, device=self.device)
        loss = torch.zeros((), device=self.device, dtype=torch.float32)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        l0 = ops.launches()
        # thread-local capture mode: the process group's watchdog thread may query its events while
        # this thread captures
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            for sg in self._symm_groups:
                sg.begin_graph()
                sg.barrier()
            loss.add_(self._micro_batch(inp, tgt, ga))
            if self.fused_tp is not None:
                self.fused_tp.join()          # side-stream pushes rejoin the captured stream
            recs = []
            for sg in self._symm_groups:
                sg.barrier()
                recs.append(sg.end_graph())
        launches = ops.launches() - l0
        ops.count_launch(-launches)          # a capture launches nothing
        # The fused paths alternate between two copies of each buffer, which is safe while a rank
        # is never two operations ahead of a peer. The group barriers at both ends of the graph
        # keep that true across replays and across eager launches around them, whichever copy
        # comes first.
        self._mb_graph = {"graph": graph, "input_ids": inp, "target_ids": tgt, "loss": loss, "epochs": recs,
                          "launches": launches}

    def close(self):
        """Release the symmetric-memory buffers (peer mappings and this rank's allocations). Collective
        over each group; the engine must not be used afterwards."""
        self._mb_graph = False
        if torch.cuda.is_available() and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        groups = list(self._symm_groups)
        if self.dp_symm is not None:
            groups.append(self.dp_symm)
        for sg in groups:
            sg.close()
        self._symm_groups = []

    @property
    def optimizer_is_sharded(self) -> bool:
        """True when each data-parallel rank holds a different slice of the optimizer state."""
        if self.flat:
            return self.optimizer.zero_stage >= 1 and self.optimizer.dp_size > 1
        return hasattr(self.optimizer, "dp")

    def average_loss(self, loss) -> float:
        """Mean of the step loss over the ranks that computed it on different data (CP x DP, and
        EP when it acts as data parallelism); other ranks receive the value of the last pipeline
        stage's replica group. One host read."""
        t = loss.detach().float().reshape(1).clone() if torch.is_tensor(loss) else \
            torch.tensor([float(loss)], device=self.device)
        n = self._grad_group_size()
        if n > 1 and self.pgm.pp_is_last_stage:
            dist.all_reduce(t, group=self._grad_group())
            t /= n
        return float(t.item())

    def _aux_loss(self):
        if getattr(self.model_config, "num_experts", 1) > 1:
            from .parallel.expert_parallel import collect_aux_loss
            return collect_aux_loss(self.model)
        return None

    def _optimizer_step(self):
        if self.flat:
            self.optimizer.step()
        else:
            self.optimizer.step()
            self.optimizer.zero_grad()
            if hasattr(self.dp_model, "reset"):
                self.dp_model.reset()
