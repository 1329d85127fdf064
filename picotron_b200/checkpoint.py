"""Model initialisation helpers and checkpoint save / load.

Checkpoints keep the reference's layout (picotron/checkpoint.py:270-316): directory
``<save_dir>/<step>/``, one file per (tp, pp) coordinate named
``weights_tp_rank_world_size={tp}_{tp_ws}_pp_rank_world_size={pp}_{pp_ws}.pth`` holding a
``torch.save`` dict with keys ``model``, ``optimizer``, ``trained_steps``, ``trained_tokens``;
model keys are the reference's state-dict names (global layer indices under pipeline
parallelism). Only ``dp_rank == 0 and cp_rank == 0`` writes.

Added on top, all ignorable by a reader of the reference format:
* with expert parallelism every EP rank holds different experts, so the file name gets an
  ``_ep_rank_world_size={ep}_{ep_ws}`` suffix and each EP rank writes its own file (the
  reference lets EP ranks overwrite each other)
* files are written to ``*.tmp`` and renamed, and a ``manifest.json`` lists the files a complete
  checkpoint must contain; ``load_checkpoint`` refuses an incomplete one
* extra keys ``rng_state`` and ``data_loader`` allow an exact resume of the data stream
* ZeRO-sharded optimizer state differs on every rank of the gradient-reduction group (data
  parallel x context parallel, and expert parallel when it doubles as data parallelism), so
  each of those ranks writes ``optimizer_dp_rank={dp}_{dp_ws}_cp_rank={cp}_{cp_ws}_<same
  suffix>.pth``; the manifest lists these files too and a load refuses a missing shard or one
  written for another group size

``init_model_with_dematerialized_weights`` / ``init_model_with_materialized_weights`` give the
meta-device construction path of the reference (checkpoint.py:17-121): build without memory,
then materialise and initialise. ``InitializationManager`` locates this rank's tensors in a
directory of Hugging Face safetensors (single file or sharded), cuts out its tensor-parallel
slice and can load it; by default the values are only checked and the model is initialised
randomly, as the reference does (it reads the files but always trains from random init,
checkpoint.py:114-119).
"""
from __future__ import annotations

import contextlib
import json
import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import process_group_manager as pgm
from .utils import assert_no_meta_tensors


@contextlib.contextmanager
def init_model_with_dematerialized_weights(include_buffers: bool = False):
    """Construct modules with their parameters on the meta device (no memory, no init)."""
    with torch.device("meta"):
        yield


def init_model_with_materialized_weights(model: nn.Module, model_config=None, save_dir: Optional[str] = None,
                                         device="cpu", load_pretrained: bool = False):
    """Allocate real storage for a meta-constructed model and initialise it.

    With a directory of Hugging Face safetensors (``save_dir``) this rank's tensors are located in
    the (single-file or sharded) checkpoint, checked against the local parameter shapes and — with
    ``load_pretrained`` — copied in, each rank reading only its own tensor-parallel slice. The
    default keeps the reference's behaviour, which reads the files and then trains from random
    initialisation anyway (checkpoint.py:114-119)."""
    manager = InitializationManager(model, model_config)
    tensors = {}
    if save_dir is not None and os.path.isdir(save_dir) and manager.has_safetensors(save_dir):
        tensors = manager.read_local_tensors(save_dir, load_values=load_pretrained)
    model.to_empty(device=device)
    manager.init_model_parameters()
    if load_pretrained:
        manager.copy_into_model(tensors)
    assert_no_meta_tensors(model)
    return model


class InitializationManager:
    """Maps this rank's parameters to the tensors of a Hugging Face Llama checkpoint and loads them
    (picotron/checkpoint.py:124-267 — ``get_layer_names_in_sft_format``, ``adjust_tensor_size``,
    ``convert_safetensors_to_hf_name`` — re-done on top of the model's own parameter names: a
    pipeline stage holds its layers under their global indices and tensor-parallel layers hold
    their shard, so the wanted names and slices follow from ``named_parameters()`` and the local
    shapes instead of from a separate description of the layout)."""

    _RENAMES = (("decoder_layers.", "model.layers."), ("attention.", "self_attn."), ("out_proj", "o_proj"))
    _TOP_LEVEL = {"embedding.weight": "model.embed_tokens.weight", "final_norm.weight": "model.norm.weight",
                  "final_proj.weight": "lm_head.weight"}

    def __init__(self, model: nn.Module, model_config=None, tp_rank: Optional[int] = None,
                 tp_world_size: Optional[int] = None):
        self.model, self.model_config = model, model_config
        if tp_rank is None or tp_world_size is None:
            m = pgm.process_group_manager
            tp_rank = m.tp_rank if m is not None else 0
            tp_world_size = m.tp_world_size if m is not None else 1
        self.tp_rank, self.tp_world_size = tp_rank, tp_world_size

    def add_missing_params_as_zeros(self, state_dict) -> None:
        """Zero placeholders (fp32) for the model's parameters that ``state_dict`` lacks: what a dense
        checkpoint cannot provide (experts, router, shared expert); ``reset_parameters`` initialises them
        afterwards (picotron/checkpoint.py:132-141)."""
        for name, param in self.model.named_parameters():
            if name not in state_dict:
                state_dict[name] = torch.zeros(param.shape, dtype=torch.float32)

    # ---------------------------------------------------------------------------------- names
    def hf_name(self, param_name: str) -> Optional[str]:
        """Checkpoint name of one of this model's parameters, or None when the dense checkpoint has
        no such tensor (routed experts, router, shared expert, latent projections)."""
        if param_name in self._TOP_LEVEL:
            return self._TOP_LEVEL[param_name]
        if not param_name.startswith("decoder_layers."):
            return None
        moe = getattr(self.model_config, "num_experts", 1) and getattr(self.model_config, "num_experts", 1) > 1
        if ".mlp." in param_name and moe:
            return None
        name = param_name
        for old, new in self._RENAMES:
            name = name.replace(old, new)
        return name

    def get_layer_names_in_sft_format(self):
        """Checkpoint tensor names this rank needs (its pipeline stage's layers; its MoE layers skip
        the dense feed-forward weights)."""
        return [n for n in (self.hf_name(k) for k, _ in self.model.named_parameters()) if n is not None]

    @staticmethod
    def convert_safetensors_to_hf_name(sft_name: str) -> str:
        """Checkpoint tensor name -> this package's parameter name."""
        for ours, theirs in InitializationManager._TOP_LEVEL.items():
            if sft_name == theirs:
                return ours
        name = sft_name
        for ours, theirs in reversed(InitializationManager._RENAMES):
            name = name.replace(theirs, ours)
        return name

    # ---------------------------------------------------------------------------------- files
    @staticmethod
    def has_safetensors(save_dir: str) -> bool:
        return any(f.endswith(".safetensors") for f in os.listdir(save_dir))

    @staticmethod
    def _locate(save_dir: str):
        """{checkpoint tensor name: file} from the shard index, or by listing the files' keys."""
        from safetensors import safe_open
        index_path = os.path.join(save_dir, "model.safetensors.index.json")
        if os.path.exists(index_path):
            with open(index_path) as fh:
                return {k: os.path.join(save_dir, v) for k, v in json.load(fh)["weight_map"].items()}
        where = {}
        for f in sorted(os.listdir(save_dir)):
            if f.endswith(".safetensors"):
                with safe_open(os.path.join(save_dir, f), framework="pt") as fh:
                    for k in fh.keys():
                        where[k] = os.path.join(save_dir, f)
        return where

    def adjust_tensor_size(self, full_shape, local_shape, name: str = ""):
        """Index expression (a tuple of slices) that cuts this rank's shard out of a checkpoint tensor
        of ``full_shape``: the dimension in which the local parameter is ``tp`` times smaller is
        split by rank; a dimension that is merely larger in the checkpoint (the config asked for
        fewer heads or layers' worth of rows) is truncated. Raises if the local shape cannot be
        obtained that way."""
        assert len(full_shape) == len(local_shape), f"{name}: rank mismatch {full_shape} vs {local_shape}"
        out = []
        for full, local in zip(full_shape, local_shape):
            if full == local:
                out.append(slice(0, local))
            elif full == local * self.tp_world_size:
                out.append(slice(self.tp_rank * local, (self.tp_rank + 1) * local))
            elif full > local:
                out.append(slice(0, local))
            else:
                raise ValueError(f"{name}: checkpoint shape {tuple(full_shape)} cannot provide local shape "
                                 f"{tuple(local_shape)} (tp={self.tp_world_size})")
        return tuple(out)

    def read_local_tensors(self, save_dir: str, load_values: bool = True):
        """{parameter name: tensor or None}: every local parameter that has a checkpoint tensor is
        checked against it and, with ``load_values``, this rank's slice of it is read (only the slice
        is read from disk). Parameters without a counterpart (MoE weights, an lm head absent because
        the checkpoint ties it to the embedding) are left out."""
        from safetensors import safe_open
        where = self._locate(save_dir)
        out, handles = {}, {}
        try:
            for pname, p in self.model.named_parameters():
                hf = self.hf_name(pname)
                if hf is None or hf not in where:
                    continue
                path = where[hf]
                if path not in handles:
                    handles[path] = safe_open(path, framework="pt", device="cpu")
                sl = handles[path].get_slice(hf)
                index = self.adjust_tensor_size(tuple(sl.get_shape()), tuple(p.shape), pname)
                out[pname] = sl[index] if load_values else None
        finally:
            for h in handles.values():
                if hasattr(h, "__exit__"):
                    h.__exit__(None, None, None)
        return out

    # ---------------------------------------------------------------------------------- init
    def init_model_parameters(self):
        """Run the initialisers: leaves own them; containers (Attention, MLP, MoELayer, ...) delegate."""
        with torch.no_grad():
            for mod in self.model.modules():
                if hasattr(mod, "reset_parameters") and next(mod.children(), None) is None:
                    mod.reset_parameters()
            for _, buf in self.model.named_buffers():
                buf.zero_()

    def copy_into_model(self, tensors) -> int:
        """Copy the loaded slices into the parameters (in place: they may be views of a flat buffer).
        Returns the number of parameters filled."""
        n = 0
        params = dict(self.model.named_parameters())
        with torch.no_grad():
            for name, t in tensors.items():
                if t is not None:
                    params[name].copy_(t.to(params[name].dtype))
                    n += 1
        return n


class CheckpointManager:
    def __init__(self):
        m = pgm.get_pgm()
        self.tp_rank, self.tp_ws = m.tp_rank, m.tp_world_size
        self.pp_rank, self.pp_ws = m.pp_rank, m.pp_world_size
        self.ep_rank, self.ep_ws = m.ep_rank, m.ep_world_size
        self.dp_rank, self.dp_ws = m.dp_rank, m.dp_world_size
        self.cp_rank, self.cp_ws = m.cp_rank, m.cp_world_size
        self.cp_dp_world_size = m.cp_dp_world_size

    def _suffix_of(self, tp: int, pp: int, ep: int) -> str:
        s = f"tp_rank_world_size={tp}_{self.tp_ws}_pp_rank_world_size={pp}_{self.pp_ws}"
        if self.ep_ws > 1:
            s += f"_ep_rank_world_size={ep}_{self.ep_ws}"
        return s

    def _suffix(self) -> str:
        return self._suffix_of(self.tp_rank, self.pp_rank, self.ep_rank)

    def _get_checkpoint_path(self, out_dir: str) -> str:
        return os.path.join(out_dir, f"weights_{self._suffix()}.pth")

    def _shard_name(self, dp: int, cp: int, suffix: str) -> str:
        return f"optimizer_dp_rank={dp}_{self.dp_ws}_cp_rank={cp}_{self.cp_ws}_{suffix}.pth"

    def _optimizer_shard_path(self, out_dir: str) -> str:
        return os.path.join(out_dir, self._shard_name(self.dp_rank, self.cp_rank, self._suffix()))

    def expected_files(self, sharded_optimizer: bool = False):
        """Every file of a complete checkpoint: one weights file per (tp, pp, ep) coordinate and,
        with a sharded optimizer, one optimizer shard per rank of the whole grid."""
        names = []
        for tp in range(self.tp_ws):
            for pp in range(self.pp_ws):
                for ep in range(self.ep_ws):
                    s = self._suffix_of(tp, pp, ep)
                    names.append(f"weights_{s}.pth")
                    if sharded_optimizer:
                        names += [self._shard_name(dp, cp, s) for dp in range(self.dp_ws) for cp in range(self.cp_ws)]
        return names

    @staticmethod
    def _unwrap(model):
        return model.module if hasattr(model, "module") and isinstance(model.module, nn.Module) else model

    @staticmethod
    def _atomic_save(obj, path):
        tmp = path + ".tmp"
        torch.save(obj, tmp)
        os.replace(tmp, path)

    def save_checkpoint(self, model, optimizer, trained_steps: int, trained_tokens: int, out_dir: str,
                        data_loader=None, sharded_optimizer: bool = False):
        os.makedirs(out_dir, exist_ok=True)
        raw = self._unwrap(model)
        if sharded_optimizer and optimizer is not None:
            # every rank: the optimizer is sharded over data x context (x expert) parallel ranks
            self._atomic_save({"optimizer": optimizer.state_dict(),
                               "grid": [self.dp_ws, self.cp_ws, self.ep_ws, self.tp_ws, self.pp_ws]},
                              self._optimizer_shard_path(out_dir))
        if self.dp_rank == 0 and self.cp_rank == 0:
            payload = {
                "model": raw.state_dict(),
                "optimizer": None if (optimizer is None or sharded_optimizer) else optimizer.state_dict(),
                "trained_steps": trained_steps,
                "trained_tokens": trained_tokens,
                "rng_state": torch.get_rng_state(),
                "data_loader": data_loader.state_dict() if hasattr(data_loader, "state_dict") else None,
            }
            self._atomic_save(payload, self._get_checkpoint_path(out_dir))
        if dist.is_initialized():
            dist.barrier()
        if (not dist.is_initialized()) or dist.get_rank() == 0:
            manifest = {"files": self.expected_files(sharded_optimizer and optimizer is not None),
                        "trained_steps": trained_steps,
                        "trained_tokens": trained_tokens}
            tmp = os.path.join(out_dir, "manifest.json.tmp")
            with open(tmp, "w") as fh:
                json.dump(manifest, fh)
            os.replace(tmp, os.path.join(out_dir, "manifest.json"))
        if dist.is_initialized():
            dist.barrier()

    def load_checkpoint(self, model, optimizer, out_dir: str, data_loader=None, sharded_optimizer: bool = False):
        """Load this rank's shard (same topology as at save time). Returns (steps, tokens)."""
        manifest_path = os.path.join(out_dir, "manifest.json")
        if os.path.exists(manifest_path):
            missing = [f for f in json.load(open(manifest_path))["files"]
                       if not os.path.exists(os.path.join(out_dir, f))]
            if missing:
                raise FileNotFoundError(f"incomplete checkpoint in {out_dir}: missing {missing}")
        path = self._get_checkpoint_path(out_dir)
        if not os.path.exists(path):
            raise FileNotFoundError(f"checkpoint not found at {path}")
        ckpt = torch.load(path, map_location="cpu", weights_only=False)
        raw = self._unwrap(model)
        with torch.no_grad():
            own = raw.state_dict()
            for k, v in ckpt["model"].items():
                own[k].copy_(v)          # in place: parameters may be views of a flat buffer
        if optimizer is not None:
            if sharded_optimizer:
                shard = self._optimizer_shard_path(out_dir)
                if not os.path.exists(shard):
                    raise FileNotFoundError(f"optimizer shard of this rank not found: {shard} (the checkpoint was "
                                            "written with a different parallel layout or is incomplete)")
                sd = torch.load(shard, map_location="cpu", weights_only=False)
                grid = [self.dp_ws, self.cp_ws, self.ep_ws, self.tp_ws, self.pp_ws]
                if sd.get("grid", grid) != grid:
                    raise ValueError(f"optimizer shard {shard} was written for grid {sd['grid']}, this run has {grid}")
                optimizer.load_state_dict(sd["optimizer"])
            elif ckpt.get("optimizer") is not None:
                optimizer.load_state_dict(ckpt["optimizer"])
        if data_loader is not None and ckpt.get("data_loader") is not None and hasattr(data_loader, "load_state_dict"):
            data_loader.load_state_dict(ckpt["data_loader"])
        if ckpt.get("rng_state") is not None:
            torch.set_rng_state(ckpt["rng_state"])
        return ckpt["trained_steps"], ckpt["trained_tokens"]
