"""Configuration: the JSON schema of ``template/base_config.json`` (a superset of the
reference's, see train.py:84-236 and create_config.py:57-123 there), validated into plain
namespaces, plus a built-in table of model shapes so no Hugging Face download is needed.

Sections and keys keep the reference's names: ``distributed`` (tp_size, cp_size, ep_size,
pp_size, dp_size, pp_engine, num_virtual_stages, backend, use_cpu), ``model``, ``training``,
``dataset``, ``checkpoint``, ``logging``, ``environment``. New optional keys switch on what the
reference only exposes as library code: ``distributed.{sequence_parallel, vocab_parallel_ce,
async_tp, overlap_comm, zero_stage, dp_engine, cp_attention, ep_as_dp}``,
``model.{parallel_block, hidden_size, intermediate_size, vocab_size, rope_theta, rms_norm_eps,
max_position_embeddings, init_std}``, ``dataset.name = "synthetic"`` and
``training.{cuda_graph, flat_params}`` (``flat_params``: bf16 parameters and fp32 gradients in two flat
device buffers, the fast path on a GPU; ``null`` = on unless ``zero_stage`` >= 2, whose gradient and
parameter sharding lives on the per-parameter path of ``parallel/zero.py``; ``true`` keeps the flat
buffers, where stages 2 and 3 shard the optimizer state only).
"""
from __future__ import annotations

import copy
import json
from types import SimpleNamespace
from typing import Any, Dict

#: architecture shapes that the reference would fetch with AutoConfig.from_pretrained
MODEL_SHAPES: Dict[str, Dict[str, Any]] = {
    "HuggingFaceTB/SmolLM-1.7B": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                                      num_attention_heads=32, num_key_value_heads=32, vocab_size=49152,
                                      max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0),
    "HuggingFaceTB/SmolLM-360M-Instruct": dict(hidden_size=960, intermediate_size=2560, num_hidden_layers=32,
                                               num_attention_heads=15, num_key_value_heads=5, vocab_size=49152,
                                               max_position_embeddings=2048, rms_norm_eps=1e-5,
                                               rope_theta=10000.0),
    "HuggingFaceTB/SmolLM-135M": dict(hidden_size=576, intermediate_size=1536, num_hidden_layers=30,
                                      num_attention_heads=9, num_key_value_heads=3, vocab_size=49152,
                                      max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0),
    "meta-llama/Llama-2-7b-hf": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                                     num_attention_heads=32, num_key_value_heads=32, vocab_size=32000,
                                     max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0),
    "tiny-llama-test": dict(hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=8,
                            num_key_value_heads=4, vocab_size=4096, max_position_embeddings=256,
                            rms_norm_eps=1e-5, rope_theta=10000.0),
    "moe-ep8-bench": dict(hidden_size=2048, intermediate_size=1024, num_hidden_layers=16, num_attention_heads=16,
                          num_key_value_heads=16, vocab_size=32000, max_position_embeddings=4096,
                          rms_norm_eps=1e-5, rope_theta=10000.0),
    "long-context-bench": dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=16,
                               num_attention_heads=32, num_key_value_heads=8, vocab_size=32000,
                               max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0),
}

DEFAULTS: Dict[str, Dict[str, Any]] = {
    "distributed": dict(tp_size=1, cp_size=1, ep_size=1, pp_size=1, dp_size=1, pp_engine="1f1b",
                        num_virtual_stages=2, backend="nccl", use_cpu=False, sequence_parallel=False,
                        vocab_parallel_ce=False, async_tp=False, overlap_comm=False, zero_stage=0,
                        dp_engine="bucket", cp_attention="ring", cp_zigzag=False, ep_as_dp=False),
    "model": dict(name="HuggingFaceTB/SmolLM-360M-Instruct", num_hidden_layers=None, num_attention_heads=None,
                  num_key_value_heads=None, num_experts=1, num_experts_per_tok=2, num_shared_experts=0,
                  norm_topk_prob=True, dtype="bfloat16", use_flash_attention=True, use_fused_adam=True,
                  ep_overlap=True, ep_num_tiles=1, ep_fp8_dispatch=False, moe_latent_dim=0, ep_backend="torch", ep_var_slack=3.0,
                  ep_capacity_factor=0.0, ep_capacity_dropless=True, ep_max_rounds=8,
                  router_aux_loss_coef=0.0, router_bias_update_rate=0.0, parallel_block=False, init_std=None,
                  shared_expert_intermediate_size=None),
    "training": dict(seed=42, learning_rate=3e-4, total_train_steps=200, seq_length=1024, micro_batch_size=32,
                     gradient_accumulation_steps=1, num_samples=400000, max_tokens=None, weight_decay=0.01,
                     cuda_graph=True, flat_params=None),
    "dataset": dict(name="roneneldan/TinyStories", subset_name=None, num_workers=0, num_proc=4, split="train"),
    "checkpoint": dict(save_dir="ckpt", save_frequency=300, load_path=""),
    "logging": dict(use_wandb=False, project_name="picotron", run_name=None, metrics_jsonl=None,
                    step_breakdown=False, log_frequency=1),
    "environment": dict(OMP_NUM_THREADS="1", TOKENIZERS_PARALLELISM="false", FLASH_ATTEN="1", HF_TOKEN=None),
}

PP_ENGINES = ("afab", "1f1b", "zb", "interleaved", "zbv")
DP_ENGINES = ("bucket", "naive", "zero", "fused")
MODEL_ARCH_KEYS = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                   "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta")


def load_config(path_or_dict) -> Dict[str, Dict[str, Any]]:
    """Read a JSON config (path or dict), fill defaults, validate. Returns a dict of dicts."""
    raw = path_or_dict if isinstance(path_or_dict, dict) else json.load(open(path_or_dict))
    cfg = copy.deepcopy(DEFAULTS)
    for section, values in raw.items():
        if section not in cfg:
            raise ValueError(f"unknown config section '{section}'")
        cfg[section].update(values)
    validate(cfg)
    return cfg


def validate(cfg) -> None:
    d, t = cfg["distributed"], cfg["training"]
    for k in ("tp_size", "cp_size", "ep_size", "pp_size", "dp_size"):
        if not (isinstance(d[k], int) and d[k] >= 1):
            raise ValueError(f"distributed.{k} must be a positive integer")
    if d["pp_engine"] not in PP_ENGINES:
        raise ValueError(f"distributed.pp_engine must be one of {PP_ENGINES}")
    if d["dp_engine"] not in DP_ENGINES:
        raise ValueError(f"distributed.dp_engine must be one of {DP_ENGINES}")
    if d["zero_stage"] not in (0, 1, 2, 3):
        raise ValueError("distributed.zero_stage must be 0..3")
    if d["cp_attention"] not in ("ring", "ulysses"):
        raise ValueError("distributed.cp_attention must be 'ring' or 'ulysses'")
    if t["seq_length"] % d["cp_size"] != 0:
        raise ValueError("training.seq_length must be divisible by distributed.cp_size")
    if d["overlap_comm"] and not d["sequence_parallel"]:
        raise ValueError("distributed.overlap_comm needs distributed.sequence_parallel")
    if d["sequence_parallel"] and t["seq_length"] // d["cp_size"] % d["tp_size"] != 0:
        raise ValueError("sequence parallelism needs seq_length/cp_size divisible by tp_size")


def world_size_of(cfg) -> int:
    d = cfg["distributed"]
    return d["tp_size"] * d["cp_size"] * d["ep_size"] * d["pp_size"] * d["dp_size"]


def model_config_from(cfg) -> SimpleNamespace:
    """The architecture namespace the model consumes (the role of HF AutoConfig + the overrides of
    train.py:209-236)."""
    m, t = cfg["model"], cfg["training"]
    base = dict(MODEL_SHAPES.get(m["name"], {}))
    for k in MODEL_ARCH_KEYS:
        if m.get(k) is not None:
            base[k] = m[k]
    missing = [k for k in MODEL_ARCH_KEYS if k not in base]
    if missing:
        raise ValueError(f"model '{m['name']}' is not in the built-in shape table; set model.{missing} explicitly")
    base["max_position_embeddings"] = max(int(t["seq_length"]), 1) if m.get("max_position_embeddings") is None \
        else m["max_position_embeddings"]
    for k in ("num_experts", "num_experts_per_tok", "num_shared_experts", "norm_topk_prob", "ep_overlap",
              "ep_num_tiles", "ep_fp8_dispatch", "moe_latent_dim", "ep_backend", "ep_var_slack", "ep_capacity_factor",
              "ep_capacity_dropless", "ep_max_rounds", "router_aux_loss_coef", "router_bias_update_rate",
              "parallel_block", "init_std", "shared_expert_intermediate_size"):
        base[k] = m[k]
    base["ep_as_dp"] = cfg["distributed"]["ep_as_dp"]
    return SimpleNamespace(**base)
