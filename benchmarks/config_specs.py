"""The benchmark configurations besides the headline one, as data shared by both arms of
``bench.py`` (this framework through ``TrainEngine``, the reference through
``baseline/reference_arms.py``) and by ``benchmarks/bench_configs.py``.

  moe   DeepSeek-style MoE Llama: 16 layers, hidden 2048, 16 heads, vocab 32000, 64 routed experts
        (SwiGLU FFN 1024, top-6 softmax routing) + shared expert (FFN 2048), aux loss 1e-3 +
        loss-free bias, seq 4096, micro-batch 2, EP = number of GPUs with every EP rank on its own
        tokens (EP doubles as data parallelism for the dense weights).
        variants: ``capacity`` (factor 1.25, rows over capacity dropped, fp8 dispatch),
        ``dropless`` (variable-size exchange; tiled over 4 token tiles where the arm has tiles)
  cp    long-context Llama: 16 layers, hidden 2048, 32 query / 8 KV heads, FFN 5632, vocab 32000,
        RoPE theta 5e5, 16384 tokens per GPU (131072 on 8), micro-batch 1, CP = number of GPUs.
        variants: ``ring``, ``ulysses``, ``ring_zigzag`` (this framework only: ring attention on
        zigzag shards, every rank holding one early and one late chunk; the reference has contiguous
        shards only, its arm then runs plain ``ring``)
  pp    Llama-2-7B shape: 32 layers, hidden 4096, 32 heads, FFN 11008, vocab 32000, seq 4096,
        micro-batch 1, 16 micro-batches; 8 GPUs = TP2 x PP2 x DP2, 4 = TP2 x PP2, 2 = PP2.
        variants: ``interleaved`` (2 virtual stages), ``zb``, ``1f1b``, ``afab``
"""
from __future__ import annotations

MOE_MODEL = dict(hidden_size=2048, intermediate_size=1024, num_hidden_layers=16, num_attention_heads=16,
                 num_key_value_heads=16, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0,
                 num_experts=64, num_experts_per_tok=6, shared_expert_intermediate_size=2048,
                 router_aux_loss_coef=1e-3, router_bias_update_rate=1e-3)
CP_MODEL = dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=16, num_attention_heads=32,
                num_key_value_heads=8, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=500000.0)
PP_MODEL = dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                num_key_value_heads=32, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)

DEFAULT_VARIANT = {"moe": "capacity", "cp": "ulysses", "pp": "interleaved"}
VARIANTS = {"moe": ("capacity", "dropless"), "cp": ("ring", "ulysses", "ring_zigzag"), "pp": ("interleaved", "zb", "1f1b", "afab")}


def make_spec(name: str, world: int, variant: str = None, layers: int = 0, seq: int = 0) -> dict:
    """Everything both arms need: ``model`` (plain numbers), ``seq``, ``mbs``, ``grad_acc``, ``lr``, the
    variant's switches, a label, and ``engine_cfg`` = the config dict of this framework's engine."""
    variant = variant or DEFAULT_VARIANT[name]
    assert variant in VARIANTS[name], f"--variant for {name}: one of {VARIANTS[name]}"
    if name == "moe":
        m = dict(MOE_MODEL)
        if layers:
            m["num_hidden_layers"] = layers
        capacity = variant == "capacity"
        m.update(ep_capacity_factor=1.25 if capacity else 0.0, ep_capacity_dropless=False,
                 ep_fp8_dispatch=True, ep_num_tiles=4)
        s = seq or 4096
        eng_model = dict(name="moe-ep8-bench", init_std=0.02, num_shared_experts=0,
                         ep_backend="torch" if capacity else "fused",
                         **{k: v for k, v in m.items() if k not in ("rms_norm_eps", "rope_theta")})
        cfg = {"distributed": dict(ep_size=world, ep_as_dp=world > 1), "model": eng_model,
               "training": dict(seed=1, learning_rate=3e-4, seq_length=s, micro_batch_size=2,
                                gradient_accumulation_steps=1, num_samples=1 << 14),
               "dataset": dict(name="synthetic")}
        label = (f"ep{world} capacity 1.25 (rows over capacity dropped), fp8 1x128 dispatch" if capacity
                 else f"ep{world} dropless variable-size exchange, fp8 1x128 dispatch")
        return dict(name=name, variant=variant, model=m, seq=s, mbs=2, grad_acc=1, lr=3e-4, engine_cfg=cfg,
                    label=label, model_label="DeepSeek-style MoE Llama (16L h2048 16h, 64 experts ffn1024 top-6 + "
                                             "shared ffn2048, v32000)")
    if name == "cp":
        m = dict(CP_MODEL)
        if layers:
            m["num_hidden_layers"] = layers
        s = seq or 16384 * world
        zigzag = variant == "ring_zigzag"
        variant_attn = "ring" if zigzag else variant
        cfg = {"distributed": dict(cp_size=world, cp_attention=variant_attn, cp_zigzag=zigzag),
               "model": dict(name="long-context-bench", init_std=0.02, max_position_embeddings=s,
                             num_hidden_layers=m["num_hidden_layers"]),
               "training": dict(seed=1, learning_rate=3e-4, seq_length=s, micro_batch_size=1,
                                gradient_accumulation_steps=1, num_samples=256),
               "dataset": dict(name="synthetic")}
        return dict(name=name, variant=variant, model=m, seq=s, mbs=1, grad_acc=1, lr=3e-4, cp_attention=variant_attn,
                    engine_cfg=cfg, label=f"cp{world} {variant}",
                    model_label="long-context Llama (16L h2048 32q/8kv heads ffn5632 v32000, rope theta 5e5)")
    if name == "pp":
        m = dict(PP_MODEL)
        if layers:
            m["num_hidden_layers"] = layers
        tp = 2 if world >= 4 else 1
        pp = 2 if world >= 2 else 1
        dp = world // (tp * pp)
        s = seq or 4096
        cfg = {"distributed": dict(tp_size=tp, pp_size=pp, dp_size=dp, pp_engine=variant, num_virtual_stages=2,
                                   sequence_parallel=tp > 1, vocab_parallel_ce=tp > 1, zero_stage=1 if dp > 1 else 0),
               "model": dict(name="meta-llama/Llama-2-7b-hf", num_hidden_layers=m["num_hidden_layers"], init_std=0.02),
               "training": dict(seed=1, learning_rate=3e-4, seq_length=s, micro_batch_size=1,
                                gradient_accumulation_steps=16, num_samples=1 << 14),
               "dataset": dict(name="synthetic")}
        return dict(name=name, variant=variant, model=m, seq=s, mbs=1, grad_acc=16, lr=3e-4, tp=tp, pp=pp, dp=dp,
                    pp_engine=variant, engine_cfg=cfg, label=f"tp{tp}xpp{pp}xdp{dp} {variant}",
                    model_label="Llama-2-7B-shaped (32L h4096 32h ffn11008 v32000)")
    raise SystemExit(f"unknown config {name}")


def active_params(m: dict) -> float:
    """Parameters that take part in one token's forward pass (routed experts count top-k times)."""
    h, L, v = m["hidden_size"], m["num_hidden_layers"], m["vocab_size"]
    hd = h // m["num_attention_heads"]
    attn = 2 * h * h + 2 * h * m["num_key_value_heads"] * hd
    ffn = 3 * h * m["intermediate_size"]
    if m.get("num_experts", 1) > 1:
        shared = m.get("shared_expert_intermediate_size") or 0
        ffn = m["num_experts_per_tok"] * 3 * h * m["intermediate_size"] + 3 * h * shared + h * m["num_experts"]
    return float(L * (attn + ffn) + 2 * v * h)


def flops_per_token(m: dict, seq: int) -> float:
    """The reference's formula (picotron/utils.py:51-62) on the active parameters."""
    return 6.0 * active_params(m) + 12.0 * m["num_hidden_layers"] * m["hidden_size"] * seq
