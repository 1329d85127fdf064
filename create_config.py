"""Write ``<out_dir>/<exp_name>/config.json`` for train.py.

Same command line as the reference's create_config.py (``--tp --cp --ep --dp --pp --pp_engine
--num_virtual_stages --model_name --num_hidden_layers ... --grad_acc_steps --mbs --seq_len
--exp_name --use_wandb --use_cpu --use_fused_adam --hf_token`` and the MoE knobs), plus switches
for what this framework wires into the trainer: ``--sequence_parallel --vocab_parallel_ce
--async_tp --overlap_comm --zero_stage --dp_engine --cp_attention --ep_as_dp --parallel_block
--init_std --dataset synthetic``. Works offline: the model shape comes from the built-in table
(``picotron_b200.config.MODEL_SHAPES``) or from explicit ``--hidden_size``-style flags, and no
model is downloaded unless ``--download`` is given.

    python create_config.py --out_dir tmp --exp_name smollm_dp2_tp4 --dp 2 --tp 4 \
        --model_name HuggingFaceTB/SmolLM-1.7B --sequence_parallel --vocab_parallel_ce --zero_stage 1 \
        --mbs 4 --grad_acc_steps 8 --seq_len 2048 --dataset synthetic
"""
import argparse
import copy
import json
import os
import shutil

from picotron_b200.config import DEFAULTS, MODEL_ARCH_KEYS, MODEL_SHAPES, load_config


def create_single_config(args) -> str:
    template = os.path.join(os.path.dirname(os.path.abspath(__file__)), "template", "base_config.json")
    cfg = json.load(open(template)) if os.path.exists(template) else copy.deepcopy(DEFAULTS)
    d, m, t = cfg["distributed"], cfg["model"], cfg["training"]
    d.update(tp_size=args.tp, cp_size=args.cp, ep_size=args.ep, dp_size=args.dp, pp_size=args.pp,
             pp_engine=args.pp_engine, num_virtual_stages=args.num_virtual_stages, use_cpu=args.use_cpu,
             backend="gloo" if args.use_cpu else "nccl", sequence_parallel=args.sequence_parallel,
             vocab_parallel_ce=args.vocab_parallel_ce, async_tp=args.async_tp, overlap_comm=args.overlap_comm,
             zero_stage=args.zero_stage, dp_engine=args.dp_engine, cp_attention=args.cp_attention, cp_zigzag=args.cp_zigzag,
             ep_as_dp=args.ep_as_dp)
    m["name"] = args.model_name
    shape = MODEL_SHAPES.get(args.model_name, {})
    for k in MODEL_ARCH_KEYS:
        v = getattr(args, k, None)
        m[k] = v if v is not None else (shape.get(k) if k in ("num_hidden_layers", "num_attention_heads",
                                                               "num_key_value_heads") else m.get(k))
    m.update(num_experts=args.num_experts, num_experts_per_tok=args.num_experts_per_tok,
             num_shared_experts=args.num_shared_experts, ep_overlap=bool(args.ep_overlap),
             ep_num_tiles=args.ep_num_tiles, ep_fp8_dispatch=bool(args.ep_fp8_dispatch),
             moe_latent_dim=args.moe_latent_dim, ep_backend=args.ep_backend,
             ep_capacity_factor=args.ep_capacity_factor, ep_capacity_dropless=bool(args.ep_capacity_dropless),
             ep_max_rounds=args.ep_max_rounds, router_aux_loss_coef=args.router_aux_loss_coef,
             router_bias_update_rate=args.router_bias_update_rate, use_fused_adam=args.use_fused_adam,
             parallel_block=args.parallel_block, init_std=args.init_std,
             dtype="float32" if args.use_cpu else "bfloat16")
    t.update(seq_length=args.seq_len, micro_batch_size=args.mbs, gradient_accumulation_steps=args.grad_acc_steps)
    if args.total_train_steps is not None:
        t["total_train_steps"] = args.total_train_steps
    cfg["dataset"]["subset_name"] = args.subset_name
    if args.dataset is not None:
        cfg["dataset"]["name"] = args.dataset
    cfg["logging"].update(use_wandb=args.use_wandb, run_name=args.exp_name, log_frequency=args.log_frequency)
    cfg["environment"]["HF_TOKEN"] = args.hf_token
    if args.use_cpu:
        cfg["environment"]["FLASH_ATTEN"] = "0"
    load_config(cfg)  # validates
    run_path = os.path.join(args.out_dir, args.exp_name)
    if os.path.exists(run_path):
        shutil.rmtree(run_path)
    os.makedirs(run_path)
    path = os.path.join(run_path, "config.json")
    with open(path, "w") as fh:
        json.dump(cfg, fh, indent=4)
    return path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser()
    p.add_argument("--out_dir", type=str, default="tmp")
    for name in ("tp", "cp", "ep", "dp", "pp"):
        p.add_argument(f"--{name}", type=int, default=1)
    p.add_argument("--pp_engine", type=str, default="1f1b", choices=["afab", "1f1b", "zb", "interleaved", "zbv"])
    p.add_argument("--num_virtual_stages", type=int, default=2)
    p.add_argument("--model_name", type=str, default="HuggingFaceTB/SmolLM-360M-Instruct")
    for k in MODEL_ARCH_KEYS:
        p.add_argument(f"--{k}", type=float if k in ("rms_norm_eps", "rope_theta") else int, default=None)
    p.add_argument("--num_experts", type=int, default=1)
    p.add_argument("--num_experts_per_tok", type=int, default=1)
    p.add_argument("--num_shared_experts", type=int, default=0)
    p.add_argument("--ep_overlap", type=int, default=1)
    p.add_argument("--ep_num_tiles", type=int, default=1)
    p.add_argument("--ep_fp8_dispatch", type=int, default=0)
    p.add_argument("--moe_latent_dim", type=int, default=0)
    p.add_argument("--ep_backend", type=str, default="torch")
    p.add_argument("--ep_capacity_factor", type=float, default=0.0)
    p.add_argument("--ep_capacity_dropless", type=int, default=1)
    p.add_argument("--ep_max_rounds", type=int, default=8)
    p.add_argument("--router_aux_loss_coef", type=float, default=0.0)
    p.add_argument("--router_bias_update_rate", type=float, default=0.0)
    p.add_argument("--grad_acc_steps", type=int, default=1)
    p.add_argument("--mbs", type=int, default=1)
    p.add_argument("--seq_len", type=int, default=1024)
    p.add_argument("--total_train_steps", type=int, default=None)
    p.add_argument("--subset_name", type=str, default=None)
    p.add_argument("--dataset", type=str, default=None, help="dataset name; 'synthetic' = seeded uniform tokens")
    p.add_argument("--exp_name", type=str, default="dummy_exp")
    p.add_argument("--use_wandb", action="store_true")
    p.add_argument("--log_frequency", type=int, default=1,
                   help="synchronise with the device and print only every N-th step")
    p.add_argument("--use_cpu", action="store_true")
    p.add_argument("--use_fused_adam", action="store_true")
    p.add_argument("--hf_token", type=str, default=None)
    p.add_argument("--sequence_parallel", action="store_true")
    p.add_argument("--vocab_parallel_ce", action="store_true")
    p.add_argument("--async_tp", action="store_true")
    p.add_argument("--overlap_comm", action="store_true")
    p.add_argument("--zero_stage", type=int, default=0, choices=[0, 1, 2, 3])
    p.add_argument("--dp_engine", type=str, default="bucket", choices=["bucket", "naive", "zero", "fused"])
    p.add_argument("--cp_attention", type=str, default="ring", choices=["ring", "ulysses"])
    p.add_argument("--cp_zigzag", action="store_true",
                   help="ring attention: give every rank one early and one late chunk of the sequence (balanced causal work)")
    p.add_argument("--ep_as_dp", action="store_true")
    p.add_argument("--parallel_block", action="store_true")
    p.add_argument("--init_std", type=float, default=None)
    p.add_argument("--download", action="store_true", help="also fetch the model from the Hugging Face hub")
    return p


if __name__ == "__main__":
    args = build_parser().parse_args()
    path = create_single_config(args)
    print("Configs saved to", path)
    if args.download:
        from picotron_b200.utils import download_model
        download_model(args.model_name, args.hf_token)
