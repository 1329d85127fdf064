"""Materialisation from Hugging Face safetensors: name mapping, tensor-parallel slicing, pipeline
stages picking their layers, sharded checkpoints, and the reference's default of reading the files but
training from random initialisation (picotron/checkpoint.py:53-267)."""
import json
import os
import types

import torch

from distributed_helpers import run_distributed


def _config(layers=4):
    return types.SimpleNamespace(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96,
                                 vocab_size=128, num_hidden_layers=layers, max_position_embeddings=32,
                                 rms_norm_eps=1e-5, rope_theta=10000.0, num_experts=1)


def _write_hf_checkpoint(path, sharded):
    """A Hugging Face style checkpoint of a single-device model; returns the model's state dict."""
    from safetensors.torch import save_file
    from picotron_b200.checkpoint import InitializationManager
    from picotron_b200.models.llama import Llama
    torch.manual_seed(5)
    model = Llama(_config())
    mgr = InitializationManager(model, _config(), tp_rank=0, tp_world_size=1)
    tensors = {mgr.hf_name(k): v.detach().clone().contiguous() for k, v in model.state_dict().items()}
    os.makedirs(path, exist_ok=True)
    if not sharded:
        save_file(tensors, os.path.join(path, "model.safetensors"))
    else:
        names = sorted(tensors)
        half = len(names) // 2
        parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
        for fname, keys in parts.items():
            save_file({k: tensors[k] for k in keys}, os.path.join(path, fname))
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as fh:
            json.dump({"weight_map": {k: f for f, keys in parts.items() for k in keys}}, fh)
    return model.state_dict()


def test_name_mapping_round_trip():
    from picotron_b200.checkpoint import InitializationManager
    from picotron_b200.models.llama import Llama
    model = Llama(_config(2))
    mgr = InitializationManager(model, _config(2), tp_rank=0, tp_world_size=1)
    names = mgr.get_layer_names_in_sft_format()
    assert "model.embed_tokens.weight" in names and "lm_head.weight" in names and "model.norm.weight" in names
    assert "model.layers.1.self_attn.o_proj.weight" in names and "model.layers.0.mlp.gate_proj.weight" in names
    for k, _ in model.named_parameters():
        assert mgr.convert_safetensors_to_hf_name(mgr.hf_name(k)) == k


def _tp_worker(rank, world, ckpt_dir, sharded):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import (init_model_with_dematerialized_weights,
                                          init_model_with_materialized_weights)
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.tensor_parallel import apply_tensor_parallel
    pgm.setup_process_group_manager(tp_size=world, cp_size=1, pp_size=1, dp_size=1)
    full = torch.load(os.path.join(ckpt_dir, "full.pt"))
    with init_model_with_dematerialized_weights():
        model = Llama(_config())
        apply_tensor_parallel(model)
    assert all(p.device.type == "meta" for p in model.parameters())
    model = init_model_with_materialized_weights(model, _config(), save_dir=ckpt_dir, load_pretrained=True)
    sd = model.state_dict()
    q = sd["decoder_layers.1.attention.q_proj.weight"]
    want = full["decoder_layers.1.attention.q_proj.weight"]
    rows = want.shape[0] // world
    assert torch.equal(q, want[rank * rows:(rank + 1) * rows])                       # column parallel: rows
    o = sd["decoder_layers.2.attention.out_proj.weight"]
    want = full["decoder_layers.2.attention.out_proj.weight"]
    cols = want.shape[1] // world
    assert torch.equal(o, want[:, rank * cols:(rank + 1) * cols])                    # row parallel: columns
    emb = sd["embedding.weight"]
    v = full["embedding.weight"].shape[0] // world
    assert torch.equal(emb, full["embedding.weight"][rank * v:(rank + 1) * v])       # vocabulary shard
    assert torch.equal(sd["final_norm.weight"], full["final_norm.weight"])           # replicated
    # default: the files are read and checked, the model is initialised randomly (reference behaviour)
    with init_model_with_dematerialized_weights():
        model2 = Llama(_config())
        apply_tensor_parallel(model2)
    model2 = init_model_with_materialized_weights(model2, _config(), save_dir=ckpt_dir)
    assert not torch.equal(model2.state_dict()["decoder_layers.1.attention.q_proj.weight"], q)


def test_tp2_loads_its_slices(tmp_path):
    for sharded in (False, True):
        d = str(tmp_path / ("sharded" if sharded else "single"))
        full = _write_hf_checkpoint(d, sharded)
        torch.save(full, os.path.join(d, "full.pt"))
        run_distributed(_tp_worker, 2, d, sharded)


def _pp_worker(rank, world, ckpt_dir):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import InitializationManager, init_model_with_materialized_weights
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.pipeline_parallel import wrap_pipeline
    pgm.setup_process_group_manager(tp_size=1, cp_size=1, pp_size=world, dp_size=1)
    full = torch.load(os.path.join(ckpt_dir, "full.pt"))
    with torch.device("meta"):
        stage = wrap_pipeline(Llama(_config()), _config(), "1f1b", 2)
    names = InitializationManager(stage, _config()).get_layer_names_in_sft_format()
    mine = {"model.layers.0", "model.layers.1"} if rank == 0 else {"model.layers.2", "model.layers.3"}
    assert {".".join(n.split(".")[:3]) for n in names if n.startswith("model.layers.")} == mine
    assert ("model.embed_tokens.weight" in names) == (rank == 0) and ("lm_head.weight" in names) == (rank == 1)
    stage = init_model_with_materialized_weights(stage, _config(), save_dir=ckpt_dir, load_pretrained=True)
    for k, v in stage.state_dict().items():
        assert torch.equal(v, full[k]), k


def test_pipeline_stage_loads_its_layers(tmp_path):
    d = str(tmp_path / "ckpt")
    full = _write_hf_checkpoint(d, False)
    torch.save(full, os.path.join(d, "full.pt"))
    run_distributed(_pp_worker, 2, d)


def test_shape_mismatch_is_reported(tmp_path):
    from picotron_b200.checkpoint import InitializationManager
    mgr = InitializationManager(torch.nn.Linear(2, 2), None, tp_rank=1, tp_world_size=2)
    assert mgr.adjust_tensor_size((8, 4), (4, 4)) == (slice(4, 8), slice(0, 4))
    assert mgr.adjust_tensor_size((4, 8), (4, 4)) == (slice(0, 4), slice(4, 8))
    assert mgr.adjust_tensor_size((6, 4), (4, 4)) == (slice(0, 4), slice(0, 4))      # checkpoint larger: truncate
    try:
        mgr.adjust_tensor_size((2, 4), (4, 4), "w")
        raise AssertionError("a checkpoint tensor that is too small was accepted")
    except ValueError:
        pass
