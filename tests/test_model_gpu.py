"""Whole-model check on the GPU: the hand-written kernel path (fused QKV/RoPE/attention, tcgen05
GEMMs, fused norms, fused cross entropy, flat AdamW) against the plain PyTorch restatement of the
same bf16 model (``PICO_REFERENCE_OPS=1``) — losses over a few optimizer steps must agree."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _losses(reference: bool, steps=4, kv_heads=4, graph=True):
    from picotron_b200 import ops, process_group_manager as pgm
    from picotron_b200.engine import TrainEngine
    os.environ["PICO_REFERENCE_OPS"] = "1" if reference else "0"
    pgm.process_group_manager = None
    cfg = {"distributed": dict(tp_size=1, dp_size=1),
           "model": dict(name="tiny-llama-test", init_std=0.02, dtype="bfloat16", num_hidden_layers=2,
                         hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=kv_heads),
           "training": dict(seed=0, learning_rate=1e-3, seq_length=256, micro_batch_size=2,
                            gradient_accumulation_steps=2, num_samples=512, cuda_graph=graph),
           "dataset": dict(name="synthetic")}
    eng = TrainEngine(cfg, device=torch.device("cuda", 0))
    out = [eng.train_step().item() for _ in range(steps)]
    if not reference:
        ops.check_status("model test")
        assert (eng._mb_graph not in (None, False)) == graph, "CUDA-graph replay was (not) used as asked"
    os.environ["PICO_REFERENCE_OPS"] = "0"
    return out


@pytest.mark.parametrize("kv_heads", [8, 4])
def test_kernel_path_matches_torch_path(kv_heads):
    a = _losses(False, kv_heads=kv_heads)
    b = _losses(True, kv_heads=kv_heads)
    for x, y in zip(a, b):
        assert abs(x - y) < 3e-2, (a, b)
    assert a[-1] < a[0]


def test_graph_replay_equals_eager_launches():
    """The micro-batch replayed from a CUDA graph runs the same kernels in the same order as eager
    launches: the losses of several optimizer steps are bit-identical."""
    a = _losses(False, steps=5, graph=True)
    b = _losses(False, steps=5, graph=False)
    assert a == b, (a, b)
