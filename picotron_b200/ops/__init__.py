"""Math ops of the framework.

Each op exists in exactly two forms: a hand-written sm_100a kernel (``csrc/``), used for bf16
CUDA tensors, and a plain PyTorch restatement (``*_ref``) that runs anywhere (CPU/gloo plumbing
tests, fp32) and is the numerical oracle of the kernel tests. ``PICO_REFERENCE_OPS=1`` forces the
restatement on the GPU for A/B comparisons.
"""
from __future__ import annotations

import importlib.util
import os
import threading
from pathlib import Path

import torch

_EXT = None
_EXT_LOCK = threading.Lock()
_SO_PATH = Path(__file__).resolve().parent.parent / "_C.so"

#: number of kernels of this library launched so far in this process (see ``count_launch``)
LAUNCHES = 0


def count_launch(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def launches() -> int:
    return LAUNCHES


def ext():
    """The compiled extension module. Raises if it has not been built."""
    global _EXT
    if _EXT is not None:
        return _EXT
    with _EXT_LOCK:
        if _EXT is None:
            if not _SO_PATH.exists():
                raise RuntimeError(
                    f"{_SO_PATH} is missing: run `python -m picotron_b200.ops._build` "
                    "(or __graft_entry__.build()) before using CUDA tensors")
            spec = importlib.util.spec_from_file_location("picotron_b200._C", str(_SO_PATH))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _EXT = mod
    return _EXT


def ext_available() -> bool:
    return _SO_PATH.exists()


def reference_ops_forced() -> bool:
    return os.environ.get("PICO_REFERENCE_OPS", "0") == "1"


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the hand-written kernels apply: bf16 CUDA tensors and no debug override.

    On a CUDA device a missing extension is an error, never a silent fallback.
    """
    t = tensors[0]
    if not t.is_cuda or reference_ops_forced():
        return False
    if t.dtype != torch.bfloat16:
        return False
    ext()
    return True


def check_status(what: str = "") -> None:
    """Synchronise and raise if any kernel abandoned a bounded wait since the last check."""
    words = ext().status_fetch()
    if words[0] != 0:
        names = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bounds check failed"}
        hints = {3100: " — the receive buffer of the dropless MoE exchange cannot hold the rows routed to one rank: "
                       "raise model.ep_var_slack (or PICO_EP_VAR_SLACK); 0 sizes it for the worst case"}
        raise RuntimeError(
            f"kernel error {words[0]} ({names.get(words[0], 'unknown')}) block={words[1]} "
            f"site={words[2]} extra={words[3]} {what}{hints.get(words[2], '')}")
