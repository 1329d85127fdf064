"""The reference's optional DeepEP backend (picotron/expert_parallel/deepep_backend.py:38-120) by name.

DeepEP is not used by this framework: ``model.ep_backend = "deepep"`` selects the same peer-memory
kernels as ``"fused"`` (``ops/fused_ep_var.py``: dropless dispatch and combine laid out on the device),
which take DeepEP's role inside ``MoELayer``. The functional API of the reference's module therefore
reports the library as unavailable, which is the answer its callers branch on.
"""
from __future__ import annotations


def deepep_available() -> bool:
    return False


def _unavailable(*_args, **_kwargs):
    raise RuntimeError('DeepEP is not part of this framework; set model.ep_backend to "fused" (or "deepep", an alias) '
                       "and let MoELayer use the peer-memory dispatch and combine kernels")


dispatch = _unavailable
combine = _unavailable
