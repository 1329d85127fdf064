"""Errors reported by kernels through the device status words.

Every wait inside the hand-written kernels (mbarrier phases, flags written by a peer GPU) is
bounded; a kernel that gives up records ``{code, block, site, extra}`` in a small device
buffer and returns normally, leaving the context usable. ``raise_if_failed`` turns a recorded
failure into a Python exception after synchronising.
"""
from __future__ import annotations

from .. import ops

CODES = {1: "mbarrier wait timed out", 2: "wait for a peer's flag timed out", 3: "bounds check failed"}


class KernelWaitError(RuntimeError):
    def __init__(self, code, block, site, extra, what=""):
        self.code, self.block, self.site, self.extra = code, block, site, extra
        super().__init__(f"kernel error {code} ({CODES.get(code, 'unknown')}) block={block} site={site} "
                         f"extra={extra} {what}".strip())


class CommTimeoutError(KernelWaitError):
    """A kernel stopped waiting for a peer GPU (code 2)."""


def raise_if_failed(what: str = "") -> None:
    words = ops.ext().status_fetch()
    if words[0] == 0:
        return
    cls = CommTimeoutError if words[0] == 2 else KernelWaitError
    raise cls(words[0], words[1], words[2], words[3], what)
