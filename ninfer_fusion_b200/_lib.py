"""Loading of the in-tree native library ``_C.so`` (torch.ops.nfb200.*).

The library is built by :mod:`ninfer_fusion_b200._build` and lives next to this
file so that it is visible to anything that inspects loaded objects.  On a
machine with a GPU a missing library is a hard error: there is no silent
PyTorch fallback for the hot path.
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent / "_C.so"
_loaded = False


def native_available() -> bool:
    return _LIB.exists()


def load_native(build_if_missing: bool = False):
    """Load ``_C.so`` once and return ``torch.ops.nfb200``."""
    global _loaded
    if not _loaded:
        if not _LIB.exists():
            if build_if_missing or os.environ.get("NFB200_BUILD_ON_IMPORT") == "1":
                from ._build import build

                build(verbose=False)
            else:
                raise RuntimeError(
                    f"{_LIB} is missing: run `python -m ninfer_fusion_b200._build` "
                    "(or __graft_entry__.build()) first; the CUDA kernels have no fallback"
                )
        torch.ops.load_library(str(_LIB))
        _loaded = True
    return torch.ops.nfb200


class StatusWord:
    """Device status word shared by kernels with bounded waits.

    Kernels record the first failure code (see ``csrc/common/ptx.cuh``); the
    host reads it at step boundaries and raises instead of hanging.
    """

    CODES = {
        1: "consumer waited for a TMA stage that never landed",
        2: "producer waited for a stage that was never released",
        3: "epilogue waited for an accumulator that never committed",
        4: "a peer-rank flag never reached the expected epoch",
        5: "bad kernel argument",
    }

    def __init__(self, device):
        self.tensor = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self, where: str = "") -> None:
        code = int(self.tensor.item())
        if code != 0:
            self.tensor.zero_()
            raise RuntimeError(f"device status {code} ({self.CODES.get(code, 'unknown')}) {where}")
