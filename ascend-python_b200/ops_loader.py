"""Loads the operator library so that ``torch.ops.npu.npu_*`` resolve.

No fallback exists: if ``lib/libop_plugin_b200.so`` is missing this raises and
tells how to build it.
"""
from __future__ import annotations

from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
PLUGIN_PATH = _PKG / "lib" / "libop_plugin_b200.so"
_loaded = False


def load():
    global _loaded
    if not _loaded:
        if not PLUGIN_PATH.exists():
            raise RuntimeError(f"{PLUGIN_PATH} is not built; run `python {_PKG / 'build.py'}` "
                               "(there is no fallback implementation)")
        from . import capi

        capi.lib()  # RTLD_GLOBAL: the plugin resolves qmm_* from it
        torch.ops.load_library(str(PLUGIN_PATH))
        _loaded = True
    return torch.ops.npu
