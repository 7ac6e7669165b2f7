"""`torch.ops.rwkv7_state_fwd_fp16.forward` backed by this library.

The reference model calls its WKV-7 kernel through a torch operator of that name (reference/rwkv7.py:48, :64;
registered at reference/cuda/rwkv7_state_fwd_fp16.cpp:12-14). `load()` registers the same operator, with the same
argument list, on top of `ab_wkv7_fwd`, so reference code that does `torch.ops.rwkv7_state_fwd_fp16.forward(...)`
runs this library's kernel without being edited (load it INSTEAD of the reference's own extension: an operator name
can be registered once per process).
"""
import os

import torch

from . import build as _build

_loaded = False


def load() -> None:
    global _loaded
    if _loaded:
        return
    if not os.path.exists(_build.TORCH_OP_LIB):
        raise ImportError(f"{_build.TORCH_OP_LIB} is missing: build it with `python -m albatross_b200.build`")
    torch.ops.load_library(_build.TORCH_OP_LIB)
    _loaded = True
