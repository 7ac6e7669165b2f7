"""albatross_b200 — sm_100a kernels for the RWKV-7 decode hot path behind the reference's model API.

`RWKV_x070`, `RWKV7_OP` and `RWKV7_BATCH_OP` mirror reference/rwkv7.py; `synth` builds seeded
synthetic checkpoints in the reference's key schema; `build` compiles the CUDA library.
Importing the model needs the built library (python -m albatross_b200.build).
"""
import importlib

__all__ = ["RWKV_x070", "RWKV7_OP", "RWKV7_BATCH_OP", "sampler_simple_batch"]


def __getattr__(name):
    if name in __all__:
        return getattr(importlib.import_module(".rwkv7", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
