"""Seeded synthetic RWKV-7 checkpoints in the reference's ``.pth`` key schema.

Trained checkpoints are not available offline, so benchmarks and parity tests run on random
weights that have the shapes and value distributions the reference loader expects
(reference/rwkv7.py:79-96 lists every key it reads; benchmark.py:26-40 the model sizes).

Each tensor is drawn from its own generator seeded by (seed, key), so a tensor's values do not
depend on the order of generation or on which other tensors were requested. CPU and CUDA generators
are different streams: a checkpoint drawn on the device (the 7.2B benchmark models) is reproducible
on the device, but is not the checkpoint the same seed gives on the CPU; parity tests draw on the CPU.
"""
from __future__ import annotations

import types
import zlib
from typing import Dict, Iterator, Optional, Tuple

import torch

HEAD = 64

CONFIGS = {
    # name: (n_layer, n_embd, vocab, (rank_w, rank_a, rank_v, rank_g))
    "tiny": (2, 256, 512, (32, 32, 16, 48)),
    "0.1b": (12, 768, 65536, (64, 64, 32, 128)),
    "7.2b": (32, 4096, 65536, (128, 128, 96, 480)),
    # the 7.2B block shapes with fewer blocks: small enough on the device for a profiler capture
    "7.2b-l4": (4, 4096, 65536, (128, 128, 96, 480)),
    "7.2b-l2": (2, 4096, 65536, (128, 128, 96, 480)),
}


def make_args(name: str, model_name: str = "") -> types.SimpleNamespace:
    """The `args` namespace the reference scripts build by hand (benchmark.py:20-40)."""
    L, D, V, ranks = CONFIGS[name]
    a = types.SimpleNamespace()
    a.MODEL_NAME, a.n_layer, a.n_embd, a.head_size, a.vocab_size = model_name, L, D, HEAD, V
    a.ranks = ranks
    return a


def _gen(seed: int, key: str) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed((seed * 1000003 + zlib.crc32(key.encode())) & 0x7FFFFFFFFFFF)
    return g


def _normal(seed, key, shape, std, mean=0.0):
    return torch.empty(shape, dtype=torch.float32).normal_(mean, std, generator=_gen(seed, key))


def _uniform(seed, key, shape, lo, hi):
    return torch.empty(shape, dtype=torch.float32).uniform_(lo, hi, generator=_gen(seed, key))


def tensor_specs(n_layer: int, n_embd: int, vocab: int, ranks) -> Iterator[Tuple[str, tuple, tuple]]:
    """Yield (key, shape, (kind, p0, p1)) for every tensor of the checkpoint."""
    D, F_, H = n_embd, 4 * n_embd, n_embd // HEAD
    rw, ra, rv, rg = ranks
    yield "emb.weight", (vocab, D), ("normal", 0.0, 1.0)
    yield "blocks.0.ln0.weight", (D,), ("uniform", 0.8, 1.2)
    yield "blocks.0.ln0.bias", (D,), ("normal", 0.0, 0.05)
    for i in range(n_layer):
        b = f"blocks.{i}."
        for ln in ("ln1", "ln2"):
            yield b + ln + ".weight", (D,), ("uniform", 0.8, 1.2)
            yield b + ln + ".bias", (D,), ("normal", 0.0, 0.05)
        a = b + "att."
        for c in "rwkvag":
            yield a + "x_" + c, (1, 1, D), ("uniform", 0.0, 1.0)
        yield a + "w0", (1, 1, D), ("uniform", -3.0, 1.0)
        yield a + "w1", (D, rw), ("normal", 0.0, 0.02)
        yield a + "w2", (rw, D), ("normal", 0.0, 0.1)
        yield a + "a0", (1, 1, D), ("normal", 0.0, 0.5)
        yield a + "a1", (D, ra), ("normal", 0.0, 0.02)
        yield a + "a2", (ra, D), ("normal", 0.0, 0.1)
        if i > 0:
            yield a + "v0", (1, 1, D), ("normal", 0.0, 0.5)
            yield a + "v1", (D, rv), ("normal", 0.0, 0.02)
            yield a + "v2", (rv, D), ("normal", 0.0, 0.1)
        yield a + "g1", (D, rg), ("normal", 0.0, 0.02)
        yield a + "g2", (rg, D), ("normal", 0.0, 0.1)
        yield a + "k_k", (1, 1, D), ("uniform", 0.7, 1.0)
        yield a + "k_a", (1, 1, D), ("uniform", 0.8, 1.2)
        yield a + "r_k", (H, HEAD), ("normal", 0.0, 0.1)
        for m in ("receptance", "key", "value", "output"):
            yield a + m + ".weight", (D, D), ("normal", 0.0, 0.02)
        yield a + "ln_x.weight", (D,), ("uniform", 0.8, 1.2)
        yield a + "ln_x.bias", (D,), ("normal", 0.0, 0.05)
        f = b + "ffn."
        yield f + "x_k", (1, 1, D), ("uniform", 0.0, 1.0)
        yield f + "key.weight", (F_, D), ("normal", 0.0, 0.02)
        yield f + "value.weight", (D, F_), ("normal", 0.0, 0.02)
    yield "ln_out.weight", (D,), ("uniform", 0.8, 1.2)
    yield "ln_out.bias", (D,), ("normal", 0.0, 0.05)
    yield "head.weight", (vocab, D), ("normal", 0.0, 0.02)


def make_tensor(seed: int, key: str, shape, dist, device="cpu") -> torch.Tensor:
    kind, p0, p1 = dist
    if device != "cpu" and torch.device(device).type == "cuda":
        # Large tensors (7.2B) are drawn on the device: same (seed, key) -> same values on every CUDA run.
        g = torch.Generator(device=device)
        g.manual_seed((seed * 1000003 + zlib.crc32(key.encode())) & 0x7FFFFFFFFFFF)
        t = torch.empty(shape, dtype=torch.float32, device=device)
        return t.normal_(p0, p1, generator=g) if kind == "normal" else t.uniform_(p0, p1, generator=g)
    return _normal(seed, key, shape, p1, p0) if kind == "normal" else _uniform(seed, key, shape, p0, p1)


def iter_checkpoint(name_or_cfg, seed: int = 0, device="cpu", dtype: Optional[torch.dtype] = None):
    """Yield (key, tensor) one at a time, so a 7.2B model never needs a second full copy."""
    cfg = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    L, D, V, ranks = cfg
    for key, shape, dist in tensor_specs(L, D, V, ranks):
        t = make_tensor(seed, key, shape, dist, device)
        yield key, (t if dtype is None else t.to(dtype))


def make_checkpoint(name_or_cfg, seed: int = 0, device="cpu", dtype=None) -> Dict[str, torch.Tensor]:
    return dict(iter_checkpoint(name_or_cfg, seed, device, dtype))
