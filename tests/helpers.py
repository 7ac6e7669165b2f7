"""Shared helpers for the parity tests: seeded models on both sides of the comparison."""
import os

import numpy as np
import torch

from albatross_b200 import synth
from oracle import quant_oracle as qo
from oracle.rwkv7_oracle import Oracle, is_big, new_state, prepare

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LOGIT_REL_TOL = 2e-2      # max |ours - oracle| / max |oracle| on fp16 logits (the stated tolerance)
ARGMAX_AGREE = 0.995      # teacher-forced greedy agreement


def rel_err(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def oracle_for(cfg: str, fmt: str, seed: int = 0, raw=None):
    """CPU oracle in fp32 on the de-quantised weights of (cfg, seed, fmt)."""
    args = synth.make_args(cfg)
    raw = raw or synth.make_checkpoint(cfg, seed)
    rq = {k: (torch.from_numpy(qo.fake_quantize(v.numpy(), fmt)) if is_big(k) else v) for k, v in raw.items()}
    z = prepare(rq, args.n_embd, torch.float32)
    return Oracle(z, args.n_layer, args.n_embd), args


def model_for(cfg: str, fmt: str, seed: int = 0, raw=None, **kw):
    from albatross_b200 import RWKV_x070
    args = synth.make_args(cfg)
    raw = raw or synth.make_checkpoint(cfg, seed)
    return RWKV_x070(args, quant=None if fmt == "none" else fmt, state_dict=raw, **kw), args


def seeded_tokens(vocab: int, n: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
