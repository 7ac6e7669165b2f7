"""What would 4-bit (or 8-bit) ACTIVATIONS cost? (TEST INFRASTRUCTURE ONLY; CPU, numpy/torch.)

The native block-scaled tensor-core instruction for NVFP4 weights (`tcgen05.mma.kind::mxf4nvf4`) takes BOTH
operands as e2m1 values with e4m3 block scales, so using it means quantising the activation that feeds every big
matrix product to NVFP4 on the fly ("W4A4"). The intermediate is e4m3 activations ("W4A8", `kind::f8f6f4` with the
weights expanded to e4m3-representable values). The reference keeps activations in fp16
(reference/rwkv7.py:230-233, :250, :308-309, :156), and the stated tolerance is a max relative logit error of 2e-2
against it. This module measures, with the CPU oracle, what each choice does to the logits, to the per-block outputs
and to the greedy arg-max, on the same NVFP4 weights:

    python -m oracle.act_quant_study [tiny|0.1b] [n_tokens]

Activation formats (per token, i.e. per row of the batched product):
    nvfp4 : t = amax/(448*6); 16-element blocks along K; sb = e4m3(amax_block/(6 t)); q = e2m1(x/(t sb))
    e4m3  : s = amax/448; q = e4m3(x/s)
"""
from __future__ import annotations

import sys
from typing import Callable, Dict, Optional

import numpy as np
import torch

from . import quant_oracle as qo
from . import rwkv7_oracle as ro


def act_nvfp4(x: torch.Tensor) -> torch.Tensor:
    a = x.detach().float().numpy().reshape(-1, x.shape[-1])
    out = np.empty_like(a)
    for r in range(a.shape[0]):   # one tensor scale per token
        out[r] = qo.nvfp4_dequantize(*qo.nvfp4_quantize(a[r:r + 1]))[0]
    return torch.from_numpy(out.reshape(x.shape)).to(x.dtype)


def act_e4m3(x: torch.Tensor) -> torch.Tensor:
    a = x.detach().float().numpy().reshape(-1, x.shape[-1])
    amax = np.abs(a).max(axis=1, keepdims=True)
    s = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    q = qo.e4m3_decode(qo.e4m3_encode_rne(np.abs(a / s).astype(np.float32))) * np.sign(a)
    return torch.from_numpy((q * s).astype(np.float32).reshape(x.shape)).to(x.dtype)


ACT_FORMATS: Dict[str, Optional[Callable]] = {"fp16 (weight-only)": None, "e4m3 (W4A8)": act_e4m3, "nvfp4 (W4A4)": act_nvfp4}


def run(cfg: str = "tiny", n_tokens: int = 24, seed: int = 0):
    """Teacher-forced decode of `n_tokens` random ids. Returns {format: dict(logit_rel_err, block_rel_err, agree)}
    measured against the fp16-activation run on the same NVFP4-de-quantised weights."""
    from albatross_b200 import synth
    args = synth.make_args(cfg)
    raw = synth.make_checkpoint(cfg, seed)
    rq = {k: (torch.from_numpy(qo.fake_quantize(v.numpy(), "nvfp4")) if ro.is_big(k) else v) for k, v in raw.items()}
    z = ro.prepare(rq, args.n_embd, torch.float32)
    toks = torch.randint(0, args.vocab_size, (n_tokens,), generator=torch.Generator().manual_seed(seed)).tolist()
    results, base = {}, None
    for name, act in ACT_FORMATS.items():
        o = ro.Oracle(z, args.n_layer, args.n_embd, act=act)
        st = ro.new_state(args.n_layer, args.n_embd)
        logits, blocks = [], []
        for t in toks:
            col = []
            lg, st = o.step(t, st, collect=col)
            logits.append(lg.numpy().copy())
            blocks.append(torch.stack(col).numpy())
        logits, blocks = np.stack(logits), np.stack(blocks)      # [T,V], [T,L,D]
        if base is None:
            base = (logits, blocks)
            continue
        bl, bb = base
        step_err = np.abs(logits - bl).max(axis=1) / np.abs(bl).max(axis=1)
        blk_err = np.abs(blocks - bb).max(axis=2) / np.abs(bb).max(axis=2)     # [T,L]
        results[name] = dict(logit_rel_err_max=float(step_err.max()), logit_rel_err_median=float(np.median(step_err)),
                             first_block_rel_err_max=float(blk_err[:, 0].max()),
                             last_block_rel_err_max=float(blk_err[:, -1].max()),
                             argmax_agree=float((logits.argmax(1) == bl.argmax(1)).mean()))
    return results


if __name__ == "__main__":
    cfg = sys.argv[1] if len(sys.argv) > 1 else "tiny"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 24
    for name, r in run(cfg, n).items():
        print(cfg, name, " ".join(f"{k}={v:.4g}" for k, v in r.items()))
