"""Generate tests/golden/*.npz by running the UNMODIFIED reference on the CPU.

Run once, in a container that has the reference checkout (it is not needed afterwards):

    TORCH_CUDA_ARCH_LIST=10.0a TORCH_EXTENSIONS_DIR=/tmp/torch_ext \
        python tests/golden/make_golden.py /path/to/reference_checkout

The reference hard-codes CUDA in two places, so three shims are applied from the outside, without
editing it: ``torch.load`` is wrapped to map to the CPU (reference/rwkv7.py:79), the module-level
``DTYPE`` is set before the model is built (reference/rwkv7.py:30, :90) and an explicit state list is
always passed (the ``state == None`` branch allocates on "cuda", reference/rwkv7.py:100-105).
Only the single-token path is pure torch and therefore valid without a GPU.

The fixtures hold *outputs only*: inputs are regenerated from (config, seed) by
``albatross_b200.synth``, and quantised variants by ``oracle.quant_oracle.fake_quantize``.
"""
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from albatross_b200 import synth  # noqa: E402
from oracle import quant_oracle as qo  # noqa: E402
from oracle.rwkv7_oracle import is_big  # noqa: E402

N_TOKENS = 12


def tokens_for(vocab, n=N_TOKENS, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_reference(ref_mod, raw, args, dtype, toks):
    ref_mod.DTYPE = dtype
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m")
        torch.save(raw, path + ".pth")
        a = types.SimpleNamespace(MODEL_NAME=path, n_layer=args.n_layer, n_embd=args.n_embd,
                                  head_size=64, vocab_size=args.vocab_size)
        model = ref_mod.RWKV_x070(a)
    H = args.n_embd // 64
    state = []
    for _ in range(args.n_layer):
        state += [torch.zeros(args.n_embd, dtype=dtype), torch.zeros(H, 64, 64), torch.zeros(args.n_embd, dtype=dtype)]
    outs = []
    for t in toks:
        logits, state = model.forward(t, state)
        outs.append(logits.float().numpy().copy())
    kv = np.stack([state[3 * i + 1].numpy() for i in range(args.n_layer)])
    xp = np.stack([state[3 * i].float().numpy() for i in range(args.n_layer)])
    return np.stack(outs), kv, xp


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <directory that contains the reference checkout as 'reference'>")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    real_load = torch.load
    torch.load = lambda f, *a, **k: real_load(f, map_location="cpu")
    import reference.rwkv7 as ref_mod  # JIT-builds its CUDA op; harmless without a GPU

    out = {}
    args = synth.make_args("tiny")
    toks = tokens_for(args.vocab_size)
    out["tokens"] = np.array(toks, dtype=np.int64)
    raw = synth.make_checkpoint("tiny", seed=0)
    for fmt in ("none", "int8", "nvfp4"):
        rq = {k: (torch.from_numpy(qo.fake_quantize(v.numpy(), fmt)) if is_big(k) else v)
              for k, v in raw.items()}
        logits, kv, xp = run_reference(ref_mod, rq, args, torch.float, toks)
        out[f"logits_fp32_{fmt}"] = logits
        out[f"kv_fp32_{fmt}"] = kv
        out[f"xprev_fp32_{fmt}"] = xp
    logits, kv, _ = run_reference(ref_mod, raw, args, torch.half, toks)
    out["logits_fp16_none"] = logits
    out["kv_fp16_none"] = kv
    np.savez_compressed(os.path.join(HERE, "tiny_ref_onepath.npz"), **out)

    # The 0.1B shapes (baseline config 2: L=12, D=768, vocab 65536), int8 big matrices, single-token path, fp32.
    # The full logits would be 3 MB; the fixture keeps every 61st column, the arg-max, the five largest values and
    # float64 checksums of each step's logits, and the kv state of the first and last block after the last token.
    args = synth.make_args("0.1b")
    toks = tokens_for(args.vocab_size, n=8, seed=0)
    raw = synth.make_checkpoint("0.1b", seed=0)
    rq = {k: (torch.from_numpy(qo.fake_quantize(v.numpy(), "int8")) if is_big(k) else v) for k, v in raw.items()}
    logits, kv, xp = run_reference(ref_mod, rq, args, torch.float, toks)
    top = np.argsort(-logits, axis=1)[:, :5]
    np.savez_compressed(os.path.join(HERE, "ref_onepath_0.1b_int8.npz"), tokens=np.array(toks, dtype=np.int64),
                        logits_strided=logits[:, ::61].astype(np.float32), argmax=logits.argmax(1),
                        top5_idx=top, top5_val=np.take_along_axis(logits, top, axis=1).astype(np.float32),
                        logits_sum=logits.astype(np.float64).sum(1), logits_sqsum=(logits.astype(np.float64) ** 2).sum(1),
                        kv_first=kv[0].astype(np.float32)[::4, ::8, ::8], kv_last=kv[-1].astype(np.float32)[::4, ::8, ::8],
                        kv_sum=kv.astype(np.float64).sum(axis=(1, 2, 3)), xprev_last=xp[-1].astype(np.float32))

    # Config 1 of the baseline: one int8 weight-only GEMV, x fp16 [1,4096] ~N(0,1), W ~N(0,0.02).
    torch.manual_seed(0)
    x = torch.randn(1, 4096).half()
    w = (torch.randn(4096, 4096) * 0.02).half()
    wq = torch.from_numpy(qo.fake_quantize(w.float().numpy(), "int8"))
    y = x.float() @ wq.t()          # the reference's `x @ W_` with W_ = storage.t(), in fp32
    c = qo.int8_col_scale(w.float().numpy())
    q2, s2 = qo.int8_quantize(w.float().numpy(), c)
    y2 = x.float() @ torch.from_numpy(qo.int8_dequantize(q2, s2, c)).t()
    np.savez_compressed(os.path.join(HERE, "gemv_int8_4096.npz"), y=y.numpy(), y_colscale=y2.numpy(),
                        x_sum=np.float64(x.double().sum()), w_sum=np.float64(w.double().sum()))
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
