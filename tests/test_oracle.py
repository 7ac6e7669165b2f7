"""CPU: the oracle against the fixtures generated from the reference, and the quantiser spec."""
import numpy as np
import torch

from albatross_b200 import synth
from helpers import GOLDEN, oracle_for, rel_err
from oracle import quant_oracle as qo
from oracle.rwkv7_oracle import Oracle, new_state, prepare

import os
import pytest


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(GOLDEN, "tiny_ref_onepath.npz"))


@pytest.mark.parametrize("fmt", ["none", "int8", "nvfp4"])
def test_onepath_matches_reference_fixture(golden, fmt):
    o, args = oracle_for("tiny", fmt)
    st = new_state(args.n_layer, args.n_embd)
    outs = []
    for t in golden["tokens"].tolist():
        l, st = o.step(t, st)
        outs.append(l.numpy())
    # same torch ops in the same order on the same machine class: bit-exact here, 1e-5 elsewhere
    assert np.abs(np.stack(outs) - golden[f"logits_fp32_{fmt}"]).max() < 1e-5
    kv = np.stack([st[3 * i + 1].numpy() for i in range(args.n_layer)])
    assert np.abs(kv - golden[f"kv_fp32_{fmt}"]).max() < 1e-5
    xp = np.stack([st[3 * i].numpy() for i in range(args.n_layer)])
    assert np.abs(xp - golden[f"xprev_fp32_{fmt}"]).max() < 1e-5


def test_onepath_matches_reference_fixture_at_the_0_1b_shapes():
    """Baseline config 2's shapes (12 blocks, 768 wide, vocabulary 65536), int8 big matrices, against the fixture
    tests/golden/make_golden.py wrote by running the unmodified reference module on the CPU."""
    g = np.load(os.path.join(GOLDEN, "ref_onepath_0.1b_int8.npz"))
    o, args = oracle_for("0.1b", "int8")
    st = new_state(args.n_layer, args.n_embd)
    for i, t in enumerate(g["tokens"].tolist()):
        l, st = o.step(t, st)
        l = l.numpy()
        assert np.abs(l[::61] - g["logits_strided"][i]).max() < 2e-5
        assert int(l.argmax()) == int(g["argmax"][i])
        assert np.abs(l[g["top5_idx"][i]] - g["top5_val"][i]).max() < 2e-5
        assert abs(float(l.astype(np.float64).sum()) - float(g["logits_sum"][i])) < 1e-2
    kv = np.stack([st[3 * i + 1].numpy() for i in range(args.n_layer)])
    assert np.abs(kv[0][::4, ::8, ::8] - g["kv_first"]).max() < 1e-5
    assert np.abs(kv[-1][::4, ::8, ::8] - g["kv_last"]).max() < 1e-5
    assert np.abs(kv.astype(np.float64).sum(axis=(1, 2, 3)) - g["kv_sum"]).max() < 1e-2
    assert np.abs(st[3 * (args.n_layer - 1)].numpy() - g["xprev_last"]).max() < 1e-5


def test_onepath_fp16_matches_reference_fixture(golden):
    args = synth.make_args("tiny")
    z = prepare(synth.make_checkpoint("tiny", 0), args.n_embd, torch.half)
    o = Oracle(z, args.n_layer, args.n_embd)
    st = new_state(args.n_layer, args.n_embd, act_dtype=torch.half)
    outs = []
    for t in golden["tokens"].tolist():
        l, st = o.step(t, st)
        outs.append(l.float().numpy())
    assert rel_err(np.stack(outs), golden["logits_fp16_none"]) < 2e-3


@pytest.mark.parametrize("fmt", ["none", "int8"])
def test_kernel_path_agrees_with_pinned_onepath(golden, fmt):
    """The sequence/batch restatement (CUDA-kernel recurrence) must equal the pinned one-path."""
    o, args = oracle_for("tiny", fmt)
    toks = golden["tokens"].tolist()
    st = new_state(args.n_layer, args.n_embd, batch=1)
    lb, st = o.forward_tokens([toks], st, full_output=True)
    assert np.abs(lb[0].numpy() - golden[f"logits_fp32_{fmt}"]).max() < 1e-4
    # token by token through the batch path, two sequences (second = reversed tokens)
    st = new_state(args.n_layer, args.n_embd, batch=2)
    for i, t in enumerate(toks):
        l, st = o.forward_tokens([[t], [toks[-1 - i]]], st)
        assert np.abs(l[0].numpy() - golden[f"logits_fp32_{fmt}"][i]).max() < 1e-4


def test_gemv_fixture():
    g = np.load(os.path.join(GOLDEN, "gemv_int8_4096.npz"))
    torch.manual_seed(0)
    x = torch.randn(1, 4096).half()
    w = (torch.randn(4096, 4096) * 0.02).half()
    assert abs(float(x.double().sum()) - float(g["x_sum"])) < 1e-9     # same seeded inputs as the generator
    q, s = qo.int8_quantize(w.float().numpy())
    y = x.float().numpy() @ qo.int8_dequantize(q, s).T
    assert rel_err(y, g["y"]) < 1e-5


def test_e4m3_and_e2m1_tables():
    codes = np.arange(0, 0x7F, dtype=np.uint8)
    vals = qo.e4m3_decode(codes)
    assert vals[0] == 0 and vals[1] == 2.0 ** -9 and vals[-1] == 448.0 and np.all(np.diff(vals) > 0)
    assert np.array_equal(qo.e4m3_encode_rne(vals), codes)                     # exact values round-trip
    t8 = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(t8, codes)                                           # torch's e4m3fn agrees bit for bit
    mid = (vals[:-1] + vals[1:]) / 2                                           # ties go to the even code
    assert np.array_equal(qo.e4m3_encode_rne(mid), np.where(codes[:-1] % 2 == 0, codes[:-1], codes[1:]))
    assert np.array_equal(qo.e2m1_decode(np.arange(16, dtype=np.uint8))[:8], qo.E2M1_VALUES)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -5.0], dtype=np.float32)
    want = np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, -4.0], dtype=np.float32)
    assert np.array_equal(qo.e2m1_decode(qo.e2m1_encode_rne(ties)), want)


@pytest.mark.parametrize("fmt", ["int8", "nvfp4"])
def test_quantisers_are_idempotent_and_bounded(fmt):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((48, 256)) * 0.02).astype(np.float32)
    w[5] = 0                      # an all-zero row
    w[7, 32:48] = 0               # an all-zero block
    w1 = qo.fake_quantize(w, fmt)
    w2 = qo.fake_quantize(w1, fmt)
    assert np.array_equal(w1, w2)                                  # de-quantised weights are a fixed point
    assert np.all(w1[5] == 0) and np.all(w1[7, 32:48] == 0)
    bound = np.abs(w).max(axis=1, keepdims=True) / 127 * 0.5001 if fmt == "int8" else np.abs(w).max() * 0.2
    assert np.all(np.abs(w1 - w) <= bound + 1e-12)


def test_int8_col_scale_roundtrip():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((32, 128)) * 0.02).astype(np.float32)
    w[:, 3] *= 20                                                   # an outlier input column
    c = qo.int8_col_scale(w)
    q, s = qo.int8_quantize(w, c)
    plain = qo.int8_dequantize(*qo.int8_quantize(w))
    scaled = qo.int8_dequantize(q, s, c)
    mask = np.ones(128, bool); mask[3] = False
    assert np.abs(scaled - w)[:, mask].mean() < np.abs(plain - w)[:, mask].mean()


def test_c_restatement_agrees_with_torch_restatement():
    """Two independent restatements (plain C loops, vectorised torch) of the kernel recurrence and of the
    NVFP4 / int8 decode must agree."""
    from oracle import c_oracle
    torch.manual_seed(5)
    B, T, H = 2, 5, 2
    Cn = H * 64
    f = lambda: torch.randn(B, T, Cn).half()
    r, k, v = f(), f(), f()
    w = (-torch.nn.functional.softplus(-torch.randn(B, T, Cn)) - 0.5).half()
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, 64), dim=-1).view(B, T, Cn).half()
    a, b = -kk, (kk * torch.sigmoid(torch.randn(B, T, Cn)).half())
    S0 = torch.randn(B, H, 64, 64) * 0.1
    S_t = S0.clone()
    y_t = Oracle.wkv7_kernel(S_t, r, w, k, v, a, b)
    S_c = S0.numpy().copy()
    y_c = c_oracle.wkv7(S_c, *[t.float().numpy() for t in (r, w, k, v, a, b)])
    assert np.abs(S_c - S_t.numpy()).max() < 1e-5
    assert rel_err(y_c, y_t.float().numpy()) < 2e-3        # y_t is rounded to fp16, y_c is not

    wmat = (torch.randn(24, 256) * 0.02).numpy()
    x = torch.randn(256).half().float().numpy()
    p, sb, t = qo.nvfp4_quantize(wmat)
    assert np.array_equal(c_oracle.dequant_nvfp4(p, sb, t), qo.nvfp4_dequantize(p, sb, t))
    assert rel_err(c_oracle.gemv_nvfp4(p, sb, t, x), qo.nvfp4_dequantize(p, sb, t).astype(np.float64) @ x) < 1e-6
    q, s = qo.int8_quantize(wmat)
    assert rel_err(c_oracle.gemv_int8(q, s, x), qo.int8_dequantize(q, s).astype(np.float64) @ x) < 1e-6
