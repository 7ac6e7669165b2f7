"""GPU: the 7.2B shapes of the benchmark configurations, checked through properties that do not need a CPU
reference of that size: determinism, agreement between the batch-1 and the batched kernels on the same packed
weights, linearity, and composition of the WKV-7 recurrence (T steps in one call = T calls of one step)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 4e-3   # both kernels accumulate in fp32 (int8: exact int32 sums) and round the result to fp16 once


def _st():
    return torch.cuda.current_stream().cuda_stream


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def _gemv(_lib, cm, x):
    y = torch.empty(cm.n_out, dtype=torch.float16, device="cuda")
    _lib.check(_lib.lib.ab_gemv(C.byref(cm), x.data_ptr(), y.data_ptr(), _st()), "ab_gemv")
    return y


def _gemm(_lib, cm, x):
    rows = x.shape[0]
    y = torch.empty(rows, cm.n_out, dtype=torch.float16, device="cuda")
    scratch = torch.zeros(_lib.lib.ab_gemm_scratch_bytes(C.byref(cm), rows) + 256, dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.ab_gemm(C.byref(cm), rows, x.data_ptr(), y.data_ptr(), 0, None, scratch.data_ptr(), _st()), "ab_gemm")
    return y


@pytest.mark.parametrize("fmt", ["int8", "nvfp4"])
@pytest.mark.parametrize("n_out,k", [(4096, 4096), (16384, 4096), (4096, 16384), (65536, 4096)])
def test_products_at_7b_shapes(fmt, n_out, k):
    from albatross_b200 import _lib, quant
    torch.manual_seed(n_out // 64 + k)
    pm = quant.quantize((torch.randn(n_out, k, device="cuda") * 0.02).half(), fmt)
    cm = pm.as_mat()
    x = torch.randn(320, k, device="cuda").half()
    # the batched kernel twice: bit-identical (fixed summation order, also across the K slices of a split product)
    y1 = _gemm(_lib, cm, x)
    y2 = _gemm(_lib, cm, x)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    # batch-1 kernel on single rows of the batch: same packed weights, different kernel, same answer
    for r in (0, 157, 319):
        g1 = _gemv(_lib, cm, x[r].contiguous())
        g2 = _gemv(_lib, cm, x[r].contiguous())
        assert torch.equal(g1, g2)
        assert _rel(g1, y1[r]) < TOL
    # linearity of the batch-1 kernel in its input (fp16 inputs chosen so that the sum is exact)
    a = (torch.randint(-8, 9, (k,), device="cuda").float() / 8).half()
    b = (torch.randint(-8, 9, (k,), device="cuda").float() / 8).half()
    ya, yb, yab = _gemv(_lib, cm, a), _gemv(_lib, cm, b), _gemv(_lib, cm, (a + b))
    assert _rel(yab, ya.float() + yb.float()) < TOL
    # and against the de-quantised weights in fp32 on the device
    want = x[:4].float() @ pm.dequantize().t()
    assert _rel(y1[:4], want) < TOL
    assert _lib.device_status() == 0


def test_wkv7_composition_at_7b_head_count():
    """64 heads, 24 sequences: one call over T = 6 tokens equals six calls over one token (state carried in place)."""
    from albatross_b200 import _lib
    torch.manual_seed(11)
    B, T, H = 24, 6, 64
    Cn = H * 64
    mk = lambda s=1.0: (torch.randn(B, T, Cn, device="cuda") * s).half()
    r, k, v = mk(), mk(0.3), mk()
    w = (-torch.rand(B, T, Cn, device="cuda") * 2 - 0.5).half()          # pre-transform decay
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, 64, device="cuda"), dim=-1).reshape(B, T, Cn)
    a, b = (-kk).half(), (kk * torch.rand(B, T, Cn, device="cuda")).half()
    s_all = torch.zeros(B, H, 64, 64, device="cuda")
    y_all = torch.empty_like(r)
    _lib.check(_lib.lib.ab_wkv7_fwd(B, T, Cn, H, s_all.data_ptr(), r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(),
                                    a.data_ptr(), b.data_ptr(), y_all.data_ptr(), _st()), "ab_wkv7_fwd")
    s_step = torch.zeros_like(s_all)
    ys = []
    for t in range(T):
        sl = [z[:, t:t + 1].contiguous() for z in (r, w, k, v, a, b)]
        y = torch.empty_like(sl[0])
        _lib.check(_lib.lib.ab_wkv7_fwd(B, 1, Cn, H, s_step.data_ptr(), *[z.data_ptr() for z in sl], y.data_ptr(), _st()),
                   "ab_wkv7_fwd")
        ys.append(y)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(ys, dim=1), y_all)
    assert torch.equal(s_step, s_all)
    assert torch.isfinite(s_all).all()


def test_decode_paths_agree_at_7b_block_shapes():
    """Two blocks at the 7.2B shapes (D 4096, 64 heads, ffn 16384, vocabulary 65536): the persistent batch-1
    kernel, the per-phase launches and the batched tensor-core path give the same logits within fp16 rounding."""
    from albatross_b200 import RWKV_x070, synth
    args = synth.make_args("7.2b-l2")
    sd = dict(synth.iter_checkpoint("7.2b-l2", seed=0, device="cuda"))
    toks = [17, 40000, 3, 65535, 123]
    outs = {}
    for mode in ("persistent", "eager"):
        m = RWKV_x070(args, quant="int8", state_dict=sd, decode_mode=mode, use_graph=(mode != "eager"))
        st, seq = None, []
        for t in toks:
            logits, st = m.forward(t, st)
            seq.append(logits.float().clone())
        outs[mode] = torch.stack(seq)
        if mode == "persistent":
            B = 320                                   # every sequence of the batch gets the same tokens
            stb, seqb = None, []
            for t in toks:
                lb, stb = m.forward_batch([[t]] * B, stb)
                seqb.append(lb.float().clone())
            outs["batch"] = torch.stack(seqb)
        del m
    ref = outs["persistent"]
    assert torch.isfinite(ref).all()
    assert _rel(outs["eager"], ref) < 2e-3
    b = outs["batch"]
    assert torch.equal(b[:, 0], b[:, 319]) and torch.equal(b[:, 0], b[:, 160])   # rows of a batch do not interact
    assert _rel(b[:, 0], ref) < 2e-2
