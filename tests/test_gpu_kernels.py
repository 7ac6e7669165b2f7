"""GPU: each kernel through the C ABI against the CPU oracle on the same seeded inputs."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from helpers import GOLDEN, rel_err
from oracle import quant_oracle as qo
from oracle.rwkv7_oracle import Oracle

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _gemv(pm, x):
    from albatross_b200 import _lib
    y = torch.empty(pm.n_out, dtype=torch.float16, device="cuda")
    mat = pm.as_mat()
    _lib.check(_lib.lib.ab_gemv(C.byref(mat), x.data_ptr(), y.data_ptr(), _stream()), "ab_gemv")
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return y


@pytest.mark.parametrize("fmt", ["int8", "nvfp4"])
@pytest.mark.parametrize("shape", [(64, 256), (100, 768), (257, 4096)])
def test_dequantised_weights_bit_exact(fmt, shape):
    """The kernels' in-register de-quantisation equals the specification bit for bit."""
    from albatross_b200 import quant
    torch.manual_seed(3)
    w = torch.randn(*shape) * 0.02
    w[1] = 0
    pm = quant.quantize(w.cuda(), fmt)
    want = qo.fake_quantize(w.numpy(), fmt)
    got = pm.dequantize().cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_int8_col_scale_dequant_bit_exact():
    from albatross_b200 import quant
    torch.manual_seed(4)
    w = torch.randn(64, 512) * 0.02
    c = qo.int8_col_scale(w.numpy())
    pm = quant.quantize_int8(w.cuda(), torch.from_numpy(c).cuda())
    q, s = qo.int8_quantize(w.numpy(), c)
    assert np.array_equal(pm.w.cpu().numpy(), q)
    assert np.array_equal(pm.dequantize().cpu().numpy(), qo.int8_dequantize(q, s, c))


def test_gemv_int8_config1_against_reference_fixture():
    """Baseline config 1: x fp16 [1,4096] ~N(0,1), W fp16 [4096,4096] ~N(0,0.02), seed 0."""
    from albatross_b200 import quant
    g = np.load(os.path.join(GOLDEN, "gemv_int8_4096.npz"))
    torch.manual_seed(0)
    x = torch.randn(1, 4096).half()
    w = (torch.randn(4096, 4096) * 0.02).half()
    pm = quant.quantize_int8(w.cuda())
    y = _gemv(pm, x.cuda().view(-1)).float().cpu().numpy()
    assert rel_err(y, g["y"][0]) < 2e-3          # fp16 output rounding; the integer sums are exact
    c = torch.from_numpy(qo.int8_col_scale(w.float().numpy())).cuda()
    pm2 = quant.quantize_int8(w.cuda(), c)
    y2 = _gemv(pm2, x.cuda().view(-1)).float().cpu().numpy()
    assert rel_err(y2, g["y_colscale"][0]) < 2e-3


@pytest.mark.parametrize("fmt", ["int8", "nvfp4", "none"])
@pytest.mark.parametrize("n,k", [(8, 256), (61, 768), (4096, 1024), (1000, 16384), (5, 3072)])
def test_gemv_against_oracle(fmt, n, k):
    """Ragged row counts (not a multiple of the rows per warp), K not a multiple of the 1024 tile."""
    from albatross_b200 import quant
    torch.manual_seed(n * 31 + k)
    w = torch.randn(n, k) * 0.02
    x = torch.randn(k).half()
    x[::97] *= 30                                    # activation outliers
    pm = quant.quantize(w.cuda(), None if fmt == "none" else fmt)
    wq = qo.fake_quantize(w.half().float().numpy() if fmt == "none" else w.numpy(), fmt)
    want = wq.astype(np.float64) @ x.double().numpy()
    got = _gemv(pm, x.cuda()).float().cpu().numpy()
    assert rel_err(got, want) < 3e-3


def test_gemv_zero_and_linearity():
    from albatross_b200 import quant
    torch.manual_seed(9)
    w = torch.randn(512, 1024) * 0.02
    pm = quant.quantize_int8(w.cuda())
    z = _gemv(pm, torch.zeros(1024, dtype=torch.float16, device="cuda"))
    assert torch.count_nonzero(z) == 0
    x = torch.randn(1024).half().cuda()
    y1 = _gemv(pm, x).float()
    y2 = _gemv(pm, (x * 2)).float()                  # scaling by 2 is exact in fp16 and in the fixed-point split
    assert torch.equal(y2, y1 * 2)


@pytest.mark.parametrize("B,T,H", [(1, 1, 2), (3, 1, 4), (2, 7, 2), (1, 33, 1)])
def test_wkv7_operator_against_oracle(B, T, H):
    """Same contract as the reference operator: state updated in place, y returned."""
    from albatross_b200 import RWKV7_BATCH_OP, RWKV7_OP
    torch.manual_seed(B * 100 + T)
    Cn = H * 64
    f = lambda s=1.0: (torch.randn(B, T, Cn) * s).half()
    r, k, v = f(), f(), f()
    w = (-torch.nn.functional.softplus(-torch.randn(B, T, Cn)) - 0.5).half()
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, 64), dim=-1).view(B, T, Cn).half()
    a, b = -kk, (kk * torch.sigmoid(torch.randn(B, T, Cn)).half())
    S0 = torch.randn(B, H, 64, 64) * 0.1
    S_ref = S0.clone()
    y_ref = Oracle.wkv7_kernel(S_ref, r, w, k, v, a, b)
    S = S0.clone().cuda()
    dev = [t.cuda().contiguous() for t in (r, w, k, v, a, b)]
    y = RWKV7_BATCH_OP(S, *dev)
    torch.cuda.synchronize()
    assert rel_err(y.float().cpu(), y_ref.float()) < 2e-3
    assert rel_err(S.cpu(), S_ref) < 1e-4
    if B == 1:                                        # the unbatched wrapper takes [T,C] and [H,64,64]
        S1 = S0[0].clone().cuda()
        y1 = RWKV7_OP(S1, *[t[0].contiguous() for t in dev])
        assert torch.equal(y1, y[0]) and torch.equal(S1, S[0])


def test_wkv7_operator_rejects_bad_shapes():
    from albatross_b200 import _lib
    assert _lib.lib.ab_wkv7_fwd(1, 1, 96, 2, 16, 16, 16, 16, 16, 16, 16, 16, None) == -1
    assert b"C == H*64" in _lib.lib.ab_last_error()


def _gemm(pm, x, epi=0, resid=None):
    from albatross_b200 import _lib
    rows = x.shape[0]
    y = torch.empty(rows, pm.n_out, dtype=torch.float16, device="cuda")
    mat = pm.as_mat()
    scratch = torch.zeros(max(256, _lib.lib.ab_gemm_scratch_bytes(C.byref(mat), rows)), dtype=torch.uint8, device="cuda")
    _lib.check(_lib.lib.ab_gemm(C.byref(mat), rows, x.data_ptr(), y.data_ptr(), epi,
                                None if resid is None else resid.data_ptr(), scratch.data_ptr(), _stream()), "ab_gemm")
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return y


@pytest.mark.parametrize("fmt", ["int8", "nvfp4", "none"])
@pytest.mark.parametrize("rows,n,k", [(1, 128, 64), (3, 200, 256), (17, 128, 768), (64, 1000, 1024), (320, 512, 4096),
                                      (300, 130, 3072), (400, 256, 512), (320, 256, 16384)])
def test_batched_product_against_oracle(fmt, rows, n, k):
    """Tensor-core path: ragged batch (not a multiple of 16), ragged output rows (not a multiple of 128),
    batch 320 (two MMAs of N = 160) and more than one batch tile (400 rows)."""
    from albatross_b200 import quant
    torch.manual_seed(rows * 7 + n + k)
    w = torch.randn(n, k) * 0.02
    x = torch.randn(rows, k).half()
    pm = quant.quantize(w.cuda(), None if fmt == "none" else fmt)
    wq = qo.fake_quantize(w.half().float().numpy() if fmt == "none" else w.numpy(), fmt)
    want = x.double().numpy() @ wq.astype(np.float64).T
    got = _gemm(pm, x.cuda()).float().cpu().numpy()
    assert rel_err(got, want) < 3e-3


@pytest.mark.parametrize("rows", [16, 32, 48, 80, 100, 130, 200, 256])
def test_batched_product_split_k_batch_sizes(rows):
    """Few output tiles and a long K loop: split K. The batch size sets how much shared memory a block has for the
    other blocks' partial sums (for some sizes the split is narrowed to make one chunk's slices fit), whether the
    last 32-row chunk is ragged, and how many chunks each block of a tile finishes. With and without the residual
    epilogue; a second call must reproduce the first bit for bit (fixed summation order)."""
    from albatross_b200 import _lib, quant
    torch.manual_seed(rows)
    n, k = 256, 4096
    w = torch.randn(n, k) * 0.02
    x = torch.randn(rows, k).half()
    resid = torch.randn(rows, n).half()
    pm = quant.quantize(w.cuda(), "nvfp4")
    base = x.double().numpy() @ qo.fake_quantize(w.numpy(), "nvfp4").astype(np.float64).T
    for epi, want in ((_lib.EPI_NONE, base), (_lib.EPI_RESID, base + resid.double().numpy())):
        r = resid.cuda() if epi == _lib.EPI_RESID else None
        got = _gemm(pm, x.cuda(), epi, r)
        assert rel_err(got.float().cpu().numpy(), want) < 3e-3
        assert torch.equal(_gemm(pm, x.cuda(), epi, r), got)


def test_batched_product_small_k_and_epilogues():
    """Adapter-sized products (K = 16 ... 480, not multiples of the 64-input k-step) and the fused epilogues."""
    from albatross_b200 import _lib, quant
    torch.manual_seed(5)
    for k in (16, 48, 96, 480):
        w = torch.randn(256, k) * 0.1
        x = torch.randn(20, k).half()
        pm = quant.pack_fp16(w.cuda())
        want = x.double().numpy() @ w.half().double().numpy().T
        assert rel_err(_gemm(pm, x.cuda()).float().cpu().numpy(), want) < 3e-3
    w = torch.randn(192, 256) * 0.05
    x = torch.randn(33, 256).half()
    pm = quant.quantize_int8(w.cuda())
    base = x.double().numpy() @ qo.fake_quantize(w.numpy(), "int8").astype(np.float64).T
    resid = torch.randn(33, 192).half()
    for epi, fn in ((_lib.EPI_TANH, np.tanh), (_lib.EPI_SIGMOID, lambda v: 1 / (1 + np.exp(-v))),
                    (_lib.EPI_RELU2, lambda v: np.maximum(v, 0) ** 2), (_lib.EPI_RESID, lambda v: v + resid.double().numpy())):
        got = _gemm(pm, x.cuda(), epi, resid.cuda() if epi == _lib.EPI_RESID else None).float().cpu().numpy()
        assert rel_err(got, fn(base)) < 4e-3


def test_device_sampler_matches_argsort():
    """ab_sample_rows: noise 0 is the arg-max the reference takes from a descending argsort; with noise the chosen
    logit is within `noise` of the row maximum and the draw is reproducible per seed."""
    from albatross_b200 import sampler_simple_batch
    torch.manual_seed(2)
    for rows, V in ((1, 65536), (320, 65536), (7, 1000), (3, 37)):
        logits = (torch.randn(rows, V, device="cuda") * 3).half()
        logits[0, min(V - 1, 11)] = logits[0].max() + 1                       # a clear winner in row 0
        got = sampler_simple_batch(logits, noise=0.0)
        want = torch.argsort(logits.float(), dim=-1, descending=True, stable=True)[:, :1]
        assert got.shape == (rows, 1) and got.dtype == torch.int64
        assert torch.equal(got, want)
        a = sampler_simple_batch(logits, noise=1.0, seed=5)
        b = sampler_simple_batch(logits, noise=1.0, seed=5)
        c = sampler_simple_batch(logits, noise=1.0, seed=6)
        assert torch.equal(a, b)
        picked = logits.float().gather(1, a)
        assert (picked >= logits.float().max(dim=1, keepdim=True).values - 1.0).all()
        if rows * V > 100000:
            assert not torch.equal(a, c)
    ties = torch.zeros(2, 64, device="cuda").half()
    assert sampler_simple_batch(ties, noise=0.0).flatten().tolist() == [0, 0]  # ties go to the lowest index
    # ids written by the kernel straight into pinned host memory (no copy of their own)
    pinned = torch.full((3, 1), -1, dtype=torch.int64).pin_memory()
    logits = torch.randn(3, 1000, device="cuda").half()
    ret = sampler_simple_batch(logits, noise=0.0, out=pinned)
    torch.cuda.current_stream().synchronize()
    assert ret.data_ptr() == pinned.data_ptr() and pinned.flatten().tolist() == logits.float().argmax(-1).tolist()
