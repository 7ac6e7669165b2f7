"""ab_gemm_static: the batched product whose split-K scratch is a fixed array inside the library.

Called through the C ABI and compared bit for bit with ab_gemm (caller-supplied scratch) on two calls in a
row, so that the second call sees the counters exactly as the first one left them. The file name makes
pytest collect it last; it also passes on its own."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

AB_ERR_TOO_LARGE = -3
AB_GEMM_STATIC_SCRATCH_BYTES = 8 * 1024 * 1024
EPI_NONE, EPI_RESID = 0, 4


def _setup(fmt, n_out, k, rows, seed):
    from albatross_b200 import _lib, quant
    torch.manual_seed(seed)
    w = (torch.randn(n_out, k, device="cuda") * 0.05).half()
    pm = quant.quantize(w, fmt)
    xs = [torch.randn(rows, k, device="cuda").half() for _ in range(2)]
    return _lib, pm, pm.as_mat(), xs


def _reference(_lib, cm, rows, x, epi, resid):
    y = torch.empty(rows, cm.n_out, dtype=torch.float16, device="cuda")
    nbytes = _lib.lib.ab_gemm_scratch_bytes(C.byref(cm), rows)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.ab_gemm(C.byref(cm), rows, x.data_ptr(), y.data_ptr(), epi, resid.data_ptr() if resid is not None else None,
                                scratch.data_ptr(), st), "ab_gemm")
    return y, nbytes


@pytest.mark.parametrize("fmt,n_out,k,rows", [
    ("int8", 1024, 4096, 64),     # few output tiles, long k: split-K, partial tiles and counters in the scratch
    ("nvfp4", 768, 8192, 96),     # split-K, batch rows not a multiple of 32
    ("int8", 16384, 512, 48),     # enough tiles: no split, the scratch is not touched
])
def test_static_scratch_matches_caller_scratch_twice(fmt, n_out, k, rows):
    _lib, pm, cm, xs = _setup(fmt, n_out, k, rows, seed=n_out + rows)
    st = torch.cuda.current_stream().cuda_stream
    resid = torch.randn(rows, n_out, device="cuda").half()
    for call, x in enumerate(xs):                      # two calls in a row, different activations
        for epi, r in ((EPI_NONE, None), (EPI_RESID, resid)):
            want, nbytes = _reference(_lib, cm, rows, x, epi, r)
            assert nbytes <= AB_GEMM_STATIC_SCRATCH_BYTES
            got = torch.empty_like(want)
            _lib.check(_lib.lib.ab_gemm_static(C.byref(cm), rows, x.data_ptr(), got.data_ptr(), epi,
                                               r.data_ptr() if r is not None else None, st), "ab_gemm_static")
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"call {call} epi {epi}: differs from ab_gemm"
    assert _lib.device_status() == 0


def test_static_scratch_rejects_products_beyond_its_size():
    _lib, pm, cm, xs = _setup("int8", 4096, 4096, 320, seed=1)
    assert _lib.lib.ab_gemm_scratch_bytes(C.byref(cm), 320) > AB_GEMM_STATIC_SCRATCH_BYTES
    y = torch.empty(320, 4096, dtype=torch.float16, device="cuda")
    rc = _lib.lib.ab_gemm_static(C.byref(cm), 320, xs[0].data_ptr(), y.data_ptr(), EPI_NONE, None,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == AB_ERR_TOO_LARGE
    msg = _lib.lib.ab_last_error().decode()
    assert "ab_gemm_static" in msg and "scratch" in msg and "ab_gemm" in msg


def test_static_scratch_counters_are_cleared_after_a_reported_device_wait():
    """A stale arrival counter (what a wait that gave up, or an aborted launch, leaves behind) would make every later
    split-K product through the built-in area wrong. No device fault is needed to show the recovery: the test
    overwrites a counter word from the host, runs the documented reset and checks the next product."""
    _lib, pm, cm, xs = _setup("int8", 1024, 4096, 64, seed=5)       # split-K: the counters are in use
    st = torch.cuda.current_stream().cuda_stream
    want, _ = _reference(_lib, cm, 64, xs[0], EPI_NONE, None)
    got = torch.empty_like(want)
    run = lambda: _lib.check(_lib.lib.ab_gemm_static(C.byref(cm), 64, xs[0].data_ptr(), got.data_ptr(), EPI_NONE, None, st))
    run()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    v = C.c_uint32(0)
    _lib.check(_lib.lib.ab_gemm_static_debug_counter(0, 0, C.byref(v)))
    assert v.value == 0                                              # the kernels leave the counters at zero
    # a stale count on a tile this product uses; nothing is launched while it sits there
    v = C.c_uint32(1)
    _lib.check(_lib.lib.ab_gemm_static_debug_counter(0, 1, C.byref(v)))
    _lib.check(_lib.lib.ab_gemm_static_reset(st))
    v = C.c_uint32(99)
    _lib.check(_lib.lib.ab_gemm_static_debug_counter(0, 0, C.byref(v)))
    assert v.value == 0
    run()
    torch.cuda.synchronize()
    assert torch.equal(got, want) and _lib.device_status() == 0
    # the same through ab_device_status: any non-zero status clears the counters. The harmless way to raise one is a
    # token id beyond the vocabulary handed straight to the kernels (it is clamped to the table and reported).
    from albatross_b200 import RWKV_x070, synth
    args = synth.make_args("tiny")
    model = RWKV_x070(args, quant="int8", state_dict=synth.make_checkpoint("tiny", seed=0), decode_mode="eager", use_graph=False)
    v = C.c_uint32(1)
    _lib.check(_lib.lib.ab_gemm_static_debug_counter(0, 1, C.byref(v)))
    tok = torch.tensor([args.vocab_size + 5], dtype=torch.int32, device="cuda")
    logits = torch.empty(args.vocab_size, dtype=torch.float16, device="cuda")
    model._run(1, 1, tok, model.new_state(), logits, False)
    assert _lib.device_status() == 8 and torch.isfinite(logits.float()).all()
    v = C.c_uint32(99)
    _lib.check(_lib.lib.ab_gemm_static_debug_counter(0, 0, C.byref(v)))
    assert v.value == 0
    run()
    torch.cuda.synchronize()
    assert torch.equal(got, want) and _lib.device_status() == 0
