"""CPU: the C-ABI library loads and exports every function the public header declares."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    src = open(os.path.join(ROOT, "include", "albatross_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ab_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported():
    from albatross_b200 import _lib
    names = _declared()
    assert len(names) >= 10
    dll = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert sorted(_lib.EXPORTS) == names


def test_version_and_error_string_without_gpu():
    from albatross_b200 import _lib
    assert _lib.lib.ab_version() >= 1
    assert isinstance(_lib.lib.ab_last_error(), bytes)


def test_bad_arguments_are_rejected_before_any_launch():
    from albatross_b200 import _lib
    m = _lib.Mat()                       # empty matrix: rejected on the host, no CUDA call
    assert _lib.lib.ab_gemv(ctypes.byref(m), 16, 16, None) == -1
    assert b"empty" in _lib.lib.ab_last_error() or b"format" in _lib.lib.ab_last_error()
    assert _lib.lib.ab_wkv7_fwd(1, 1, 100, 2, 16, 16, 16, 16, 16, 16, 16, 16, None) == -1   # C != H*64


def test_python_struct_layout_matches_header():
    from albatross_b200 import _lib
    assert ctypes.sizeof(_lib.Mat) == 48
    assert ctypes.sizeof(_lib.Layer) == 19 * 8 + 10 * 48 + 4 * 8 + 4 * 48


def test_streaming_kernels_do_not_spill():
    """The batch-1 kernels run at their register cap; a spill in them (easily introduced by code added to the
    persistent kernel) slows every matrix-vector phase, so the build's ptxas report is checked."""
    from albatross_b200 import build
    build.build(force=True)
    usage = build.resource_usage()
    hot = {k: v for k, v in usage.items() if "decode_kernel" in k or "gemv_stream_kernel" in k or "head_batch_kernel" in k
           or "gemm_tc_kernel" in k}
    assert len(hot) == 5, sorted(usage)
    for name, u in hot.items():
        # the persistent kernel keeps one 16-byte stack slot (spill stores + loads: 28 bytes in ptxas' count) outside its
        # streaming loop; measured harmless (the same build is the fastest one), anything beyond that is not
        limit = 32 if "decode_kernel" in name else 0
        assert u["spill_bytes"] <= limit, (name, u)
