"""ctypes loader for the plain-C restatement in hotpath_oracle.c (TEST INFRASTRUCTURE ONLY)."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libhotpath_oracle.so")


def build() -> str:
    src = os.path.join(_HERE, "hotpath_oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def _lib():
    lib = C.CDLL(build())
    return lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def wkv7(state, r, w, k, v, a, b):
    """state [B,H,64,64] float32 (updated in place); r..b [B,T,C] float32. Returns y [B,T,C] float32."""
    B, T, Cn = r.shape
    H = Cn // 64
    arrs = [np.ascontiguousarray(x, dtype=np.float32) for x in (r, w, k, v, a, b)]
    y = np.empty_like(arrs[0])
    assert state.dtype == np.float32 and state.flags.c_contiguous
    _lib().oracle_wkv7(B, T, Cn, H, _p(state, C.c_float), *[_p(x, C.c_float) for x in arrs], _p(y, C.c_float))
    return y


def gemv_int8(q, s, x):
    n, k = q.shape
    y = np.empty(n, dtype=np.float64)
    x = np.ascontiguousarray(x, dtype=np.float32)
    _lib().oracle_gemv_int8(n, k, _p(np.ascontiguousarray(q), C.c_int8), _p(np.ascontiguousarray(s), C.c_float),
                            _p(x, C.c_float), _p(y, C.c_double))
    return y


def dequant_nvfp4(packed, sb, t):
    n, kh = packed.shape
    out = np.empty((n, kh * 2), dtype=np.float32)
    _lib().oracle_dequant_nvfp4(n, kh * 2, _p(np.ascontiguousarray(packed), C.c_uint8),
                                _p(np.ascontiguousarray(sb), C.c_uint8), C.c_float(float(t)), _p(out, C.c_float))
    return out


def gemv_nvfp4(packed, sb, t, x):
    n, kh = packed.shape
    y = np.empty(n, dtype=np.float64)
    x = np.ascontiguousarray(x, dtype=np.float32)
    _lib().oracle_gemv_nvfp4(n, kh * 2, _p(np.ascontiguousarray(packed), C.c_uint8),
                             _p(np.ascontiguousarray(sb), C.c_uint8), C.c_float(float(t)), _p(x, C.c_float),
                             _p(y, C.c_double))
    return y
