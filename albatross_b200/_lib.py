"""ctypes binding of the C ABI declared in include/albatross_b200.h.

The library is the product: there is no fallback. Importing this module without the built
shared object raises, and every call that returns a non-zero status raises with the library's
own message.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# AB_BOUNDS_CHECK=1 selects the range-checking build of the same library (python -m albatross_b200.build --bounds-check)
LIB_PATH = os.path.join(_HERE, "_C", "libalbatross_b200_checked.so" if os.environ.get("AB_BOUNDS_CHECK") == "1"
                        else "libalbatross_b200.so")

FMT_F16, FMT_I8, FMT_FP4 = 0, 1, 2
EPI_NONE, EPI_TANH, EPI_SIGMOID, EPI_RELU2, EPI_RESID = 0, 1, 2, 3, 4


class Mat(C.Structure):
    _fields_ = [("fmt", C.c_int32), ("n_out", C.c_int32), ("k", C.c_int32), ("_pad", C.c_int32),
                ("w", C.c_void_p), ("scale", C.c_void_p), ("col_scale", C.c_void_p),
                ("tscale", C.c_float), ("_pad2", C.c_float)]


_LAYER_PTRS = ["ln1_w", "ln1_b", "ln2_w", "ln2_b", "x_r", "x_w", "x_k", "x_v", "x_a", "x_g",
               "w0", "a0", "v0", "k_k", "k_a", "r_k", "lnx_w", "lnx_b", "ffn_x_k"]
_LAYER_MATS = ["receptance", "key", "value", "output", "ffn_key", "ffn_value", "w1t", "a1t", "v1t", "g1t"]
_LAYER_UPS = ["w2", "a2", "v2", "g2"]
_LAYER_UPS_T = ["w2t", "a2t", "v2t", "g2t"]


class Layer(C.Structure):
    _fields_ = ([(n, C.c_void_p) for n in _LAYER_PTRS] + [(n, Mat) for n in _LAYER_MATS] +
                [(n, C.c_void_p) for n in _LAYER_UPS] + [(n, Mat) for n in _LAYER_UPS_T])


class ModelDesc(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("vocab", C.c_int32), ("_pad", C.c_int32),
                ("emb", C.c_void_p), ("lnout_w", C.c_void_p), ("lnout_b", C.c_void_p),
                ("head", Mat), ("layers", C.POINTER(Layer))]


class LibraryError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m albatross_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the kernels.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t
    lib.ab_last_error.restype = C.c_char_p
    lib.ab_version.restype = i32
    lib.ab_device_status.argtypes = [C.POINTER(C.c_uint32)]
    lib.ab_wkv7_fwd.argtypes = [i32, i32, i32, i32] + [vp] * 9
    lib.ab_gemv.argtypes = [C.POINTER(Mat), vp, vp, vp]
    lib.ab_gemm_scratch_bytes.argtypes = [C.POINTER(Mat), i32]
    lib.ab_gemm_scratch_bytes.restype = sz
    lib.ab_gemm.argtypes = [C.POINTER(Mat), i32, vp, vp, i32, vp, vp, vp]
    lib.ab_gemm_static.argtypes = [C.POINTER(Mat), i32, vp, vp, i32, vp, vp]
    lib.ab_gemm_static_reset.argtypes = [vp]
    lib.ab_gemm_static_debug_counter.argtypes = [i32, i32, C.POINTER(C.c_uint32)]
    lib.ab_dequant.argtypes = [C.POINTER(Mat), vp, vp]
    lib.ab_gemv_plan_selftest.argtypes = [vp, vp, vp, i32, i32, vp, vp]
    lib.ab_sample_rows.argtypes = [vp, i32, i32, C.c_float, C.c_uint32, vp, vp]
    lib.ab_sample_rows_i64.argtypes = [vp, i32, i32, C.c_float, C.c_uint32, vp, vp]
    lib.ab_model_create.argtypes = [C.POINTER(ModelDesc), C.POINTER(vp)]
    lib.ab_model_destroy.argtypes = [vp]
    lib.ab_model_destroy.restype = None
    lib.ab_workspace_bytes.argtypes = [vp, i32, i32]
    lib.ab_workspace_bytes.restype = sz
    lib.ab_forward.argtypes = [vp, i32, i32, vp, C.POINTER(vp), vp, vp, i32, vp]
    lib.ab_model_set_option.argtypes = [vp, C.c_char_p, i32]
    lib.ab_forward_stage.argtypes = [vp, i32, i32, vp, vp, vp, C.POINTER(vp), vp, vp, vp, vp]
    lib.ab_decode_program_bytes.argtypes = [vp]
    lib.ab_decode_program_bytes.restype = sz
    lib.ab_decode_timeline_offset.argtypes = [vp]
    lib.ab_decode_timeline_offset.restype = sz
    lib.ab_decode_program_build.argtypes = [vp, vp, C.POINTER(vp), vp, vp, vp, vp]
    lib.ab_decode_run.argtypes = [vp, vp, vp]
    return lib


lib = _load()

EXPORTS = ["ab_last_error", "ab_version", "ab_device_status", "ab_wkv7_fwd", "ab_gemv", "ab_gemm_scratch_bytes",
           "ab_gemm", "ab_gemm_static", "ab_gemm_static_reset", "ab_gemm_static_debug_counter", "ab_sample_rows", "ab_sample_rows_i64", "ab_gemv_plan_selftest", "ab_dequant", "ab_model_create", "ab_model_destroy", "ab_workspace_bytes", "ab_forward", "ab_forward_stage",
           "ab_model_set_option", "ab_decode_program_bytes", "ab_decode_timeline_offset", "ab_decode_program_build", "ab_decode_run"]


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = lib.ab_last_error().decode(errors="replace")
        raise LibraryError(f"{what or 'albatross_b200'} failed with status {status}: {msg}")


def device_status() -> int:
    v = C.c_uint32(0)
    check(lib.ab_device_status(C.byref(v)), "ab_device_status")
    return v.value
