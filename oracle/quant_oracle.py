"""CPU oracle for the two weight formats of the RWKV-7 decode path (TEST INFRASTRUCTURE ONLY).

Nothing under ``albatross_b200/`` may import this file: it is the checker for the CUDA path,
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``.

Parity status: **unpinned against the reference for the quantisers.**  The reference snapshot
holds no quantiser (every matrix product there is a plain fp16 ``x @ W``, reference/rwkv7.py:230-233,
:250, :308-309, :156), so the int8 and NVFP4 formats are defined by this build and this file is
their normative restatement in numpy.  What *is* pinned is the storage convention the quantisers
work on: the ``[out, in]`` row-major ``nn.Linear`` storage that reference/rwkv7.py:88-90 turns
into transposed views, i.e. one output channel per K-contiguous row.

int8 (symmetric, weight only)
    per output row o:  s_o = max_i |W_oi| / 127 (fp32);  q_oi = clip(rint(W_oi / s_o), -127, 127);
    de-quantised value = float32(q_oi) * s_o  (a single fp32 rounding).
    Optional per-input-column scale c_i > 0:  W is divided by c_i before the row quantiser and the
    product multiplies x by c_i instead, so that  W_oi ~= q_oi * s_o * c_i.

NVFP4 (public format: e2m1 values, 16-element blocks along K, e4m3 block scales, fp32 tensor scale)
    t    = max|W| / (448 * 6)                                  (fp32)
    sb   = e4m3_rne(min(max_block|W| / (6 * t), 448))          (one per 16 consecutive K elements)
    q    = e2m1_rne(W / (t * sb))  saturated to +-6 ; q = 0 where sb == 0
    de-quantised value = (q * sb) * t                          (q*sb is exact in fp32)
    Packed storage: two e2m1 codes per byte, even k in the low nibble.
"""
from __future__ import annotations

import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# Decision thresholds between neighbouring e2m1 magnitudes and which side a tie goes to
# (round-to-nearest-even on the 3-bit magnitude code: ties go to the even code).
_E2M1_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
_E2M1_TIE_UP = np.array([False, True, False, True, False, True, False])


# ----------------------------------------------------------------------------------------------
# e4m3 (fn variant: no infinities, max 448, subnormal step 2**-9), written out bit by bit
# ----------------------------------------------------------------------------------------------
def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn code -> float32 value (NaN codes 0x7f/0xff never produced by the quantiser)."""
    code = code.astype(np.uint8)
    sign = np.where(code & 0x80, -1.0, 1.0).astype(np.float32)
    e = ((code >> 3) & 0xF).astype(np.int32)
    m = (code & 0x7).astype(np.float32)
    sub = m * np.float32(2.0 ** -9)
    nor = (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float32))
    return (sign * np.where(e == 0, sub, nor)).astype(np.float32)


_E4M3_POS = e4m3_decode(np.arange(0, 0x7F, dtype=np.uint8))  # codes 0..126 ascending, 126 -> 448


def e4m3_encode_rne(x: np.ndarray) -> np.ndarray:
    """Non-negative float32 -> nearest e4m3fn code (ties to even code), saturating at 448."""
    x = np.minimum(np.asarray(x, dtype=np.float32), np.float32(448.0))
    hi = np.searchsorted(_E4M3_POS, x, side="left").clip(0, len(_E4M3_POS) - 1)
    lo = (hi - 1).clip(0)
    d_hi = _E4M3_POS[hi].astype(np.float64) - x.astype(np.float64)
    d_lo = x.astype(np.float64) - _E4M3_POS[lo].astype(np.float64)
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)


# ----------------------------------------------------------------------------------------------
# e2m1
# ----------------------------------------------------------------------------------------------
def e2m1_encode_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 code (bit 3 = sign), round to nearest, ties to even code, saturating."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x)
    code = np.zeros(x.shape, dtype=np.uint8)
    for mid, tie_up in zip(_E2M1_MID, _E2M1_TIE_UP):
        code += ((mag > mid) | ((mag == mid) & tie_up)).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 3)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    code = code.astype(np.uint8)
    mag = E2M1_VALUES[code & 7]
    return np.where(code & 8, -mag, mag).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# int8
# ----------------------------------------------------------------------------------------------
def int8_col_scale(w: np.ndarray) -> np.ndarray:
    """Optional per-input-column scale: sqrt of the column's max magnitude relative to the mean one."""
    colmax = np.abs(w.astype(np.float32)).max(axis=0)
    mean = np.float32(colmax.mean())
    c = np.sqrt(np.maximum(colmax, np.float32(1e-12)) / max(mean, np.float32(1e-12)), dtype=np.float32)
    return c.astype(np.float32)


def int8_quantize(w: np.ndarray, col_scale: np.ndarray | None = None):
    """w: [out, in] float -> (q int8 [out, in], row_scale fp32 [out])."""
    w = w.astype(np.float32)
    if col_scale is not None:
        w = (w / col_scale.astype(np.float32)[None, :]).astype(np.float32)
    amax = np.abs(w).max(axis=1)
    s = (amax / np.float32(127.0)).astype(np.float32)
    safe = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
    q = np.rint((w / safe[:, None]).astype(np.float32)).clip(-127, 127).astype(np.int8)
    return q, s


def int8_dequantize(q: np.ndarray, s: np.ndarray, col_scale: np.ndarray | None = None) -> np.ndarray:
    w = (q.astype(np.float32) * s.astype(np.float32)[:, None]).astype(np.float32)
    if col_scale is not None:
        w = (w * col_scale.astype(np.float32)[None, :]).astype(np.float32)
    return w


# ----------------------------------------------------------------------------------------------
# NVFP4
# ----------------------------------------------------------------------------------------------
def nvfp4_quantize(w: np.ndarray):
    """w: [out, in] float, in % 16 == 0 -> (packed uint8 [out, in/2], sb uint8 [out, in/16], t fp32)."""
    w = w.astype(np.float32)
    n, k = w.shape
    assert k % 16 == 0
    amax = np.float32(np.abs(w).max())
    t = np.float32(amax / np.float32(448.0 * 6.0))
    if t == 0:
        t = np.float32(1.0)
    blk = w.reshape(n, k // 16, 16)
    bmax = np.abs(blk).max(axis=2)
    sb_code = e4m3_encode_rne((bmax / (np.float32(6.0) * t)).astype(np.float32))
    sb = e4m3_decode(sb_code)
    denom = (t * sb).astype(np.float32)
    safe = np.where(denom > 0, denom, np.float32(1.0)).astype(np.float32)
    code = e2m1_encode_rne((blk / safe[:, :, None]).astype(np.float32))
    code = np.where((denom > 0)[:, :, None], code, 0).astype(np.uint8).reshape(n, k)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8)
    return packed, sb_code, t


def nvfp4_dequantize(packed: np.ndarray, sb_code: np.ndarray, t) -> np.ndarray:
    n, kh = packed.shape
    code = np.empty((n, kh * 2), dtype=np.uint8)
    code[:, 0::2] = packed & 0xF
    code[:, 1::2] = packed >> 4
    q = e2m1_decode(code).reshape(n, kh * 2 // 16, 16)
    sb = e4m3_decode(sb_code)
    w = ((q * sb[:, :, None]).astype(np.float32) * np.float32(t)).astype(np.float32)
    return w.reshape(n, kh * 2)


def fake_quantize(w: np.ndarray, fmt: str) -> np.ndarray:
    """Round trip through a format: what the reference sees as its fp32 weight."""
    if fmt == "int8":
        return int8_dequantize(*int8_quantize(w))
    if fmt == "nvfp4":
        return nvfp4_dequantize(*nvfp4_quantize(w))
    if fmt in (None, "none", "fp16"):
        return w.astype(np.float32)
    raise ValueError(fmt)
