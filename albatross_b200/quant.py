"""Load-time weight quantisers (torch, any device) and the packed-matrix container.

The reference stores every big matrix as fp16 and multiplies with `x @ W` (reference/rwkv7.py:88-90,
:230-233, :250, :308-309, :156). Here the same `[out, in]` row-major storage is quantised per
output row at load time and the product kernels de-quantise on the fly.

int8   : s_o = max_i|W_oi| / 127 ; q = clip(rint(W / s_o), -127, 127) ; W ~= q * s_o [* c_i]
NVFP4  : t = max|W| / (448*6) ; sb = e4m3(max_block|W| / (6 t)) per 16 inputs ;
         q = e2m1(W / (t*sb)) ; W ~= (q * sb) * t ; two codes per byte, even input in the low nibble
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_E2M1_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_E2M1_TIE_UP = (False, True, False, True, False, True, False)  # ties go to the even code


@dataclass
class PackedMatrix:
    """A weight matrix in kernel format. `shape` is the reference's view shape [in, out]."""
    fmt: int
    n_out: int
    k: int
    w: torch.Tensor
    scale: Optional[torch.Tensor] = None
    col_scale: Optional[torch.Tensor] = None
    tscale: float = 1.0

    @property
    def shape(self):
        return (self.k, self.n_out)

    def numel(self) -> int:
        return self.n_out * self.k

    def nbytes(self) -> int:
        n = self.w.numel() * self.w.element_size()
        for t in (self.scale, self.col_scale):
            if t is not None:
                n += t.numel() * t.element_size()
        return n

    def as_mat(self) -> _lib.Mat:
        m = _lib.Mat()
        m.fmt, m.n_out, m.k = self.fmt, self.n_out, self.k
        m.w = self.w.data_ptr()
        m.scale = self.scale.data_ptr() if self.scale is not None else None
        m.col_scale = self.col_scale.data_ptr() if self.col_scale is not None else None
        m.tscale = float(self.tscale)
        return m

    def dequantize(self) -> torch.Tensor:
        """fp32 [n_out, k] through the library's own de-quantisation kernel."""
        out = torch.empty(self.n_out, self.k, dtype=torch.float32, device=self.w.device)
        mat = self.as_mat()
        _lib.check(_lib.lib.ab_dequant(C.byref(mat), out.data_ptr(), torch.cuda.current_stream().cuda_stream),
                   "ab_dequant")
        return out


def int8_col_scale(w: torch.Tensor) -> torch.Tensor:
    colmax = w.float().abs().amax(dim=0)
    mean = colmax.mean().clamp_min(1e-12)
    return torch.sqrt(colmax.clamp_min(1e-12) / mean)


def quantize_int8(w: torch.Tensor, col_scale: Optional[torch.Tensor] = None) -> PackedMatrix:
    """w: [out, in] (any float dtype, contiguous rows)."""
    w = w.float()
    if col_scale is not None:
        w = w / col_scale.float()[None, :]
    amax = w.abs().amax(dim=1)
    s = amax / torch.full_like(amax, 127.0)   # tensor / tensor: a true division on every device
    safe = torch.where(s > 0, s, torch.ones_like(s))
    q = torch.round(w / safe[:, None]).clamp_(-127, 127).to(torch.int8)
    return PackedMatrix(_lib.FMT_I8, w.shape[0], w.shape[1], q.contiguous(), s.contiguous(),
                        None if col_scale is None else col_scale.float().contiguous())


def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    mag = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for mid, tie_up in zip(_E2M1_MID, _E2M1_TIE_UP):
        code += ((mag >= mid) if tie_up else (mag > mid)).to(torch.uint8)
    return code | (torch.signbit(x).to(torch.uint8) << 3)


def quantize_nvfp4(w: torch.Tensor) -> PackedMatrix:
    w = w.float()
    n, k = w.shape
    assert k % 16 == 0, "NVFP4 needs in-features divisible by 16"
    amax = w.abs().amax()
    t = amax / torch.full_like(amax, 448.0 * 6.0)
    if float(t) == 0.0:
        t = torch.ones_like(t)
    blk = w.view(n, k // 16, 16)
    bmax = blk.abs().amax(dim=2)
    sb8 = (bmax / (torch.full_like(t, 6.0) * t).expand_as(bmax)).clamp_(max=448.0).to(torch.float8_e4m3fn)
    sb = sb8.float()
    denom = t.expand_as(sb) * sb
    safe = torch.where(denom > 0, denom, torch.ones_like(denom))
    code = _e2m1_codes(blk / safe[:, :, None])
    code = torch.where((denom > 0)[:, :, None], code, torch.zeros_like(code)).view(n, k)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return PackedMatrix(_lib.FMT_FP4, n, k, packed, sb8.view(torch.uint8).contiguous(), None, float(t))


def pack_fp16(w: torch.Tensor) -> PackedMatrix:
    w = w.to(torch.float16).contiguous()
    return PackedMatrix(_lib.FMT_F16, w.shape[0], w.shape[1], w)


def quantize(w: torch.Tensor, fmt: Optional[str]) -> PackedMatrix:
    if fmt == "int8":
        return quantize_int8(w)
    if fmt == "nvfp4":
        return quantize_nvfp4(w)
    if fmt in (None, "fp16", "none"):
        return pack_fp16(w)
    raise ValueError(f"unknown weight format {fmt!r}")
