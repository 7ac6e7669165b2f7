"""CPU: the load-time quantisers of the package are bit-identical to the oracle's specification."""
import numpy as np
import pytest
import torch

from albatross_b200 import quant
from oracle import quant_oracle as qo


def _w(seed, n=96, k=768, scale=0.02):
    torch.manual_seed(seed)
    w = torch.randn(n, k) * scale
    w[3] = 0
    w[11, 64:80] = 0
    w[17, 5] = 1.0            # an outlier
    return w


@pytest.mark.parametrize("seed", [0, 1])
def test_int8_bit_exact(seed):
    w = _w(seed)
    pm = quant.quantize_int8(w)
    q, s = qo.int8_quantize(w.numpy())
    assert np.array_equal(pm.w.numpy(), q) and np.array_equal(pm.scale.numpy(), s)


@pytest.mark.parametrize("seed", [0, 1])
def test_nvfp4_bit_exact(seed):
    w = _w(seed)
    pm = quant.quantize_nvfp4(w)
    p, sb, t = qo.nvfp4_quantize(w.numpy())
    assert np.array_equal(pm.w.numpy(), p) and np.array_equal(pm.scale.numpy(), sb)
    assert np.float32(pm.tscale) == np.float32(t)


def test_fp16_input_storage_order():
    """Quantising from fp16 [out,in] storage (what the reference keeps) equals quantising its fp32 copy."""
    w = _w(2).half()
    a = quant.quantize_int8(w)
    b = quant.quantize_int8(w.float())
    assert torch.equal(a.w, b.w) and torch.equal(a.scale, b.scale)
