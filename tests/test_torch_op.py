"""The operator shim: `torch.ops.rwkv7_state_fwd_fp16.forward` (the name and argument list the reference calls at
reference/rwkv7.py:48, :64, registered at reference/cuda/rwkv7_state_fwd_fp16.cpp:12-14) backed by ab_wkv7_fwd."""
import pytest
import torch

from albatross_b200 import torch_op


def _args(B, T, H, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    C = H * 64
    mk = lambda s=1.0: (torch.randn(B, T, C, generator=g) * s).half().to(device)
    state = (torch.randn(B, H, 64, 64, generator=g) * 0.1).to(device)
    r, k, v = mk(), mk(), mk()
    w = (-torch.nn.functional.softplus(-torch.randn(B, T, C, generator=g)) - 0.5).half().to(device)
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, 64, generator=g), dim=-1).view(B, T, C)
    a = (-kk).half().to(device)
    b = (kk * torch.rand(B, T, C, generator=g)).half().to(device)
    return C, state, r, w, k, v, a, b


def test_operator_is_registered_and_checks_its_arguments():
    torch_op.load()
    op = torch.ops.rwkv7_state_fwd_fp16.forward
    C, state, r, w, k, v, a, b = _args(1, 2, 2, "cpu")
    y = torch.empty_like(r)
    with pytest.raises(RuntimeError, match="CUDA tensor"):        # the reference's binding silently does nothing here
        op(1, 2, C, 2, state, r, w, k, v, a, b, y)
    with pytest.raises(RuntimeError, match="H \\* 64"):
        op(1, 2, C + 1, 2, state, r, w, k, v, a, b, y)


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H", [(1, 1, 4), (1, 7, 3), (5, 3, 2)])
def test_operator_matches_the_c_abi_and_the_oracle(B, T, H):
    """Called the way the reference's WKV_7 / WKV_7_batch wrappers call it: y allocated by the caller, state updated in
    place. Bit-identical to ab_wkv7_fwd through ctypes, and within fp16 accuracy of the oracle's recurrence."""
    from albatross_b200 import rwkv7
    from oracle.rwkv7_oracle import Oracle
    torch_op.load()
    C, state, r, w, k, v, a, b = _args(B, T, H, "cuda", seed=B * 100 + T)
    s_op, s_abi = state.clone(), state.clone()
    y = torch.empty((B, T, C), device="cuda", dtype=torch.half)
    torch.ops.rwkv7_state_fwd_fp16.forward(B, T, C, H, s_op, r, w, k, v, a, b, y)
    want = rwkv7.RWKV7_BATCH_OP(s_abi, r, w, k, v, a, b)
    assert torch.equal(y, want) and torch.equal(s_op, s_abi)
    s_or = state.clone().cpu()
    y_or = Oracle.wkv7_kernel(s_or, *(t.cpu() for t in (r, w, k, v, a, b)))
    assert (y.cpu().float() - y_or.float()).abs().max() <= 2e-2 * y_or.float().abs().max()
    assert (s_op.cpu() - s_or).abs().max() <= 2e-3 * s_or.abs().max()
    # a side stream: the kernel runs on torch's current stream, not on the legacy default stream
    side = torch.cuda.Stream()
    s2 = state.clone()
    y2 = torch.empty_like(y)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        torch.ops.rwkv7_state_fwd_fp16.forward(B, T, C, H, s2, r, w, k, v, a, b, y2)
    side.synchronize()
    assert torch.equal(y2, y) and torch.equal(s2, s_op)
