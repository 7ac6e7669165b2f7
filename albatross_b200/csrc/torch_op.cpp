// Registers the library's WKV-7 kernel under the operator name the reference model calls,
// `torch.ops.rwkv7_state_fwd_fp16.forward(B, T, C, H, state, r, w, k, v, a, b, y)`
// (schema as at reference/cuda/rwkv7_state_fwd_fp16.cpp:8-14; call sites reference/rwkv7.py:48, :64), so that the
// unmodified reference resolves to this library once the shim is loaded instead of its own JIT-built extension.
// Differences from the reference binding: the tensors are checked (CUDA, dtype, contiguity, sizes) and errors raise,
// and the kernel runs on torch's CURRENT stream of the tensors' device, not on the legacy default stream.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "../../include/albatross_b200.h"

namespace {

void check(const at::Tensor& t, const char* name, at::ScalarType dt, int64_t numel) {
    TORCH_CHECK(t.is_cuda(), "rwkv7_state_fwd_fp16.forward: ", name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == dt, "rwkv7_state_fwd_fp16.forward: ", name, " has the wrong dtype");
    TORCH_CHECK(t.is_contiguous(), "rwkv7_state_fwd_fp16.forward: ", name, " must be contiguous");
    TORCH_CHECK(t.numel() == numel, "rwkv7_state_fwd_fp16.forward: ", name, " has ", t.numel(), " elements, expected ", numel);
}

void forward(int64_t B, int64_t T, int64_t C, int64_t H, at::Tensor& state, at::Tensor& r, at::Tensor& w,
             at::Tensor& k, at::Tensor& v, at::Tensor& a, at::Tensor& b, at::Tensor& y) {
    TORCH_CHECK(B > 0 && T > 0 && H > 0 && C == H * 64, "rwkv7_state_fwd_fp16.forward: need C == H * 64");
    check(state, "state", at::kFloat, B * H * 64 * 64);
    const int64_t n = B * T * C;
    check(r, "r", at::kHalf, n); check(w, "w", at::kHalf, n); check(k, "k", at::kHalf, n); check(v, "v", at::kHalf, n);
    check(a, "a", at::kHalf, n); check(b, "b", at::kHalf, n); check(y, "y", at::kHalf, n);
    const c10::cuda::CUDAGuard guard(state.device());
    const int st = ab_wkv7_fwd((int)B, (int)T, (int)C, (int)H, state.data_ptr<float>(), r.data_ptr(), w.data_ptr(), k.data_ptr(),
                               v.data_ptr(), a.data_ptr(), b.data_ptr(), y.data_ptr(),
                               (void*)at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(st == AB_OK, "rwkv7_state_fwd_fp16.forward: ", ab_last_error());
}

}  // namespace

TORCH_LIBRARY(rwkv7_state_fwd_fp16, m) { m.def("forward", forward); }
