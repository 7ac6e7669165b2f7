// Batched matrix product Y[rows, n_out] = X[rows, k] * W^T with fused de-quantisation (see gemm.cu).
#pragma once
#include "../../include/albatross_b200.h"
#include "common.cuh"

namespace ab {

// One product of a grouped launch: Y[rows, n_out] = epilogue(X[rows, k] * W^T).
struct GemmOp {
    ab_mat w;
    const __half* x;
    __half* y;
    const __half* resid;
    int epi;
};
// Scratch: split-K arrival counters and fp32 partial tiles. It must be zero when first used; the kernels
// leave the counters at zero again.
size_t gemm_group_scratch_bytes(const GemmOp* ops, int n, int rows);
// pdl: launch with programmatic stream serialisation (the kernel waits for the preceding grid itself, after it has
// started its weight stream).
int gemm_group_launch(const GemmOp* ops, int n, int rows, void* scratch, cudaStream_t stream, bool pdl = false);
size_t gemm_scratch_bytes(const ab_mat& m, int rows);
int static_scratch_reset(cudaStream_t stream);   // built-in scratch of ab_gemm_static: counters back to zero
int gemm_launch(const ab_mat& m, int rows, const __half* x, __half* y, int epi, const __half* resid, void* scratch,
                cudaStream_t stream, bool pdl = false);
int dequant_launch(const ab_mat& m, float* out, cudaStream_t stream);
int check_mat(const ab_mat& m, const char* what);

}  // namespace ab
