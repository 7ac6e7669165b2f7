// Batched matrix product Y[rows, n_out] = X[rows, k] * W^T with fused de-quantisation (see gemm.cu).
#pragma once
#include "../../include/albatross_b200.h"
#include "common.cuh"

namespace ab {

size_t gemm_scratch_bytes(const ab_mat& m, int rows);
int gemm_launch(const ab_mat& m, int rows, const __half* x, __half* y, int epi, const __half* resid, void* scratch,
                cudaStream_t stream);
int dequant_launch(const ab_mat& m, float* out, cudaStream_t stream);
int check_mat(const ab_mat& m, const char* what);

}  // namespace ab
