// Row-wise glue kernels of the batched path (see rows.cu).
#pragma once
#include "common.cuh"

namespace ab {

struct MixParams {
    const __half* xn;     // [B*T, D] normalised activations
    __half* x_prev;       // [B, D] token-shift state, replaced by the last row of each sequence
    const __half* mix[6]; // lerp vectors [D]
    __half* out[6];       // [B*T, D] each
    int n_mix, B, T, D;
};

int gather_rows(const __half* table, const int* idx, int rows, int D, int vocab, __half* out, cudaStream_t s);
int ln_rows(const __half* x, const __half* w, const __half* b, int rows, int D, int stride, int offset, __half* out,
            cudaStream_t s);
int mix_rows(const MixParams& p, cudaStream_t s);
int sample_rows(const __half* logits, int rows, int V, float noise, uint32_t seed, void* out, bool out_i64, cudaStream_t s);
// Layer norm of x (weights w, b) fused with the lerps, for T == 1 (p.xn is not used).
bool ln_mix_rows_ok(const MixParams& p);
int ln_mix_rows(const __half* x, const __half* w, const __half* b, const MixParams& p, cudaStream_t s, bool pdl = false);

}  // namespace ab
