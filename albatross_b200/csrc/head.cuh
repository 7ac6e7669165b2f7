// Parameter block of the fused per-head time-mix kernel (see head.cu).
#pragma once
#include "common.cuh"

namespace ab {

struct HeadParams {
    int B, T, D, H;
    int layer0;     // layer 0 defines v_first instead of mixing towards it (reference/rwkv7.py:239)
    float* state;   // [B,H,64,64] fp32, updated in place
    const __half *r, *k, *v;   // [B*T, D] projections
    __half* v_first;           // [B*T, D]: written by layer 0, read by the others
    // adapter up-projections already applied (batched path): raw sums before bias / activation
    const __half *w_raw, *a_raw, *vg_raw, *g;
    // or: adapter hidden vectors and up-projection matrices [rank, D] (batch-1 path, B = T = 1)
    const __half *hw, *ha, *hv, *hg;
    const __half *w2, *a2, *v2, *g2;
    int rw, ra, rv, rg;
    const __half *w0, *a0, *v0, *k_k, *k_a, *r_k, *lnx_w, *lnx_b;  // [D]
    __half* out;               // [B*T, D]: group-normed, bonus added, gated
    const __half* copy_src;    // optional [D] -> copy_dst (token-shift state hand-over, batch-1 path)
    __half* copy_dst;
    int use_pdl;
    // Persistent batch-1 kernel, dataflow mode: head h is run by block 2h (pair_mode); r, k, v, the adapter hidden
    // vectors and `out` are arrays of tagged words (tag_in / tag_out: 1 + index of the writing phase, 0 = plain fp16).
    int pair_mode, tag_in, tag_out, pad_;
};

int head_launch(const HeadParams& p, cudaStream_t stream);
int wkv7_launch(int B, int T, int C, int H, float* state, const __half* r, const __half* w, const __half* k,
                const __half* v, const __half* a, const __half* b, __half* y, cudaStream_t stream);

}  // namespace ab
