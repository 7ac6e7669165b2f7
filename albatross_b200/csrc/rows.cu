// Row-wise glue of the batched path: embedding gather, layer norm, token-shift lerps.
//
// Restates, for [B,T,D] activations, reference/rwkv7.py:195 (embedding gather), :203/:213/:219
// (layer norms) and :280-281 / :319-320 (token shift + lerps). One block per row; fp16 in and
// out with the reference's rounding points (each torch op on an fp16 tensor rounds once).
#include "rows.cuh"

namespace ab {

namespace {

constexpr int RT = 256;

__device__ __forceinline__ float block_sum_rt(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < RT / 32; ++i) t += red[i];
    return t;
}

__global__ void __launch_bounds__(RT) gather_rows_kernel(const __half* __restrict__ table, const int* __restrict__ idx,
                                                         int D, __half* __restrict__ out) {
    const size_t m = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)idx[m] * D);
    uint4* dst = reinterpret_cast<uint4*>(out + m * D);
    for (int i = threadIdx.x; i < D / 8; i += RT) dst[i] = src[i];
}

// out[m] = LN(x[src_row(m)]) with src_row = m * stride + offset (stride/offset pick last tokens).
__global__ void __launch_bounds__(RT) ln_rows_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                     const __half* __restrict__ b, int D, int stride, int offset,
                                                     __half* __restrict__ out) {
    __shared__ float red[RT / 32];
    const size_t m = blockIdx.x;
    const __half* xr = x + (m * stride + offset) * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += RT) s += __half2float(xr[i]);
    const float mean = block_sum_rt(s, red) / (float)D;
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += RT) {
        const float d = __half2float(xr[i]) - mean;
        q += d * d;
    }
    const float rstd = rsqrtf(block_sum_rt(q, red) / (float)D + 1e-5f);
    for (int i = threadIdx.x; i < D; i += RT)
        out[m * D + i] = __float2half_rn((__half2float(xr[i]) - mean) * rstd * __half2float(w[i]) + __half2float(b[i]));
}

// For row m = (b, t): prev = t ? xn[m-1] : x_prev[b];  out_c[m] = xn[m] + (prev - xn[m]) * mix_c.
// With T == 1 the same block also stores the new token-shift state (x_prev[b] = xn[m]).
__global__ void __launch_bounds__(RT) mix_rows_kernel(MixParams p) {
    const size_t m = blockIdx.x;
    const int b = (int)(m / p.T), t = (int)(m % p.T);
    const __half* cur = p.xn + m * p.D;
    const __half* prev = t ? cur - p.D : p.x_prev + (size_t)b * p.D;
    for (int i = threadIdx.x; i < p.D; i += RT) {
        const float c = __half2float(cur[i]);
        const float d = rh(__half2float(prev[i]) - c);
        for (int j = 0; j < p.n_mix; ++j)
            p.out[j][m * p.D + i] = __float2half_rn(c + rh(d * __half2float(p.mix[j][i])));
        if (p.T == 1) p.x_prev[(size_t)b * p.D + i] = cur[i];
    }
}

// x_prev[b] = xn[b, T-1]
__global__ void __launch_bounds__(RT) last_rows_kernel(const __half* __restrict__ xn, int T, int D, __half* __restrict__ x_prev) {
    const size_t b = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(xn + (b * T + T - 1) * D);
    uint4* dst = reinterpret_cast<uint4*>(x_prev + b * D);
    for (int i = threadIdx.x; i < D / 8; i += RT) dst[i] = src[i];
}

}  // namespace

int gather_rows(const __half* table, const int* idx, int rows, int D, __half* out, cudaStream_t s) {
    AB_CHECK_ARG(table && idx && out && rows > 0 && D % 8 == 0, "gather_rows: bad argument");
    gather_rows_kernel<<<rows, RT, 0, s>>>(table, idx, D, out);
    AB_CUDA(cudaGetLastError());
    return OK;
}
int ln_rows(const __half* x, const __half* w, const __half* b, int rows, int D, int stride, int offset, __half* out,
            cudaStream_t s) {
    AB_CHECK_ARG(x && w && b && out && rows > 0, "ln_rows: bad argument");
    ln_rows_kernel<<<rows, RT, 0, s>>>(x, w, b, D, stride, offset, out);
    AB_CUDA(cudaGetLastError());
    return OK;
}
int mix_rows(const MixParams& p, cudaStream_t s) {
    AB_CHECK_ARG(p.xn && p.x_prev && p.n_mix >= 1 && p.n_mix <= 6 && p.B > 0 && p.T > 0, "mix_rows: bad argument");
    mix_rows_kernel<<<p.B * p.T, RT, 0, s>>>(p);
    AB_CUDA(cudaGetLastError());
    if (p.T > 1) {
        last_rows_kernel<<<p.B, RT, 0, s>>>(p.xn, p.T, p.D, p.x_prev);
        AB_CUDA(cudaGetLastError());
    }
    return OK;
}

}  // namespace ab
