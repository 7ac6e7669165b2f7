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
                                                         int D, int vocab, __half* __restrict__ out) {
    const size_t m = blockIdx.x;
    int tok = idx[m];
    if ((unsigned)tok >= (unsigned)vocab) {   // never index past the table: clamp and tell the host
        tok = tok < 0 ? 0 : vocab - 1;
        if (threadIdx.x == 0) atomicOr(&g_device_status, DEV_BAD_TOKEN);
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * D);
    uint4* dst = reinterpret_cast<uint4*>(out + m * D);
    for (int i = threadIdx.x; i < D / 8; i += RT)
        if (AB_BC(tok >= 0 && tok < vocab && (i + 1) * 8 <= D)) dst[i] = src[i];
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

// T == 1: layer norm and token-shift lerps of one row in one pass; the row stays in registers (16-byte loads and
// stores), the normalised row becomes the new token-shift state. Same rounding points as ln_rows + mix_rows.
constexpr int LM_MAXV = 4;   // 16-byte chunks per thread: D <= 8 * RT * LM_MAXV
__global__ void __launch_bounds__(RT) ln_mix_rows_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                         const __half* __restrict__ b, const __grid_constant__ MixParams p,
                                                         int use_pdl) {
    __shared__ float red[RT / 32];
    const size_t m = blockIdx.x;
    const int nv = p.D / 8;
    const uint4* xr = reinterpret_cast<const uint4*>(x + m * p.D);
    uint4 raw[LM_MAXV], prv[LM_MAXV], wv_[LM_MAXV], bv_[LM_MAXV];
    float s = 0.f;
    // everything that does not depend on the row statistics is requested up front (norm weights into registers, the
    // lerp vectors into L1), so that the two block reductions are the only waits after the first load. Under
    // programmatic stream serialisation the parameters are requested while the preceding kernel still runs, and the
    // next kernel (a product, which starts with its weight stream) may start at once.
    if (use_pdl) pdl_launch_dependents();
#pragma unroll
    for (int v = 0; v < LM_MAXV; ++v) {
        const int i = threadIdx.x + v * RT;
        if (i < nv) {
            wv_[v] = reinterpret_cast<const uint4*>(w)[i];
            bv_[v] = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
            for (int j = 0; j < 6; ++j)
                if (j < p.n_mix) asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const uint4*>(p.mix[j]) + i));
        }
    }
    if (use_pdl) pdl_wait();
#pragma unroll
    for (int v = 0; v < LM_MAXV; ++v) {
        const int i = threadIdx.x + v * RT;
        if (i < nv) {
            // an ordinary (coherent) load that stays behind the wait above: the row was written by the preceding kernel
            asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(raw[v].x), "=r"(raw[v].y), "=r"(raw[v].z), "=r"(raw[v].w)
                         : "l"(xr + i)
                         : "memory");
            prv[v] = reinterpret_cast<const uint4*>(p.x_prev + m * p.D)[i];
            const __half2* h = reinterpret_cast<const __half2*>(&raw[v]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); s += f.x + f.y; }
        }
    }
    const float mean = block_sum_rt(s, red) / (float)p.D;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < LM_MAXV; ++v) {
        if (threadIdx.x + v * RT < nv) {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[v]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                q += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
            }
        }
    }
    const float rstd = rsqrtf(block_sum_rt(q, red) / (float)p.D + 1e-5f);
#pragma unroll
    for (int v = 0; v < LM_MAXV; ++v) {
        const int i = threadIdx.x + v * RT;
        if (i < nv) {
            const uint4 wv = wv_[v], bv = bv_[v];
            const __half2* h = reinterpret_cast<const __half2*>(&raw[v]);
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
            const __half2* bh = reinterpret_cast<const __half2*>(&bv);
            const __half2* ph = reinterpret_cast<const __half2*>(&prv[v]);
            uint4 xn;
            __half2* xh = reinterpret_cast<__half2*>(&xn);
            float c[8], d[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]), wf = __half22float2(wh[e]), bf = __half22float2(bh[e]);
                xh[e] = __floats2half2_rn((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
                const float2 cf = __half22float2(xh[e]), pf = __half22float2(ph[e]);
                c[2 * e] = cf.x; c[2 * e + 1] = cf.y;
                d[2 * e] = rh(pf.x - cf.x); d[2 * e + 1] = rh(pf.y - cf.y);
            }
            reinterpret_cast<uint4*>(p.x_prev + m * p.D)[i] = xn;
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                if (j < p.n_mix) {
                    const uint4 mv = reinterpret_cast<const uint4*>(p.mix[j])[i];
                    const __half2* mh = reinterpret_cast<const __half2*>(&mv);
                    uint4 o;
                    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 mf = __half22float2(mh[e]);
                        oh[e] = __floats2half2_rn(c[2 * e] + rh(d[2 * e] * mf.x), c[2 * e + 1] + rh(d[2 * e + 1] * mf.y));
                    }
                    reinterpret_cast<uint4*>(p.out[j] + m * p.D)[i] = o;
                }
            }
        }
    }
}

// Greedy / noisy-greedy sampling of one token per row: argmax over the row of logit + U(0, noise)
// (reference/utils.py:43-45 adds uniform noise and takes the first entry of a descending argsort). Ties go to the
// lowest index. The noise is a counter-based hash of (seed, row, column): reproducible, not torch's generator.
__device__ __forceinline__ float sample_noise(uint32_t seed, uint32_t row, uint32_t col) {
    uint32_t x = seed ^ (row * 0x9E3779B9u) ^ (col * 0x85EBCA6Bu);
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    return (float)(x >> 8) * (1.0f / 16777216.0f);   // [0, 1)
}
// NT threads per row: 1024 when there are only a few rows (a single row of 65536 logits is otherwise read by 256 threads,
// 32 loads one after the other: 16 us), 256 otherwise.
template <class OutT, int NT>
__global__ void __launch_bounds__(NT) sample_rows_kernel(const __half* __restrict__ logits, int V, float noise, uint32_t seed,
                                                         OutT* __restrict__ out) {
    __shared__ float bv[NT / 32];
    __shared__ int bi[NT / 32];
    const size_t row = blockIdx.x;
    const __half* lr = logits + row * V;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (noise > 0.f) v += noise * sample_noise(seed, (uint32_t)row, (uint32_t)i);
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    };
    const int nv = (V % 8 == 0 && ((uintptr_t)lr & 15) == 0) ? V / 8 : 0;
#pragma unroll 4
    for (int c = threadIdx.x; c < nv; c += NT) {
        const uint4 q = reinterpret_cast<const uint4*>(lr)[c];
        const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            take(f.x, c * 8 + 2 * e);
            take(f.y, c * 8 + 2 * e + 1);
        }
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += NT) take(__half2float(lr[i]), i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < NT / 32; ++w)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        out[row] = (OutT)idx;
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

int gather_rows(const __half* table, const int* idx, int rows, int D, int vocab, __half* out, cudaStream_t s) {
    AB_CHECK_ARG(table && idx && out && rows > 0 && D % 8 == 0 && vocab > 0, "gather_rows: bad argument");
    gather_rows_kernel<<<rows, RT, 0, s>>>(table, idx, D, vocab, out);
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
bool ln_mix_rows_ok(const MixParams& p) { return p.T == 1 && p.D % 8 == 0 && p.D <= 8 * RT * LM_MAXV; }
int ln_mix_rows(const __half* x, const __half* w, const __half* b, const MixParams& p, cudaStream_t s, bool pdl) {
    AB_CHECK_ARG(x && w && b && p.x_prev && p.n_mix >= 1 && p.n_mix <= 6 && p.B > 0 && ln_mix_rows_ok(p), "ln_mix_rows: bad argument");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.B);
    cfg.blockDim = dim3(RT);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    AB_CUDA(cudaLaunchKernelEx(&cfg, ln_mix_rows_kernel, x, w, b, p, pdl ? 1 : 0));
    return OK;
}
int sample_rows(const __half* logits, int rows, int V, float noise, uint32_t seed, void* out, bool out_i64, cudaStream_t s) {
    AB_CHECK_ARG(logits && out && rows > 0 && V > 0 && noise >= 0.f, "sample_rows: bad argument");
    if (rows <= 16) {
        if (out_i64) sample_rows_kernel<long long, 1024><<<rows, 1024, 0, s>>>(logits, V, noise, seed, (long long*)out);
        else sample_rows_kernel<int, 1024><<<rows, 1024, 0, s>>>(logits, V, noise, seed, (int*)out);
    } else {
        if (out_i64) sample_rows_kernel<long long, RT><<<rows, RT, 0, s>>>(logits, V, noise, seed, (long long*)out);
        else sample_rows_kernel<int, RT><<<rows, RT, 0, s>>>(logits, V, noise, seed, (int*)out);
    }
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
