// Batch-1 weight-streaming matrix-vector product for sm_100a.
//
// Replaces the reference's fp16 `x @ W` GEMV call sites at batch 1
// (reference/rwkv7.py:230-235, :240, :250 time-mix; :308-309 channel-mix; :156 vocabulary head)
// with ONE fused launch per group of matrices that share an input:
//   prologue : optional embedding gather, layer norm (reference/rwkv7.py:140,150,155) and the
//              token-shift lerps (reference/rwkv7.py:227-228, :306-307), computed per block in smem;
//   stream   : every warp owns a private ring of shared-memory stages filled by 1-D bulk (TMA)
//              copies that complete on mbarriers; rows are K-contiguous, so each stage is a few
//              contiguous runs of HBM; the issue cursor runs `stages` tiles ahead of the consumer;
//   math     : int8 rows  -> dp4a against x split into a signed high byte and an unsigned low byte
//                            of a 16-bit fixed-point value (one scale per 512 inputs), exact integer sums;
//              NVFP4 rows -> e2m1 pairs converted in registers to half2, one e4m3 scale per 16 inputs;
//              fp16 rows  -> fp32 FMA (low-rank adapter down-projections ride along as extra rows);
//   epilogue : warp-shuffle reduction, row / tensor scale, activation or residual add, fp16 store.
#include "gemv.cuh"

namespace ab {

namespace {

struct Cursor {
    int s, g, kc;  // segment, row group inside the segment, K chunk
};

struct BlockPlan {
    int g_lo[GEMV_MAX_SEG], g_hi[GEMV_MAX_SEG];  // this block's row-group range inside each segment
    int nkc;
};

__device__ __forceinline__ void cursor_settle(const GemvParams& p, const BlockPlan& bp, Cursor& c, int warp) {
    while (c.s < p.nseg && c.g >= bp.g_hi[c.s]) {
        ++c.s;
        if (c.s < p.nseg) c.g = bp.g_lo[c.s] + warp;
    }
}
__device__ __forceinline__ void cursor_next(const GemvParams& p, const BlockPlan& bp, Cursor& c, int warp) {
    if (++c.kc == bp.nkc) {
        c.kc = 0;
        c.g += GEMV_WARPS;
        cursor_settle(p, bp, c, warp);
    }
}

// Issue the bulk copies of one tile into a stage. Called by the whole warp; lanes < rows issue.
__device__ __forceinline__ void issue_tile(const GemvParams& p, const Cursor& c, unsigned char* stage, uint64_t* bar,
                                           int lane, uint64_t policy) {
    const GemvSeg& sg = p.seg[c.s];
    const int R = gemv_rows_per_group(sg.fmt);
    const int row0 = c.g * R;
    const int rows = min(R, sg.n_rows - row0);
    const int k0 = c.kc * GEMV_TILE_K;
    const int kn = min(GEMV_TILE_K, p.K - k0);
    const int row_bytes = gemv_row_bytes(sg.fmt, p.K);
    const int off_bytes = gemv_row_bytes(sg.fmt, k0);
    const int cp_bytes = gemv_row_bytes(sg.fmt, kn);
    const int tile_row_stride = GEMV_TILE_BYTES / R;
    const int sc_bytes = (sg.fmt == FMT_FP4) ? kn / 16 : 0;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(rows * (cp_bytes + sc_bytes)));
    __syncwarp();
    if (lane < rows) {
        const unsigned char* src = (const unsigned char*)sg.w + (size_t)(row0 + lane) * row_bytes + off_bytes;
        bulk_g2s_hint(stage + lane * tile_row_stride, src, (uint32_t)cp_bytes, bar, policy);
        if (sc_bytes) {
            const unsigned char* ssrc = (const unsigned char*)sg.scale + (size_t)(row0 + lane) * (p.K / 16) + k0 / 16;
            bulk_g2s_hint(stage + GEMV_TILE_BYTES + lane * 64, ssrc, (uint32_t)sc_bytes, bar, policy);
        }
    }
}

__device__ __forceinline__ float block_sum(float v, float* red, int tid) {
    v = warp_sum(v);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < GEMV_WARPS; ++i) t += red[i];
    return t;
}

__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_stream_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = p.K;
    const int Kp = (K + 511) & ~511;
    const int S = p.stages;

    // ---- shared memory carve-up
    unsigned char* ring = smem + (size_t)warp * S * GEMV_STAGE_BYTES;
    size_t off = (size_t)GEMV_WARPS * S * GEMV_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off) + warp * S;
    off += (size_t)GEMV_WARPS * S * 8;
    off = (off + 127) & ~(size_t)127;
    __half* xn = reinterpret_cast<__half*>(smem + off);
    off += (size_t)Kp * 2;
    signed char* xh = reinterpret_cast<signed char*>(smem + off);
    unsigned char* xl = smem + off + Kp;
    if (p.smem_flags & 1) off += (size_t)Kp * 2;
    __half* xf = reinterpret_cast<__half*>(smem + off);
    if (p.smem_flags & 2) off += (size_t)Kp * 2;
    __half* dx = reinterpret_cast<__half*>(smem + off);
    if (p.smem_flags & 4) off += (size_t)Kp * 2;
    float* sx = reinterpret_cast<float*>(smem + off);
    off += (size_t)(Kp / 512) * 4;
    float* red = reinterpret_cast<float*>(smem + off);

    // ---- this block's share of every segment (contiguous run of row groups, split evenly)
    BlockPlan bp;
    bp.nkc = (K + GEMV_TILE_K - 1) / GEMV_TILE_K;
    {
        int total = 0;
        for (int s = 0; s < p.nseg; ++s)
            total += (p.seg[s].n_rows + gemv_rows_per_group(p.seg[s].fmt) - 1) / gemv_rows_per_group(p.seg[s].fmt);
        const int G0 = (int)(((long long)total * blockIdx.x) / gridDim.x);
        const int G1 = (int)(((long long)total * (blockIdx.x + 1)) / gridDim.x);
        int base = 0;
        for (int s = 0; s < GEMV_MAX_SEG; ++s) {
            if (s < p.nseg) {
                const int R = gemv_rows_per_group(p.seg[s].fmt);
                const int n = (p.seg[s].n_rows + R - 1) / R;
                bp.g_lo[s] = max(G0, base) - base;
                bp.g_hi[s] = min(G1, base + n) - base;
                base += n;
            } else {
                bp.g_lo[s] = 0;
                bp.g_hi[s] = 0;
            }
        }
    }

    if (lane == 0) {
        for (int i = 0; i < S; ++i) mbar_init(&bars[i], 1);
        fence_mbar_init();
    }
    __syncwarp();

    // ---- start streaming weights before anything that depends on the previous kernel
    const uint64_t policy = policy_evict_first();
    Cursor ci{0, bp.g_lo[0] + warp, 0};
    cursor_settle(p, bp, ci, warp);
    Cursor cc = ci;
    for (int i = 0; i < S; ++i) {
        if (ci.s < p.nseg) {
            issue_tile(p, ci, ring + (size_t)i * GEMV_STAGE_BYTES, &bars[i], lane, policy);
            cursor_next(p, bp, ci, warp);
        }
    }

    if (p.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }

    if (p.copy_src && blockIdx.x == 0)
        for (int i = tid; i < p.copy_n / 8; i += GEMV_THREADS)
            reinterpret_cast<uint4*>(p.copy_dst)[i] = reinterpret_cast<const uint4*>(p.copy_src)[i];

    // ---- phase A: input vector, optional layer norm, token-shift difference
    const __half* xin = p.emb ? p.emb + (size_t)p.token[0] * K : p.x;
    for (int i = tid; i < K / 8; i += GEMV_THREADS) {
        uint4 v = reinterpret_cast<const uint4*>(xin)[i];
        reinterpret_cast<uint4*>(xn)[i] = v;
        if (p.x_copy && blockIdx.x == 0) reinterpret_cast<uint4*>(p.x_copy)[i] = v;
    }
    __syncthreads();
    if (p.ln_w) {
        float s = 0.f;
        for (int i = tid; i < K; i += GEMV_THREADS) s += __half2float(xn[i]);
        const float mean = block_sum(s, red, tid) / (float)K;
        float q = 0.f;
        for (int i = tid; i < K; i += GEMV_THREADS) {
            const float d = __half2float(xn[i]) - mean;
            q += d * d;
        }
        const float var = block_sum(q, red, tid) / (float)K;
        const float rstd = rsqrtf(var + 1e-5f);
        for (int i = tid; i < K; i += GEMV_THREADS) {
            const float v = (__half2float(xn[i]) - mean) * rstd * __half2float(p.ln_w[i]) + __half2float(p.ln_b[i]);
            const __half hv = __float2half_rn(v);
            xn[i] = hv;
            if (p.ln_out && blockIdx.x == 0) p.ln_out[i] = hv;
        }
    }
    if (p.smem_flags & 4) {
        __syncthreads();
        for (int i = tid; i < K; i += GEMV_THREADS)
            dx[i] = __float2half_rn(__half2float(p.x_prev[i]) - __half2float(xn[i]));
    }
    __syncthreads();

    uint32_t n_consumed = 0;  // tiles this warp has consumed (stage = n % S, parity = (n / S) & 1)
    bool failed = false;

    for (int s = 0; s < p.nseg; ++s) {
        if (bp.g_lo[s] >= bp.g_hi[s]) continue;  // block-uniform
        const GemvSeg& sg = p.seg[s];
        const int fmt = sg.fmt;

        // ---- phase B: the segment's input in the form its rows consume
        for (int c0 = warp * 32; c0 < Kp / 16; c0 += GEMV_THREADS) {
            const int c = c0 + lane;          // 16-element chunk
            const bool in = c * 16 < K;
            float v[16];
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                float t = 0.f;
                if (in) {
                    const int i = c * 16 + e;
                    t = __half2float(xn[i]);
                    if (sg.mix) t = rh(t + rh(__half2float(dx[i]) * __half2float(sg.mix[i])));
                }
                v[e] = t;
            }
            if (fmt != FMT_I8) {
                if (in) {
                    __half2 h[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                    reinterpret_cast<uint4*>(xf)[c * 2] = *reinterpret_cast<uint4*>(&h[0]);
                    reinterpret_cast<uint4*>(xf)[c * 2 + 1] = *reinterpret_cast<uint4*>(&h[4]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    if (sg.col_scale && in) v[e] *= sg.col_scale[c * 16 + e];
                    amax = fmaxf(amax, fabsf(v[e]));
                }
                amax = warp_max(amax);  // one scale per 512 inputs = the 32 chunks of this warp pass
                const float inv = amax > 0.f ? 32767.0f / amax : 0.f;
                uint32_t hw[4], lw[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t hh = 0, ll = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int X = __float2int_rn(v[q * 4 + e] * inv);
                        hh |= (uint32_t)((X >> 8) & 0xff) << (8 * e);
                        ll |= (uint32_t)(X & 0xff) << (8 * e);
                    }
                    hw[q] = hh;
                    lw[q] = ll;
                }
                reinterpret_cast<uint4*>(xh)[c] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                reinterpret_cast<uint4*>(xl)[c] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                if (lane == 0) sx[c0 / 32] = amax / 32767.0f;
            }
        }
        __syncthreads();

        // ---- stream this warp's row groups of the segment
        const int R = gemv_rows_per_group(fmt);
        while (cc.s == s) {
            float acc[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) acc[r] = 0.f;
            const int g = cc.g;
            for (int kc = 0; kc < bp.nkc; ++kc) {
                const uint32_t st = n_consumed % S;
                unsigned char* tile = ring + (size_t)st * GEMV_STAGE_BYTES;
                if (!failed && !mbar_wait_bounded(&bars[st], (n_consumed / S) & 1)) {
                    failed = true;
                    if (lane == 0) atomicOr(&g_device_status, DEV_WAIT_GEMV);
                }
                const int k0 = kc * GEMV_TILE_K;
                if (fmt == FMT_I8) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int k = k0 + j * 512 + lane * 16;
                        if (k < K) {
                            const uint4 a = *reinterpret_cast<const uint4*>(xh + k);
                            const uint4 b = *reinterpret_cast<const uint4*>(xl + k);
                            const float sc = sx[(k0 + j * 512) >> 9];
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                const uint4 w = *reinterpret_cast<const uint4*>(tile + r * 1024 + j * 512 + lane * 16);
                                int ah = dp4a_ss(w.x, a.x, 0);
                                ah = dp4a_ss(w.y, a.y, ah);
                                ah = dp4a_ss(w.z, a.z, ah);
                                ah = dp4a_ss(w.w, a.w, ah);
                                int al = dp4a_su(w.x, b.x, 0);
                                al = dp4a_su(w.y, b.y, al);
                                al = dp4a_su(w.z, b.z, al);
                                al = dp4a_su(w.w, b.w, al);
                                acc[r] = fmaf((float)(ah * 256 + al), sc, acc[r]);
                            }
                        }
                    }
                } else if (fmt == FMT_F16) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int k = k0 + j * 256 + lane * 8;
                        if (k < K) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xf + k);
                            const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                            for (int r = 0; r < 2; ++r) {
                                const uint4 wv = *reinterpret_cast<const uint4*>(tile + r * 2048 + j * 512 + lane * 16);
                                const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 wf = __half22float2(w2[e]);
                                    const float2 xq = __half22float2(x2[e]);
                                    acc[r] = fmaf(wf.x, xq.x, acc[r]);
                                    acc[r] = fmaf(wf.y, xq.y, acc[r]);
                                }
                            }
                        }
                    }
                } else {  // FMT_FP4
                    const int k = k0 + lane * 32;
                    if (k < K) {
                        uint4 xv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) xv[e] = *reinterpret_cast<const uint4*>(xf + k + e * 8);
                        const __half2* x2 = reinterpret_cast<const __half2*>(xv);
#pragma unroll
                        for (int r = 0; r < 8; ++r) {
                            const uint4 wv = *reinterpret_cast<const uint4*>(tile + r * 512 + lane * 16);
                            const uint32_t sc2 = *reinterpret_cast<const unsigned short*>(tile + GEMV_TILE_BYTES + r * 64 + lane * 2);
                            const float2 scf = __half22float2(e4m3x2_to_half2(sc2));
                            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                            for (int b = 0; b < 2; ++b) {
                                __half2 h = __floats2half2_rn(0.f, 0.f);
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const uint32_t byte = (ww[b * 2 + (e >> 2)] >> (8 * (e & 3))) & 0xffu;
                                    h = __hfma2(e2m1x2_to_half2(byte), x2[b * 8 + e], h);
                                }
                                const float2 hf = __half22float2(h);
                                acc[r] = fmaf(hf.x + hf.y, b ? scf.y : scf.x, acc[r]);
                            }
                        }
                    }
                }
                __syncwarp();
                ++n_consumed;
                // refill the stage just drained with the tile `S` ahead
                if (ci.s < p.nseg) {
                    issue_tile(p, ci, tile, &bars[st], lane, policy);
                    cursor_next(p, bp, ci, warp);
                }
            }
            // ---- epilogue for the R rows of this group
#pragma unroll
            for (int r = 0; r < 8; ++r) acc[r] = warp_sum(acc[r]);
            const int row = g * R + lane;
            if (lane < R && row < sg.n_rows) {
                float val = 0.f;
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r == lane) val = acc[r];
                if (fmt == FMT_I8) val *= reinterpret_cast<const float*>(sg.scale)[row];
                else if (fmt == FMT_FP4) val *= sg.tscale;
                float o = rh(val);
                switch (sg.epi) {
                    case EPI_TANH: o = tanhf(o); break;
                    case EPI_SIGMOID: o = sigmoidf_(o); break;
                    case EPI_RELU2: o = fmaxf(o, 0.f); o = o * o; break;
                    case EPI_RESID: o = __half2float(sg.resid[row]) + o; break;
                    default: break;
                }
                sg.out[row] = __float2half_rn(o);
            }
            cc.kc = bp.nkc - 1;
            cursor_next(p, bp, cc, warp);
        }
        __syncthreads();  // all warps are done with this segment's x before it is rebuilt
    }
}

}  // namespace

size_t gemv_smem_bytes(const GemvParams& p) {
    const size_t Kp = ((size_t)p.K + 511) & ~(size_t)511;
    size_t off = (size_t)GEMV_WARPS * p.stages * GEMV_STAGE_BYTES + (size_t)GEMV_WARPS * p.stages * 8;
    off = (off + 127) & ~(size_t)127;
    off += Kp * 2;
    if (p.smem_flags & 1) off += Kp * 2;
    if (p.smem_flags & 2) off += Kp * 2;
    if (p.smem_flags & 4) off += Kp * 2;
    off += (Kp / 512) * 4 + 64 * 4;
    return off;
}

int gemv_launch(const GemvParams& p_in, cudaStream_t stream) {
    GemvParams p = p_in;
    AB_CHECK_ARG(p.nseg >= 1 && p.nseg <= GEMV_MAX_SEG, "gemv: nseg %d out of range", p.nseg);
    AB_CHECK_ARG(p.K >= 16 && p.K % 16 == 0 && p.K <= 32768, "gemv: K=%d must be a multiple of 16 in [16, 32768]", p.K);
    int groups = 0;
    p.smem_flags = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const GemvSeg& g = p.seg[s];
        p.smem_flags |= (g.fmt == FMT_I8 ? 1 : 2) | (g.mix ? 4 : 0);
        AB_CHECK_ARG(g.w && g.out && g.n_rows > 0, "gemv: segment %d has a null pointer or no rows", s);
        AB_CHECK_ARG(((uintptr_t)g.w & 15) == 0, "gemv: segment %d weights not 16-byte aligned", s);
        AB_CHECK_ARG(g.fmt == FMT_F16 || g.scale, "gemv: segment %d needs scales", s);
        AB_CHECK_ARG(g.fmt != FMT_FP4 || (((uintptr_t)g.scale & 15) == 0 && p.K % 256 == 0),
                     "gemv: segment %d: NVFP4 needs 16-byte aligned block scales and K %% 256 == 0", s);
        AB_CHECK_ARG(g.epi != EPI_RESID || g.resid, "gemv: segment %d residual missing", s);
        const int R = gemv_rows_per_group(g.fmt);
        groups += (g.n_rows + R - 1) / R;
    }
    AB_CHECK_ARG(p.emb || p.x, "gemv: no input vector");
    AB_CHECK_ARG(!(p.smem_flags & 4) || p.x_prev, "gemv: token-shift state missing");
    if (p.stages <= 0) p.stages = 4;
    static int n_sm = 0;
    static size_t max_smem = 0;
    if (!n_sm) {
        int dev = 0, v = 0;
        AB_CUDA(cudaGetDevice(&dev));
        AB_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        int m = 0;
        AB_CUDA(cudaDeviceGetAttribute(&m, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        AB_CUDA(cudaFuncSetAttribute(gemv_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, m));
        max_smem = (size_t)m;
        n_sm = v;
    }
    size_t smem = gemv_smem_bytes(p);
    while (smem > max_smem && p.stages > 2) {
        --p.stages;
        smem = gemv_smem_bytes(p);
    }
    AB_CHECK_ARG(smem <= max_smem, "gemv: K=%d needs %zu bytes of shared memory", p.K, smem);
    const int grid = max(1, min(n_sm, (groups + GEMV_WARPS - 1) / GEMV_WARPS));

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.use_pdl ? 1 : 0;
    AB_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel, p));
    return OK;
}

}  // namespace ab
