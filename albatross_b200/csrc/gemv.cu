// Batch-1 weight-streaming matrix-vector product for sm_100a.
//
// Replaces the reference's fp16 `x @ W` GEMV call sites at batch 1
// (reference/rwkv7.py:230-235, :240, :250 time-mix; :308-309 channel-mix; :156 vocabulary head)
// with ONE fused launch per group of matrices that share an input:
//   prologue : optional embedding gather, layer norm (reference/rwkv7.py:140,150,155) and the
//              token-shift lerps (reference/rwkv7.py:227-228, :306-307), computed per block in smem;
//   stream   : one producer warp per block; its lane w feeds consumer warp w's private ring of
//              shared-memory stages with 1-D bulk (TMA) copies that complete on "full" mbarriers;
//              consumers hand stages back through "empty" mbarriers. Rows are K-contiguous, so a
//              stage is a few contiguous runs of HBM. Weights do not depend on the previous kernel,
//              so the producer starts before the programmatic-dependent-launch wait;
//   math     : int8 rows  -> dp4a against x split into a signed high byte and an unsigned low byte
//                            of a 16-bit fixed-point value (one scale per 512 inputs), exact integer sums;
//              NVFP4 rows -> e2m1 pairs converted in registers to half2, one e4m3 scale per 16 inputs;
//              fp16 rows  -> fp32 FMA (low-rank adapter down-projections ride along as extra rows);
//   epilogue : warp-shuffle reduction, row / tensor scale, activation or residual add, fp16 store.
#include "gemv.cuh"

namespace ab {

namespace {

constexpr int NT_CONS = GEMV_WARPS * 32;  // consumer threads

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NT_CONS) : "memory"); }

// this block's row-group range [lo, hi) inside segment s
__device__ __forceinline__ void seg_range(const GemvParams& p, int s, int G0, int G1, int& lo, int& hi) {
    int base = 0;
    for (int i = 0; i < s; ++i) {
        const int R = gemv_rows_per_group(p.seg[i].fmt, p.K);
        base += (p.seg[i].n_rows + R - 1) / R;
    }
    const int R = gemv_rows_per_group(p.seg[s].fmt, p.K);
    const int n = (p.seg[s].n_rows + R - 1) / R;
    lo = max(G0, base) - base;
    hi = min(G1, base + n) - base;
}

__device__ __forceinline__ float cons_block_sum(float v, float* red, int tid) {
    v = warp_sum(v);
    cons_sync();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    cons_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < GEMV_WARPS; ++i) t += red[i];
    return t;
}

// ---- per-format tile consumers: acc[r] += sum over this lane's slice of the tile -----------------
// tile: R rows of `piece` bytes each; the tile covers kn elements of K starting at k0.
template <int RMAX>
__device__ __forceinline__ void consume_i8(const unsigned char* tile, int piece, int R, const signed char* xh,
                                           const unsigned char* xl, const float* sx, int k0, int kn, int lane,
                                           float* acc) {
    for (int j = 0; j * 512 < kn; ++j) {
        const int k = j * 512 + lane * 16;
        if (k < kn) {
            const uint4 a = *reinterpret_cast<const uint4*>(xh + k0 + k);
            const uint4 b = *reinterpret_cast<const uint4*>(xl + k0 + k);
            const float sc = sx[(k0 >> 9) + j];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                if (r < R) {
                    const uint4 w = *reinterpret_cast<const uint4*>(tile + r * piece + k);
                    int ah = dp4a_ss(w.x, a.x, 0);
                    int al = dp4a_su(w.x, b.x, 0);
                    ah = dp4a_ss(w.y, a.y, ah);
                    al = dp4a_su(w.y, b.y, al);
                    ah = dp4a_ss(w.z, a.z, ah);
                    al = dp4a_su(w.z, b.z, al);
                    ah = dp4a_ss(w.w, a.w, ah);
                    al = dp4a_su(w.w, b.w, al);
                    acc[r] = fmaf((float)(ah * 256 + al), sc, acc[r]);
                }
            }
        }
    }
}

template <int RMAX>
__device__ __forceinline__ void consume_f16(const unsigned char* tile, int piece, int R, const __half* xf, int k0,
                                            int kn, int lane, float* acc) {
    for (int j = 0; j * 256 < kn; ++j) {
        const int k = j * 256 + lane * 8;
        if (k < kn) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xf + k0 + k);
            const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                if (r < R) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(tile + r * piece + k * 2);
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
    }
}

template <int RMAX>
__device__ __forceinline__ void consume_fp4(const unsigned char* tile, int piece, int R, const __half* xf, int k0,
                                            int kn, int lane, float* acc) {
    const unsigned char* scales = tile + GEMV_TILE_BYTES;
    const int srow = kn / 16;  // scale bytes per row in this tile
    for (int j = 0; j * 1024 < kn; ++j) {
        const int k = j * 1024 + lane * 32;
        if (k < kn) {
            uint4 xv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) xv[e] = *reinterpret_cast<const uint4*>(xf + k0 + k + e * 8);
            const __half2* x2 = reinterpret_cast<const __half2*>(xv);
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                if (r < R) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(tile + r * piece + k / 2);
                    const uint32_t sc2 = *reinterpret_cast<const unsigned short*>(scales + r * srow + k / 16);
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
    }
}

__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_stream_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = p.K;
    const int Kp = (K + 511) & ~511;
    const int S = p.stages;

    // ---- shared memory carve-up (must match gemv_smem_bytes)
    size_t off = (size_t)GEMV_WARPS * S * GEMV_STAGE_BYTES;
    uint64_t* full_bars = reinterpret_cast<uint64_t*>(smem + off);
    uint64_t* empty_bars = full_bars + GEMV_WARPS * S;
    off += (size_t)GEMV_WARPS * S * 16;
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

    // ---- this block's contiguous run of row groups over the concatenated segments
    int total = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const int R = gemv_rows_per_group(p.seg[s].fmt, K);
        total += (p.seg[s].n_rows + R - 1) / R;
    }
    const int G0 = (int)(((long long)total * blockIdx.x) / gridDim.x);
    const int G1 = (int)(((long long)total * (blockIdx.x + 1)) / gridDim.x);

    if (tid == 0) {
        for (int i = 0; i < GEMV_WARPS * S; ++i) {
            mbar_init(&full_bars[i], 1);
            mbar_init(&empty_bars[i], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == GEMV_WARPS) {
        // ================= producer warp: lane w streams consumer warp w's tiles =================
        if (lane < GEMV_WARPS) {
            const uint64_t policy = policy_evict_first();
            unsigned char* ring = smem + (size_t)lane * S * GEMV_STAGE_BYTES;
            uint64_t* fb = full_bars + lane * S;
            uint64_t* eb = empty_bars + lane * S;
            int slot = 0;
            uint32_t fills = 0;   // tiles issued so far
            uint32_t ephase = 0;  // parity of the empty barrier to wait for once the ring has wrapped
            bool dead = false;
            for (int s = 0; s < p.nseg && !dead; ++s) {
                int lo, hi;
                seg_range(p, s, G0, G1, lo, hi);
                if (lo >= hi) continue;
                const GemvSeg& sg = p.seg[s];
                const GemvGeom gm = gemv_geom(sg.fmt, K);
                const int row_bytes = gemv_row_bytes(sg.fmt, K);
                const int srow_bytes = K / 16;
                for (int g = lo + lane; g < hi && !dead; g += GEMV_WARPS) {
                    const int row0 = g * gm.R;
                    const int rows = min(gm.R, sg.n_rows - row0);
                    const unsigned char* src = (const unsigned char*)sg.w + (size_t)row0 * row_bytes;
                    const unsigned char* ssrc =
                        sg.fmt == FMT_FP4 ? (const unsigned char*)sg.scale + (size_t)row0 * srow_bytes : nullptr;
                    for (int kc = 0; kc < gm.nkc; ++kc) {
                        if (fills >= (uint32_t)S) {  // wait until the consumer has drained this slot
                            uint32_t it = 0;
                            while (!mbar_test_wait(&eb[slot], ephase)) {
                                if (++it > (1u << 24)) {
                                    dead = true;
                                    break;
                                }
                            }
                            if (dead) {
                                atomicOr(&g_device_status, DEV_WAIT_GEMV);
                                break;
                            }
                        }
                        const int k0 = kc * gm.kc;
                        const int kn = min(gm.kc, K - k0);
                        const int cpb = gemv_row_bytes(sg.fmt, kn);
                        const int scb = ssrc ? kn / 16 : 0;
                        unsigned char* stage = ring + (size_t)slot * GEMV_STAGE_BYTES;
                        mbar_expect_tx(&fb[slot], (uint32_t)(rows * (cpb + scb)));
                        if (gm.contig) {  // whole rows: the group is one contiguous run
                            bulk_g2s_hint(stage, src, (uint32_t)(rows * cpb), &fb[slot], policy);
                            if (scb) bulk_g2s_hint(stage + GEMV_TILE_BYTES, ssrc, (uint32_t)(rows * scb), &fb[slot], policy);
                        } else {
                            const int koff = gemv_row_bytes(sg.fmt, k0);
                            for (int r = 0; r < rows; ++r) {
                                bulk_g2s_hint(stage + r * gm.piece, src + (size_t)r * row_bytes + koff, (uint32_t)cpb,
                                              &fb[slot], policy);
                                if (scb)
                                    bulk_g2s_hint(stage + GEMV_TILE_BYTES + r * scb, ssrc + (size_t)r * srow_bytes + k0 / 16,
                                                  (uint32_t)scb, &fb[slot], policy);
                            }
                        }
                        ++fills;
                        if (++slot == S) {
                            slot = 0;
                            if (fills > (uint32_t)S) ephase ^= 1;
                        }
                    }
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    if (p.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }

    if (p.copy_src && blockIdx.x == 0)
        for (int i = tid; i < p.copy_n / 8; i += NT_CONS)
            reinterpret_cast<uint4*>(p.copy_dst)[i] = reinterpret_cast<const uint4*>(p.copy_src)[i];

    // ---- phase A: input vector, optional layer norm, token-shift difference (8 halves per thread per pass)
    const __half* xin = p.emb ? p.emb + (size_t)p.token[0] * K : p.x;
    float lsum = 0.f;
    for (int i = tid; i < K / 8; i += NT_CONS) {
        const uint4 v = reinterpret_cast<const uint4*>(xin)[i];
        reinterpret_cast<uint4*>(xn)[i] = v;
        if (p.x_copy && blockIdx.x == 0) reinterpret_cast<uint4*>(p.x_copy)[i] = v;
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            lsum += f.x + f.y;
        }
    }
    if (p.ln_w) {
        const float mean = cons_block_sum(lsum, red, tid) / (float)K;
        float q = 0.f;
        for (int i = tid; i < K / 8; i += NT_CONS) {
            const uint4 v = reinterpret_cast<const uint4*>(xn)[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                q += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
            }
        }
        const float rstd = rsqrtf(cons_block_sum(q, red, tid) / (float)K + 1e-5f);
        for (int i = tid; i < K / 8; i += NT_CONS) {
            const uint4 v = reinterpret_cast<const uint4*>(xn)[i];
            const uint4 wv = reinterpret_cast<const uint4*>(p.ln_w)[i];
            const uint4 bv = reinterpret_cast<const uint4*>(p.ln_b)[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
            const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
            uint4 o;
            __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]), wf = __half22float2(w2[e]), bf = __half22float2(b2[e]);
                o2[e] = __floats2half2_rn((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
            }
            reinterpret_cast<uint4*>(xn)[i] = o;
            if (p.ln_out && blockIdx.x == 0) reinterpret_cast<uint4*>(p.ln_out)[i] = o;
        }
    }
    if (p.smem_flags & 4) {
        for (int i = tid; i < K / 8; i += NT_CONS) {  // the same thread wrote xn[i] above: no barrier needed
            const uint4 v = reinterpret_cast<const uint4*>(xn)[i];
            const uint4 pv = reinterpret_cast<const uint4*>(p.x_prev)[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const __half2* q2 = reinterpret_cast<const __half2*>(&pv);
            uint4 o;
            __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) o2[e] = __hsub2(q2[e], h[e]);
            reinterpret_cast<uint4*>(dx)[i] = o;
        }
    }
    cons_sync();

    unsigned char* ring = smem + (size_t)warp * S * GEMV_STAGE_BYTES;
    uint64_t* fb = full_bars + warp * S;
    uint64_t* eb = empty_bars + warp * S;
    int slot = 0;
    uint32_t fphase = 0;
    bool failed = false;

    for (int s = 0; s < p.nseg; ++s) {
        int lo, hi;
        seg_range(p, s, G0, G1, lo, hi);
        if (lo >= hi) continue;  // block-uniform
        const GemvSeg& sg = p.seg[s];
        const int fmt = sg.fmt;

        // ---- phase B: the segment's input in the form its rows consume (16 elements per thread per pass)
        for (int c0 = warp * 32; c0 < Kp / 16; c0 += NT_CONS) {
            const int c = c0 + lane;
            const bool in = c * 16 < K;
            float v[16];
            if (in) {
                const uint4 a0 = reinterpret_cast<const uint4*>(xn)[2 * c], a1 = reinterpret_cast<const uint4*>(xn)[2 * c + 1];
                const __half2* h0 = reinterpret_cast<const __half2*>(&a0);
                const __half2* h1 = reinterpret_cast<const __half2*>(&a1);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f0 = __half22float2(h0[e]), f1 = __half22float2(h1[e]);
                    v[2 * e] = f0.x;
                    v[2 * e + 1] = f0.y;
                    v[8 + 2 * e] = f1.x;
                    v[9 + 2 * e] = f1.y;
                }
                if (sg.mix) {
                    const uint4 d0 = reinterpret_cast<const uint4*>(dx)[2 * c], d1 = reinterpret_cast<const uint4*>(dx)[2 * c + 1];
                    const uint4 m0 = reinterpret_cast<const uint4*>(sg.mix)[2 * c], m1 = reinterpret_cast<const uint4*>(sg.mix)[2 * c + 1];
                    const __half2* dd[2] = {reinterpret_cast<const __half2*>(&d0), reinterpret_cast<const __half2*>(&d1)};
                    const __half2* mm[2] = {reinterpret_cast<const __half2*>(&m0), reinterpret_cast<const __half2*>(&m1)};
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 df = __half22float2(dd[hh][e]), mf = __half22float2(mm[hh][e]);
                            v[8 * hh + 2 * e] = rh(v[8 * hh + 2 * e] + rh(df.x * mf.x));
                            v[8 * hh + 2 * e + 1] = rh(v[8 * hh + 2 * e + 1] + rh(df.y * mf.y));
                        }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.f;
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
                float amax = 0.f;
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
        cons_sync();

        // ---- stream this warp's row groups of the segment
        const GemvGeom gm = gemv_geom(fmt, K);
        const int R = gm.R;
        for (int g = lo + warp; g < hi; g += GEMV_WARPS) {
            float acc[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) acc[r] = 0.f;
            const int rows = min(R, sg.n_rows - g * R);
            for (int kc = 0; kc < gm.nkc; ++kc) {
                const unsigned char* tile = ring + (size_t)slot * GEMV_STAGE_BYTES;
                if (!failed && !mbar_wait_bounded(&fb[slot], fphase)) {
                    failed = true;
                    if (lane == 0) atomicOr(&g_device_status, DEV_WAIT_GEMV);
                }
                const int k0 = kc * gm.kc;
                const int kn = min(gm.kc, K - k0);
                if (fmt == FMT_I8) {
                    if (R <= 2) consume_i8<2>(tile, gm.piece, rows, xh, xl, sx, k0, kn, lane, acc);
                    else consume_i8<8>(tile, gm.piece, rows, xh, xl, sx, k0, kn, lane, acc);
                } else if (fmt == FMT_F16) {
                    if (R <= 2) consume_f16<2>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                    else consume_f16<8>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                } else {
                    if (R <= 2) consume_fp4<2>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                    else consume_fp4<8>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&eb[slot]);
                if (++slot == S) {
                    slot = 0;
                    fphase ^= 1;
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
        }
        cons_sync();  // all warps are done with this segment's x before it is rebuilt
    }
}

}  // namespace

size_t gemv_smem_bytes(const GemvParams& p) {
    const size_t Kp = ((size_t)p.K + 511) & ~(size_t)511;
    size_t off = (size_t)GEMV_WARPS * p.stages * GEMV_STAGE_BYTES + (size_t)GEMV_WARPS * p.stages * 16;
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
        const int R = gemv_rows_per_group(g.fmt, p.K);
        groups += (g.n_rows + R - 1) / R;
    }
    AB_CHECK_ARG(p.emb || p.x, "gemv: no input vector");
    AB_CHECK_ARG(!(p.smem_flags & 4) || p.x_prev, "gemv: token-shift state missing");
    if (p.stages <= 0) p.stages = 1;
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
    while (smem > max_smem && p.stages > 1) {
        --p.stages;
        smem = gemv_smem_bytes(p);
    }
    AB_CHECK_ARG(smem <= max_smem, "gemv: K=%d needs %zu bytes of shared memory", p.K, smem);
    const int grid = max(1, min(n_sm, groups));

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
