// Device-side body of the weight-streaming matrix-vector product, shared by the stand-alone kernel
// (gemv.cu) and the persistent batch-1 decode kernel (decode.cu).
//
//   producer : lane w of the producer warp feeds consumer warp w's private ring of shared-memory
//              stages with 1-D bulk (TMA) copies of >= 4 KB that complete on "full" mbarriers;
//              consumers hand stages back through "empty" mbarriers.
//   consumer : prologue (optional embedding gather, layer norm, token-shift lerp), per-segment input
//              preparation, dp4a / fp16 / NVFP4 tile math, warp-shuffle reduction, fused epilogue.
#pragma once
#include "gemv.cuh"

namespace ab {

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

// Activations written by other SMs earlier in the same kernel must not be served from a stale L1 line.
__device__ __forceinline__ uint4 ld_act16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// ---- shared-memory layout ------------------------------------------------------------------------
struct GemvLayout {
    size_t ring, bars, xn, dx, xq, sx, red, total;
};
// Kn: length of the shared (normalised) input kept in smem, 0 if unused; with_dx: token-shift difference kept;
// Kq: longest per-segment input in the form the rows consume (int8 hi/lo bytes or fp16).
__host__ __device__ inline GemvLayout gemv_layout(int stages, int Kn, int with_dx, int Kq) {
    GemvLayout L;
    const size_t Knp = ((size_t)Kn + 511) & ~(size_t)511, Kqp = ((size_t)Kq + 511) & ~(size_t)511;
    size_t off = 0;
    L.ring = off; off += (size_t)GEMV_WARPS * stages * GEMV_STAGE_BYTES;
    L.bars = off; off += (size_t)GEMV_WARPS * stages * 16;
    off = (off + 127) & ~(size_t)127;
    L.xn = off; off += Knp * 2;
    L.dx = off; off += with_dx ? Knp * 2 : 0;
    L.xq = off; off += Kqp * 2;
    L.sx = off; off += (Kqp / 512) * 4 + 16;
    L.red = off; off += 64 * 4;
    L.total = off;
    return L;
}

struct GemvSmem {
    unsigned char* ring;
    uint64_t *full, *empty;
    __half *xn, *dx;
    unsigned char* xq;
    float *sx, *red;
    int stages;
};
__device__ __forceinline__ GemvSmem gemv_smem(unsigned char* base, const GemvLayout& L, int stages) {
    GemvSmem m;
    m.ring = base + L.ring;
    m.full = reinterpret_cast<uint64_t*>(base + L.bars);
    m.empty = m.full + GEMV_WARPS * stages;
    m.xn = reinterpret_cast<__half*>(base + L.xn);
    m.dx = reinterpret_cast<__half*>(base + L.dx);
    m.xq = base + L.xq;
    m.sx = reinterpret_cast<float*>(base + L.sx);
    m.red = reinterpret_cast<float*>(base + L.red);
    m.stages = stages;
    return m;
}
__device__ __forceinline__ void gemv_init_barriers(const GemvSmem& m) {
    for (int i = 0; i < GEMV_WARPS * m.stages; ++i) {
        mbar_init(&m.full[i], 1);
        mbar_init(&m.empty[i], 1);
    }
    fence_mbar_init();
}

struct ProducerState {
    int slot;
    uint32_t fills;   // tiles issued so far
    uint32_t ephase;  // parity of the empty barrier to wait for once the ring has wrapped
    bool dead;
};
struct ConsumerState {
    int slot;
    uint32_t fphase;
    bool failed;
};

// Work is split between blocks in cost units (gemv_group_cost): block `bid` owns the cost range [C0, C1) of the
// concatenated segments; seg_range converts it to the row-group range [lo, hi) of segment s.
__device__ __forceinline__ void block_range(const GemvParams& p, int bid, int nb, long long& C0, long long& C1) {
    long long total = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const int R = gemv_rows_per_group(p.seg[s].fmt, p.seg[s].K);
        total += (long long)((p.seg[s].n_rows + R - 1) / R) * gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
    }
    C0 = total * bid / nb;
    C1 = total * (bid + 1) / nb;
}
__device__ __forceinline__ void seg_range(const GemvParams& p, int s, long long C0, long long C1, int& lo, int& hi) {
    long long base = 0;
    for (int i = 0; i < s; ++i) {
        const int R = gemv_rows_per_group(p.seg[i].fmt, p.seg[i].K);
        base += (long long)((p.seg[i].n_rows + R - 1) / R) * gemv_group_cost(p.seg[i].fmt, p.seg[i].K);
    }
    const int R = gemv_rows_per_group(p.seg[s].fmt, p.seg[s].K);
    const long long n = (p.seg[s].n_rows + R - 1) / R;
    const long long unit = gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
    long long l = (C0 - base + unit - 1) / unit, h = (C1 - base + unit - 1) / unit;
    if (C0 <= base) l = 0;
    if (C1 <= base) h = 0;
    lo = (int)(l > n ? n : l);
    hi = (int)(h > n ? n : h);
}

// ---- producer ------------------------------------------------------------------------------------
// Called by lanes < GEMV_WARPS of the producer warp (convergent); lane = index of the consumer warp it
// feeds. Each pass of the loop serves, in lockstep, every lane whose next ring slot is free, so one
// instruction stream issues up to GEMV_WARPS tiles; a lane's cursor advances by pointer increments.
__device__ __forceinline__ void gemv_produce(const GemvParams& p, const GemvSmem& m, ProducerState& ps, int lane, int bid,
                                             int nb, uint64_t policy) {
    const int S = m.stages;
    const unsigned mask = (1u << GEMV_WARPS) - 1u;
    unsigned char* ring = m.ring + (size_t)lane * S * GEMV_STAGE_BYTES;
    uint64_t* fb = m.full + lane * S;
    uint64_t* eb = m.empty + lane * S;
    long long C0, C1;
    block_range(p, bid, nb, C0, C1);

    // cursor of this lane
    int s = -1, g = 0, hi = 0, kc = 0;
    int R = 1, piece = 0, nkc = 1, contig = 1, row_bytes = 0, srow_bytes = 0, n_rows = 0, fp4 = 0;
    const unsigned char* src = nullptr;   // first row of group g
    const unsigned char* ssrc = nullptr;  // its block scales (NVFP4)
    auto next_segment = [&]() {
        for (++s; s < p.nseg; ++s) {
            int lo;
            seg_range(p, s, C0, C1, lo, hi);
            g = lo + lane;
            if (g < hi) break;
        }
        if (s < p.nseg) {
            const GemvSeg& sg = p.seg[s];
            const GemvGeom gm = gemv_geom(sg.fmt, sg.K);
            R = gm.R; piece = gm.piece; nkc = gm.nkc; contig = gm.contig;
            row_bytes = gemv_row_bytes(sg.fmt, sg.K);
            srow_bytes = sg.K / 16;
            n_rows = sg.n_rows;
            fp4 = sg.fmt == FMT_FP4;
            src = (const unsigned char*)sg.w + (size_t)g * R * row_bytes;
            ssrc = fp4 ? (const unsigned char*)sg.scale + (size_t)g * R * srow_bytes : nullptr;
            kc = 0;
        }
    };
    next_segment();

    uint32_t idle = 0;
    while (true) {
        const bool has = s < p.nseg && !ps.dead;
        if (__ballot_sync(mask, has) == 0) break;
        const bool ready = has && (ps.fills < (uint32_t)S || mbar_test_wait(&eb[ps.slot], ps.ephase));
        if (__ballot_sync(mask, ready) == 0) {
            __nanosleep(40);
            if (++idle > (1u << 22)) {  // bounded: report and stop instead of spinning for ever
                if (has) {
                    ps.dead = true;
                    atomicOr(&g_device_status, DEV_WAIT_GEMV);
                }
            }
            continue;
        }
        idle = 0;
        if (ready) {
            const int koff = kc * piece;
            const int cpb = min(piece, row_bytes - koff);
            const int rows = min(R, n_rows - g * R);
            const int scb = fp4 ? cpb / 8 : 0;   // one scale byte per 16 inputs = per 8 weight bytes
            unsigned char* stage = ring + (size_t)ps.slot * GEMV_STAGE_BYTES;
            uint64_t* bar = &fb[ps.slot];
            mbar_expect_tx(bar, (uint32_t)(rows * (cpb + scb)));
            if (contig) {  // whole rows: the group is one contiguous run
                bulk_g2s_hint(stage, src, (uint32_t)(rows * cpb), bar, policy);
                if (scb) bulk_g2s_hint(stage + GEMV_TILE_BYTES, ssrc, (uint32_t)(rows * scb), bar, policy);
            } else {
                for (int r = 0; r < rows; ++r) {
                    bulk_g2s_hint(stage + r * piece, src + (size_t)r * row_bytes + koff, (uint32_t)cpb, bar, policy);
                    if (scb)
                        bulk_g2s_hint(stage + GEMV_TILE_BYTES + r * scb, ssrc + (size_t)r * srow_bytes + koff / 8,
                                      (uint32_t)scb, bar, policy);
                }
            }
            ++ps.fills;
            if (++ps.slot == S) {
                ps.slot = 0;
                if (ps.fills > (uint32_t)S) ps.ephase ^= 1;
            }
            if (++kc == nkc) {
                kc = 0;
                g += GEMV_WARPS;
                src += (size_t)GEMV_WARPS * R * row_bytes;
                if (fp4) ssrc += (size_t)GEMV_WARPS * R * srow_bytes;
                if (g >= hi) next_segment();
            }
        }
    }
}

// ---- per-format tile math: acc[r] += sum over this lane's slice of the tile ----------------------
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

// One whole int8 row piece of 4096 inputs: all loads of half a tile are issued before the math, and the
// sixteen dp4a chains of a half are independent.
__device__ __forceinline__ void consume_i8_4096(const unsigned char* tile, const signed char* xh, const unsigned char* xl,
                                                const float* sx, int k0, int lane, float& acc) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint4 w[4], a[4], b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = (half * 4 + j) * 512 + lane * 16;
            w[j] = *reinterpret_cast<const uint4*>(tile + k);
            a[j] = *reinterpret_cast<const uint4*>(xh + k0 + k);
            b[j] = *reinterpret_cast<const uint4*>(xl + k0 + k);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int ah = dp4a_ss(w[j].x, a[j].x, 0);
            int al = dp4a_su(w[j].x, b[j].x, 0);
            ah = dp4a_ss(w[j].y, a[j].y, ah);
            al = dp4a_su(w[j].y, b[j].y, al);
            ah = dp4a_ss(w[j].z, a[j].z, ah);
            al = dp4a_su(w[j].z, b[j].z, al);
            ah = dp4a_ss(w[j].w, a[j].w, ah);
            al = dp4a_su(w[j].w, b[j].w, al);
            acc = fmaf((float)(ah * 256 + al), sx[(k0 >> 9) + half * 4 + j], acc);
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

// ---- consumer ------------------------------------------------------------------------------------
// Called by all consumer threads (tid < NT_CONS) of a block.
__device__ __forceinline__ void gemv_consume(const GemvParams& p, const GemvSmem& m, ConsumerState& cs, int tid, int bid,
                                             int nb) {
    const int warp = tid >> 5, lane = tid & 31;
    const int S = m.stages;
    __half* xn = m.xn;
    __half* dx = m.dx;

    if (p.copy_src && bid == 0)
        for (int i = tid; i < p.copy_n / 8; i += NT_CONS)
            reinterpret_cast<uint4*>(p.copy_dst)[i] = ld_act16(reinterpret_cast<const uint4*>(p.copy_src) + i);

    // ---- phase A: shared input vector, optional layer norm, token-shift difference
    const bool shared_in = p.emb || p.x;
    bool any_mix = false;
    for (int s = 0; s < p.nseg; ++s) any_mix |= p.seg[s].mix != nullptr;
    if (shared_in) {
        const int K = p.K;
        const __half* xin = p.emb ? p.emb + (size_t)__ldcg(p.token) * K : p.x;
        float lsum = 0.f;
        for (int i = tid; i < K / 8; i += NT_CONS) {
            const uint4 v = ld_act16(reinterpret_cast<const uint4*>(xin) + i);
            reinterpret_cast<uint4*>(xn)[i] = v;
            if (p.x_copy && bid == 0) reinterpret_cast<uint4*>(p.x_copy)[i] = v;
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                lsum += f.x + f.y;
            }
        }
        if (p.ln_w) {
            const float mean = cons_block_sum(lsum, m.red, tid) / (float)K;
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
            const float rstd = rsqrtf(cons_block_sum(q, m.red, tid) / (float)K + 1e-5f);
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
                if (p.ln_out && bid == 0) reinterpret_cast<uint4*>(p.ln_out)[i] = o;
            }
        }
        if (any_mix) {
            for (int i = tid; i < K / 8; i += NT_CONS) {  // the same thread wrote xn[i] above: no barrier needed
                const uint4 v = reinterpret_cast<const uint4*>(xn)[i];
                const uint4 pv = ld_act16(reinterpret_cast<const uint4*>(p.x_prev) + i);
                const __half2* h = reinterpret_cast<const __half2*>(&v);
                const __half2* q2 = reinterpret_cast<const __half2*>(&pv);
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) o2[e] = __hsub2(q2[e], h[e]);
                reinterpret_cast<uint4*>(dx)[i] = o;
            }
        }
    }
    cons_sync();

    unsigned char* ring = m.ring + (size_t)warp * S * GEMV_STAGE_BYTES;
    uint64_t* fb = m.full + warp * S;
    uint64_t* eb = m.empty + warp * S;
    long long G0, G1;
    block_range(p, bid, nb, G0, G1);

    for (int s = 0; s < p.nseg; ++s) {
        int lo, hi;
        seg_range(p, s, G0, G1, lo, hi);
        if (lo >= hi) continue;  // block-uniform
        const GemvSeg& sg = p.seg[s];
        const int fmt = sg.fmt;
        const int K = sg.K;
        const int Kp = (K + 511) & ~511;
        signed char* xh = reinterpret_cast<signed char*>(m.xq);
        unsigned char* xl = m.xq + Kp;
        __half* xf = reinterpret_cast<__half*>(m.xq);

        // ---- phase B: the segment's input in the form its rows consume (16 elements per thread per pass)
        for (int c0 = warp * 32; c0 < Kp / 16; c0 += NT_CONS) {
            const int c = c0 + lane;
            const bool in = c * 16 < K;
            float v[16];
            if (in) {
                uint4 a0, a1;
                if (sg.x) {
                    a0 = ld_act16(reinterpret_cast<const uint4*>(sg.x) + 2 * c);
                    a1 = ld_act16(reinterpret_cast<const uint4*>(sg.x) + 2 * c + 1);
                } else {
                    a0 = reinterpret_cast<const uint4*>(xn)[2 * c];
                    a1 = reinterpret_cast<const uint4*>(xn)[2 * c + 1];
                }
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
                if (lane == 0) m.sx[c0 / 32] = amax / 32767.0f;
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
                const unsigned char* tile = ring + (size_t)cs.slot * GEMV_STAGE_BYTES;
                if (!cs.failed && !mbar_wait_bounded(&fb[cs.slot], cs.fphase)) {
                    cs.failed = true;
                    if (lane == 0) atomicOr(&g_device_status, DEV_WAIT_GEMV);
                }
                const int k0 = kc * gm.kc;
                const int kn = min(gm.kc, K - k0);
                if (fmt == FMT_I8) {
                    if (R == 1 && kn == 4096) consume_i8_4096(tile, xh, xl, m.sx, k0, lane, acc[0]);
                    else if (R <= 2) consume_i8<2>(tile, gm.piece, rows, xh, xl, m.sx, k0, kn, lane, acc);
                    else consume_i8<8>(tile, gm.piece, rows, xh, xl, m.sx, k0, kn, lane, acc);
                } else if (fmt == FMT_F16) {
                    if (R <= 2) consume_f16<2>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                    else consume_f16<8>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                } else {
                    if (R <= 2) consume_fp4<2>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                    else consume_fp4<8>(tile, gm.piece, rows, xf, k0, kn, lane, acc);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&eb[cs.slot]);
                if (++cs.slot == S) {
                    cs.slot = 0;
                    cs.fphase ^= 1;
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
                    case EPI_RESID: o = __half2float(__ldcg(sg.resid + row)) + o; break;
                    default: break;
                }
                sg.out[row] = __float2half_rn(o);
            }
        }
        cons_sync();  // all warps are done with this segment's x before it is rebuilt
    }
}

}  // namespace ab
