// Device-side body of the fused per-head time-mix step, shared by the stand-alone kernel (head.cu)
// and the persistent batch-1 decode kernel (decode.cu). See head.cu for the math and its citations.
#pragma once
#include "head.cuh"

namespace ab {

constexpr int HT = 256;  // threads working on one (sequence, head)

struct HeadShared {
    float r[64], w[64], k[64], a[64], b[64], v[64], y[64];
    float up[4][64];  // adapter up-projection sums (w, a, v-gate, g) of the batch-1 stand-alone path
};
struct SyncBlock {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};
struct SyncNamed256 {  // the first 256 threads of a larger block
    __device__ __forceinline__ void operator()() const { asm volatile("bar.sync 2, 256;" ::: "memory"); }
};
// activations may have been written by another SM earlier in the same kernel: bypass L1
__device__ __forceinline__ float lda(const __half* p) { return __half2float(__ldcg(p)); }

// Dataflow mode of the persistent kernel: the vectors that cross blocks (r, k, v, the adapter hidden vectors in; the
// head output out) are arrays of tagged 32-bit words (fp16 value | phase tag << 16, see gemv_body.cuh); a reader spins
// on the word itself until it carries the expected tag. `on == false`: plain fp16 arrays.
struct HeadTags {
    bool on;
    uint32_t in, out;
};
__device__ __forceinline__ float head_ld(const __half* base, size_t idx, const HeadTags& tg) {
    if (!tg.on) return lda(base + idx);
    const uint32_t* p = reinterpret_cast<const uint32_t*>(base) + idx;
    uint32_t w, it = 0;
    while (true) {
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
        if ((w >> 16) == tg.in) break;
        if (++it > (1u << 21)) {
            atomicOr(&g_device_status, DEV_WAIT_HEAD);
            break;
        }
        __nanosleep(TAG_POLL_NS);
    }
    return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
}
// r, k, v of this lane's two channels (c = lane, lane + 32) in one go: six loads in flight, validated together (one
// after the other, each with its own wait, they cost six memory round trips on the head's critical path).
__device__ __forceinline__ void head_ld_rkv(const HeadParams& p, size_t off, int lane, const HeadTags& tg, float* rr, float* kr,
                                            float* vv) {
    if (!tg.on) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            rr[e] = lda(p.r + off + lane + 32 * e);
            kr[e] = lda(p.k + off + lane + 32 * e);
            vv[e] = lda(p.v + off + lane + 32 * e);
        }
        return;
    }
    const uint32_t* pr = reinterpret_cast<const uint32_t*>(p.r) + off + lane;
    const uint32_t* pk = reinterpret_cast<const uint32_t*>(p.k) + off + lane;
    const uint32_t* pv = reinterpret_cast<const uint32_t*>(p.v) + off + lane;
    uint32_t w0, w1, w2, w3, w4, w5, it = 0;
    while (true) {
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w0) : "l"(pr) : "memory");
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w1) : "l"(pr + 32) : "memory");
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w2) : "l"(pk) : "memory");
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w3) : "l"(pk + 32) : "memory");
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w4) : "l"(pv) : "memory");
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w5) : "l"(pv + 32) : "memory");
        const uint32_t bad = ((w0 >> 16) ^ tg.in) | ((w1 >> 16) ^ tg.in) | ((w2 >> 16) ^ tg.in) | ((w3 >> 16) ^ tg.in) |
                             ((w4 >> 16) ^ tg.in) | ((w5 >> 16) ^ tg.in);
        if (!bad) break;
        if (++it > (1u << 21)) {
            atomicOr(&g_device_status, DEV_WAIT_HEAD);
            break;
        }
        __nanosleep(TAG_POLL_NS);
    }
    auto val = [](uint32_t x) { return __half2float(__ushort_as_half((unsigned short)(x & 0xffffu))); };
    rr[0] = val(w0); rr[1] = val(w1); kr[0] = val(w2); kr[1] = val(w3); vv[0] = val(w4); vv[1] = val(w5);
}
__device__ __forceinline__ void head_st(__half* base, size_t idx, float v, const HeadTags& tg) {
    if (!tg.on) {
        base[idx] = __float2half_rn(v);
        return;
    }
    const uint32_t w = (uint32_t)__half_as_ushort(__float2half_rn(v)) | (tg.out << 16);
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(base) + idx), "r"(w) : "memory");
}

struct StateRow {
    float s[16];
};

__device__ __forceinline__ void load_state(StateRow& st, const float* base, int i, int q) {
    if (!AB_BC(i >= 0 && i < 64 && q >= 0 && q < 4)) return;
    const float4* src = reinterpret_cast<const float4*>(base + i * 64 + q * 16);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float4 f = src[e];
        st.s[4 * e] = f.x; st.s[4 * e + 1] = f.y; st.s[4 * e + 2] = f.z; st.s[4 * e + 3] = f.w;
    }
}
__device__ __forceinline__ void store_state(const StateRow& st, float* base, int i, int q) {
    if (!AB_BC(i >= 0 && i < 64 && q >= 0 && q < 4)) return;
    float4* dst = reinterpret_cast<float4*>(base + i * 64 + q * 16);
#pragma unroll
    for (int e = 0; e < 4; ++e) dst[e] = make_float4(st.s[4 * e], st.s[4 * e + 1], st.s[4 * e + 2], st.s[4 * e + 3]);
}

__device__ __forceinline__ void head_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void head_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
// Bytes of scratch shared memory the in-kernel adapter up-projections of one head need.
__host__ __device__ inline size_t head_ups_smem(int rtot) {
    return (size_t)rtot * 128 + (size_t)((rtot + 3) & ~3) * 4 + 8 * 4 * 64 * 4;
}

// Batch-1 adapter up-projections of head h, part 1: start copying this head's 64-channel slices of the four
// up-projection matrices ([rank, D] each) into scratch shared memory. They are weights: no dependency on activations.
__device__ __forceinline__ void head_ups_stage(const HeadParams& p, int h, int tid, unsigned char* dsm) {
    __half* w2s = reinterpret_cast<__half*>(dsm);   // [rtot][64], swizzled
    const int rtot = p.rw + p.ra + p.rv + p.rg;
    for (int pc = tid; pc < rtot * 8; pc += HT) {
        int row = pc >> 3;
        const int seg8 = pc & 7;
        const __half* m;
        if (row < p.rw) m = p.w2;
        else if ((row -= p.rw) < p.ra) m = p.a2;
        else if ((row -= p.ra) < p.rv) m = p.v2;
        else { row -= p.rv; m = p.g2; }
        // 16-byte pieces of a row are stored at piece ^ (row & 7): the 8x8 tiles the tensor-core loads read (eight
        // consecutive rows, the same piece) then touch eight different bank groups
        head_cp_async16(w2s + (size_t)(pc >> 3) * 64 + (seg8 ^ ((pc >> 3) & 7)) * 8, m + (size_t)row * p.D + h * 64 + seg8 * 8);
    }
}
// The head's eight per-channel parameter vectors (64 fp16 each) behind the staged up-projection slices: [8][64] fp16.
__device__ __forceinline__ __half* head_par_area(const HeadParams& p, unsigned char* dsm) {
    return reinterpret_cast<__half*>(dsm + head_ups_smem(p.rw + p.ra + p.rv + p.rg));
}
__device__ __forceinline__ void head_par_stage(const HeadParams& p, int h, int tid, unsigned char* dsm) {
    if (tid < 64) {
        const int which = tid >> 3, chunk = tid & 7;
        const __half* v[8] = {p.w0, p.a0, p.v0, p.k_k, p.k_a, p.r_k, p.lnx_w, p.lnx_b};
        const __half* src = v[0];
#pragma unroll
        for (int e = 1; e < 8; ++e)
            if (which == e) src = v[e];
        if (src) head_cp_async16(head_par_area(p, dsm) + which * 64 + chunk * 8, src + h * 64 + chunk * 8);
    }
}
// Part 2: sh.up[m][c] = sum_j hidden_m[j] * W2_m[j, h*64 + c] for the four adapters m (w, a, v-gate, g).
template <class Sync>
__device__ __forceinline__ void head_ups_compute(const HeadParams& p, int tid, unsigned char* dsm, HeadShared& sh, Sync sync,
                                                 const HeadTags tg = HeadTags{false, 0u, 0u}, unsigned long long* tl = nullptr) {
    const int rtot = p.rw + p.ra + p.rv + p.rg;
    const int lane = tid & 31, warp = tid >> 5;
    const __half* w2s = reinterpret_cast<const __half*>(dsm);
    unsigned short* hv16 = reinterpret_cast<unsigned short*>(dsm + (size_t)rtot * 128);   // [rtot] fp16 bits
    float* part = reinterpret_cast<float*>(hv16) + ((rtot + 3) & ~3);                    // [8][4][64]
    // all of this thread's entries are requested before the first one is looked at (each is a tagged word that may
    // have to be waited for: one after the other they would cost a memory round trip each)
    constexpr int HV_MAX = 4;   // entries per thread: adapter ranks up to 4 * 256 in total (longer lists loop)
    auto addr = [&](int j) -> const __half* {   // entry j of the concatenated hidden vectors (a word each when tagged)
        int row = j;
        const __half* hv;
        if (row < p.rw) hv = p.hw;
        else if ((row -= p.rw) < p.ra) hv = p.ha;
        else if ((row -= p.ra) < p.rv) hv = p.hv;
        else { row -= p.rv; hv = p.hg; }
        return tg.on ? hv + 2 * (size_t)row : hv + row;
    };
    for (int j0 = tid; j0 < rtot; j0 += HV_MAX * HT) {
        if (!tg.on) {
#pragma unroll
            for (int e = 0; e < HV_MAX; ++e)
                if (j0 + e * HT < rtot) hv16[j0 + e * HT] = __half_as_ushort(__ldcg(addr(j0 + e * HT)));
            continue;
        }
        uint32_t w[HV_MAX], it = 0;
        while (true) {
            uint32_t bad = 0;
#pragma unroll
            for (int e = 0; e < HV_MAX; ++e)
                if (j0 + e * HT < rtot) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w[e]) : "l"(addr(j0 + e * HT)) : "memory");
#pragma unroll
            for (int e = 0; e < HV_MAX; ++e)
                if (j0 + e * HT < rtot) bad |= (w[e] >> 16) ^ tg.in;
            if (!bad) break;
            if (++it > (1u << 21)) {
                atomicOr(&g_device_status, DEV_WAIT_HEAD);
                break;
            }
            __nanosleep(TAG_POLL_NS);
        }
#pragma unroll
        for (int e = 0; e < HV_MAX; ++e)
            if (j0 + e * HT < rtot) hv16[j0 + e * HT] = (unsigned short)(w[e] & 0xffffu);
    }
    if (tl) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tl[0]));   // this thread's hidden-vector entries are in
    head_cp_async_wait_all();
    sync();
    if (tl) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tl[1]));   // everybody's are, and the staged weights
    // On the tensor cores (mma.sync m16n8k16, fp16 in, fp32 accumulate): with scalar code the 53 k fp16 -> fp32
    // conversions of the weights alone take longer than everything else in the head. Weights and hidden values are fp16 in
    // memory, so nothing is rounded on the way in. A tile is 16 rows x 64 channels: four instructions with the weights
    // as the 16 (channels) x 16 (rows) operand and the hidden values in column 0 of the 16 x 8 one. Warp w takes the
    // tiles w, w + 8, ... of the concatenated tile list of the four matrices.
    const int bounds[5] = {0, p.rw, p.rw + p.ra, p.rw + p.ra + p.rv, rtot};
    // lane's row address for the four 8x8 tiles of a 16 x 16 weight operand: tile (lane >> 3): bit 0 = channels 8-15,
    // bit 1 = rows 8-15; row (lane & 7) of that tile
    const int lrow = (lane & 7) + ((lane >> 4) << 3), lpiece = (lane >> 3) & 1;
    const uint32_t w2s_u32 = (uint32_t)__cvta_generic_to_shared(w2s);
    int tbase = 0;   // index of the matrix' first tile in the concatenated tile list
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        float acc[4][4];
#pragma unroll
        for (int ct = 0; ct < 4; ++ct) acc[ct][0] = acc[ct][1] = acc[ct][2] = acc[ct][3] = 0.f;
        const int rows = bounds[m + 1] - bounds[m], nt = (rows + 15) >> 4;
        for (int kt = (warp - tbase) & 7; kt < nt; kt += 8) {
            // hidden values: column 0 of the 16 x 8 operand lives in lanes 0-3 (rows 2*lane, 2*lane+1 and those + 8);
            // rows past the end of the matrix are zeros
            uint32_t b0 = 0, b1 = 0;
            if (lane < 4) {
                const int r = kt * 16 + 2 * lane;
                const unsigned short* hp = hv16 + bounds[m] + r;
                b0 = (r < rows ? hp[0] : 0u) | ((r + 1 < rows ? hp[1] : 0u) << 16);
                b1 = (r + 8 < rows ? hp[8] : 0u) | ((r + 9 < rows ? hp[9] : 0u) << 16);
            }
            // the address of a row past the end is clamped to the last row: only weights are multiplied by those zeros
            int krow = bounds[m] + min(kt * 16 + lrow, rows - 1);
            if (!AB_BC(krow >= 0 && krow < rtot)) krow = 0;
#pragma unroll
            for (int ct = 0; ct < 4; ++ct) {
                uint32_t a0, a1, a2, a3;
                const uint32_t a_addr = w2s_u32 + (uint32_t)(krow * 128 + (((2 * ct + lpiece) ^ (krow & 7)) << 4));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(a_addr));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                             : "+f"(acc[ct][0]), "+f"(acc[ct][1]), "+f"(acc[ct][2]), "+f"(acc[ct][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
            }
        }
        // column 0 of the result: lanes 0, 4, .. 28 hold channels lane / 4 and lane / 4 + 8 of each 16-channel tile
        if ((lane & 3) == 0) {
#pragma unroll
            for (int ct = 0; ct < 4; ++ct) {
                if (AB_BC((warp * 4 + m) * 64 + ct * 16 + (lane >> 2) + 8 < 8 * 4 * 64)) {
                    part[(warp * 4 + m) * 64 + ct * 16 + (lane >> 2)] = acc[ct][0];
                    part[(warp * 4 + m) * 64 + ct * 16 + (lane >> 2) + 8] = acc[ct][2];
                }
            }
        }
        tbase += nt;
    }
    sync();
    {
        const int m = tid >> 6, c = tid & 63;
        float s = 0.f;
#pragma unroll
        for (int wq = 0; wq < 8; ++wq) s += part[(wq * 4 + m) * 64 + c];
        sh.up[m][c] = rh(s);
    }
    sync();
}

// One recurrence step for this thread's 16 columns. Vectors are indexed by key column j.
// Returns y_i (valid in all four lanes of the row).
__device__ __forceinline__ float wkv_step(StateRow& st, const float* w, const float* k, const float* a,
                                          const float* b, const float* r, float v_i, int q) {
    float sa = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) sa = fmaf(a[q * 16 + e], st.s[e], sa);
    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    float y = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int j = q * 16 + e;
        float s = st.s[e];
        s = fmaf(s, w[j], fmaf(k[j], v_i, sa * b[j]));
        st.s[e] = s;
        y = fmaf(s, r[j], y);
    }
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    return y;
}


// All T steps of one (sequence b, head h) for the 256 threads tid = 0..255.
// `par`: the head's per-channel parameters staged in shared memory as [8][64] fp16 in the order w0, a0, v0, k_k, k_a, r_k,
// ln_x weight, ln_x bias (null: read them from global memory).
__device__ __forceinline__ float head_par(const __half* par, int which, const __half* global_vec, int gc, int c) {
    return __half2float(par ? par[which * 64 + c] : global_vec[gc]);
}
template <class Sync>
__device__ __forceinline__ void head_steps(const HeadParams& p, int b, int h, int tid, StateRow& st, HeadShared& sh,
                                           bool ups, Sync sync, const HeadTags tg = HeadTags{false, 0u, 0u},
                                           const __half* par = nullptr) {
    const int i = tid >> 2, q = tid & 3, lane = tid & 31, warp = tid >> 5;
    const int D = p.D;
    float* sr = sh.r; float* sw = sh.w; float* sk = sh.k; float* sa_ = sh.a; float* sb = sh.b; float* sv = sh.v; float* sy = sh.y;
    float (*up)[64] = sh.up;
    for (int t = 0; t < p.T; ++t) {
        const size_t off = ((size_t)b * p.T + t) * D + h * 64;
        if (warp == 0) {
            // per-channel glue on two channels per lane; head-wide sums are warp shuffles
            float kk0[2], av[2], rk[2];
            float ssq = 0.f, rkr = 0.f;
            // what needs only the adapter outputs and the parameters comes first: in the persistent kernel r, k, v are
            // the last inputs to arrive, and everything below the wait for them is on the token's critical path
            float kfac[2], wd2[2], vg2[2], vf2[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e, gc = h * 64 + c;
                const float w_raw = ups ? up[0][c] : lda(p.w_raw + off + c);
                const float a_raw = ups ? up[1][c] : lda(p.a_raw + off + c);
                av[e] = rh(sigmoidf_(rh(head_par(par, 1, p.a0, gc, c) + a_raw)));
                kfac[e] = rh(1.f + rh(rh(av[e] - 1.f) * head_par(par, 4, p.k_a, gc, c)));
                vg2[e] = vf2[e] = 0.f;
                if (!p.layer0) {
                    const float vg_raw = ups ? up[2][c] : lda(p.vg_raw + off + c);
                    vg2[e] = rh(sigmoidf_(rh(head_par(par, 2, p.v0, gc, c) + vg_raw)));
                    vf2[e] = lda(p.v_first + off + c);
                }
                // decay in fp32 as on the reference's single-token path (reference/rwkv7.py:241)
                wd2[e] = __expf(-0.606531f * sigmoidf_(rh(head_par(par, 0, p.w0, gc, c) + w_raw)));
            }
            float rr2[2], kr2[2], vv2[2];
            head_ld_rkv(p, off, lane, tg, rr2, kr2, vv2);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e, gc = h * 64 + c;
                const float rr = rr2[e];
                const float kr = kr2[e];
                float vv = vv2[e];
                kk0[e] = rh(kr * head_par(par, 3, p.k_k, gc, c));
                ssq = fmaf(kk0[e], kk0[e], ssq);
                const float k2 = rh(kr * kfac[e]);
                if (p.layer0) p.v_first[off + c] = __float2half_rn(vv);
                else vv = rh(vv + rh(rh(vf2[e] - vv) * vg2[e]));
                sr[c] = rr; sw[c] = wd2[e]; sk[c] = k2; sv[c] = vv;
                rk[e] = rh(rh(rr * k2) * head_par(par, 5, p.r_k, gc, c));
                rkr += rk[e];
            }
            ssq = warp_sum(ssq);
            rkr = rh(warp_sum(rkr));
            const float nrm = fmaxf(rh(sqrtf(ssq)), 1e-12f);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e;
                const float kk = rh(kk0[e] / nrm);
                sa_[c] = -kk;
                sb[c] = rh(kk * av[e]);
            }
            sync();
            const float y = wkv_step(st, sw, sk, sa_, sb, sr, sv[i], q);
            if (q == 0) sy[i] = rh(y);
            sync();
            // group norm over the head's 64 channels (eps 64e-5), bonus, gate
            const float y0 = sy[lane], y1 = sy[lane + 32];
            const float mean = warp_sum(y0 + y1) * (1.f / 64.f);
            const float d0 = y0 - mean, d1 = y1 - mean;
            const float var = warp_sum(d0 * d0 + d1 * d1) * (1.f / 64.f);
            const float rstd = rsqrtf(var + 64e-5f);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e, gc = h * 64 + c;
                float o = rh((e ? d1 : d0) * rstd * head_par(par, 6, p.lnx_w, gc, c) + head_par(par, 7, p.lnx_b, gc, c));
                o = rh(o + rh(rkr * sv[c]));
                const float g = ups ? up[3][c] : lda(p.g + off + c);
                head_st(p.out, off + c, o * g, tg);
            }
        } else {
            sync();
            const float y = wkv_step(st, sw, sk, sa_, sb, sr, sv[i], q);
            if (q == 0) sy[i] = rh(y);
            sync();
        }
    }
}

}  // namespace ab
