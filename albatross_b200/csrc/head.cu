// WKV-7 state update for sm_100a, alone (operator ABI of the reference) and fused with its glue.
//
//  * wkv7_kernel      : same contract as the reference operator
//                       torch.ops.rwkv7_state_fwd_fp16.forward (reference/cuda/rwkv7_state_fwd_fp16.cpp:8-14,
//                       kernel reference/cuda/rwkv7_state_fwd_fp16.cu:7-56).
//  * head_fused_kernel: everything between the r/k/v projections and the output projection of one
//                       time-mix block (reference/rwkv7.py:231, 234-249 and the batch twins :284-299):
//                       adapter up-projections (batch 1), k normalisation and modulation, v residual
//                       gate, decay, state update + read-out, per-head group norm, bonus term, gate.
//
// One block of 256 threads per (sequence, head). Thread (i = tid/4, q = tid%4) keeps columns
// [16q, 16q+16) of state row i in registers for all T steps, so a warp's state traffic is one
// contiguous 2 KiB run (8 rows x 256 B) in each direction and row sums need two shuffles.
#include "head_body.cuh"

namespace ab {

namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// Operator-ABI kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(HT) wkv7_kernel(int T, int C, int H, float* __restrict__ state,
                                                  const __half* __restrict__ r_, const __half* __restrict__ w_,
                                                  const __half* __restrict__ k_, const __half* __restrict__ v_,
                                                  const __half* __restrict__ a_, const __half* __restrict__ b_,
                                                  __half* __restrict__ y_) {
    __shared__ float sr[2][64], sw[2][64], sk[2][64], sa_[2][64], sb[2][64], sv[2][64];
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, i = tid >> 2, q = tid & 3;
    float* sbase = state + (size_t)bh * 4096;
    StateRow st;
    load_state(st, sbase, i, q);
    for (int t = 0; t < T; ++t) {
        const int buf = t & 1;
        const size_t off = ((size_t)b * T + t) * C + h * 64;
        if (tid < 64) {
            sr[buf][tid] = __half2float(r_[off + tid]);
            sw[buf][tid] = __expf(-__expf(__half2float(w_[off + tid])));
            sk[buf][tid] = __half2float(k_[off + tid]);
        } else if (tid < 128) {
            const int c = tid - 64;
            sa_[buf][c] = __half2float(a_[off + c]);
            sb[buf][c] = __half2float(b_[off + c]);
            sv[buf][c] = __half2float(v_[off + c]);
        }
        __syncthreads();  // double-buffered vectors: one barrier per step
        const float y = wkv_step(st, sw[buf], sk[buf], sa_[buf], sb[buf], sr[buf], sv[buf][i], q);
        if (q == 0) y_[off + i] = __float2half_rn(y);
    }
    store_state(st, sbase, i, q);
}

// ---------------------------------------------------------------------------------------------
// Fused kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(HT) head_fused_kernel(const __grid_constant__ HeadParams p) {
    extern __shared__ __align__(16) unsigned char dsm[];
    __shared__ HeadShared sh;
    float (*up)[64] = sh.up;
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, i = tid >> 2, q = tid & 3, lane = tid & 31, warp = tid >> 5;
    const int D = p.D;
    const bool ups = p.w2 != nullptr;
    const int rtot = p.rw + p.ra + p.rv + p.rg;

    // ---- batch-1 path: pull this head's slices of the four up-projection matrices into smem.
    // They are weights, so this runs before the wait on the previous kernel.
    __half* w2s = reinterpret_cast<__half*>(dsm);             // [rtot][64]
    float* hvec = reinterpret_cast<float*>(dsm + (size_t)rtot * 128);  // [rtot]
    float* part = hvec + ((rtot + 3) & ~3);                   // [8][4][64]
    if (ups) {
        for (int pc = tid; pc < rtot * 8; pc += HT) {
            int row = pc >> 3;
            const int seg8 = pc & 7;
            const __half* m;
            if (row < p.rw) m = p.w2;
            else if ((row -= p.rw) < p.ra) m = p.a2;
            else if ((row -= p.ra) < p.rv) m = p.v2;
            else { row -= p.rv; m = p.g2; }
            cp_async16(w2s + (size_t)(pc >> 3) * 64 + seg8 * 8, m + (size_t)row * D + h * 64 + seg8 * 8);
        }
    }
    if (p.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }

    float* sbase = p.state + (size_t)bh * 4096;
    StateRow st;
    load_state(st, sbase, i, q);

    if (ups) {
        for (int j = tid; j < rtot; j += HT) {
            int row = j;
            const __half* hv;
            if (row < p.rw) hv = p.hw;
            else if ((row -= p.rw) < p.ra) hv = p.ha;
            else if ((row -= p.ra) < p.rv) hv = p.hv;
            else { row -= p.rv; hv = p.hg; }
            hvec[j] = __half2float(hv[row]);
        }
        cp_async_wait_all();
        __syncthreads();
        // warp `warp` takes rows j = warp (mod 8); lane covers channels 2*lane, 2*lane+1
        const int bounds[5] = {0, p.rw, p.rw + p.ra, p.rw + p.ra + p.rv, rtot};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            float s0 = 0.f, s1 = 0.f;
            for (int j = bounds[m] + warp; j < bounds[m + 1]; j += 8) {
                const float2 wv = __half22float2(reinterpret_cast<const __half2*>(w2s + (size_t)j * 64)[lane]);
                s0 = fmaf(hvec[j], wv.x, s0);
                s1 = fmaf(hvec[j], wv.y, s1);
            }
            part[(warp * 4 + m) * 64 + 2 * lane] = s0;
            part[(warp * 4 + m) * 64 + 2 * lane + 1] = s1;
        }
        __syncthreads();
        {
            const int m = tid >> 6, c = tid & 63;
            float s = 0.f;
#pragma unroll
            for (int wq = 0; wq < 8; ++wq) s += part[(wq * 4 + m) * 64 + c];
            up[m][c] = rh(s);
        }
        if (p.copy_src && tid < 32)
            reinterpret_cast<__half2*>(p.copy_dst + h * 64)[tid] = reinterpret_cast<const __half2*>(p.copy_src + h * 64)[tid];
        __syncthreads();
    }

    head_steps(p, b, h, tid, st, sh, ups, SyncBlock());
    store_state(st, sbase, i, q);
}


// ---------------------------------------------------------------------------------------------
// Batched single-step kernel (T = 1, many sequences): persistent blocks walk a list of (sequence, head) items.
// ---------------------------------------------------------------------------------------------
// The state (16 KiB per item, read once and written once per token) is all of the traffic, so the kernel is built
// around keeping it moving:
//   * warps 0-7 (256 threads) run the recurrence. The item's state arrives as ONE 16 KiB bulk copy into a ring of
//     HB_STAGES shared-memory stages (mbarrier, byte-counted), up to HB_STAGES-1 items ahead of the one being worked on;
//     the updated state goes straight from registers to global memory.
//   * warp 8 does the per-channel glue (k normalisation and modulation, v residual gate, decay) of item n+1 while
//     warps 0-7 are on item n, and the group norm / bonus / gate of item n afterwards; its lane 0 issues the bulk copies.
// Thread (i = tid/4, q = tid%4) owns, of state row i, the four 16-byte chunks {4m + q, m = 0..3} and visits them in
// the order m = (e + i) % 4: a quarter-warp then reads eight different bank groups of the stage (no conflicts).
constexpr int HB_STAGES = 4;
constexpr int HB_THREADS = HT + 32;
constexpr int HB_STATE_BYTES = 64 * 64 * 4;

struct HeadVec {
    float r[64], w[64], k[64], a[64], b[64], v[64];
    float rkr;
    float pad[3];
};

__device__ __forceinline__ void bar_sync_id(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive_id(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void st_cs16(float* p, float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__global__ void __launch_bounds__(HB_THREADS) head_batch_kernel(const __grid_constant__ HeadParams p, int n_items) {
    extern __shared__ __align__(128) unsigned char dsm[];   // HB_STAGES x 16 KiB
    __shared__ __align__(16) HeadVec vec[2];
    __shared__ float sy[2][64];
    __shared__ uint64_t full[HB_STAGES];
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_mine = ((int)blockIdx.x < n_items) ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    auto item_of = [&](int n) { return (int)blockIdx.x + n * (int)gridDim.x; };
    if (tid == 0) {
        for (int s = 0; s < HB_STAGES; ++s) mbar_init(&full[s], 1);
        fence_mbar_init();
        s_failed = 0;
    }
    __syncthreads();
    // named barriers: 1, 2 = vectors of an even / odd item are ready; 3, 4 = its read-out is ready
    if (warp == 8) {
        auto load_state_of = [&](int n) {
            const int s = n % HB_STAGES;
            mbar_expect_tx(&full[s], HB_STATE_BYTES);
            bulk_g2s(dsm + s * HB_STATE_BYTES, p.state + (size_t)item_of(n) * 4096, HB_STATE_BYTES, &full[s]);
        };
        // the state was last written by this kernel one token ago: it does not depend on the preceding kernel
        if (lane == 0)
            for (int n = 0; n < HB_STAGES && n < n_mine; ++n) load_state_of(n);
        if (p.use_pdl) {
            pdl_wait();
            pdl_launch_dependents();
        }
        // activations of the two channels of this lane, fetched one item ahead
        struct Act { float r[2], k[2], v[2], w_raw[2], a_raw[2], vg_raw[2], vf[2]; };
        auto fetch = [&](int n, Act& a) {
            const int it = item_of(n), b = it / p.H, h = it - b * p.H;
            const size_t off = (size_t)b * p.D + h * 64;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e;
                a.r[e] = lda(p.r + off + c);
                a.k[e] = lda(p.k + off + c);
                a.v[e] = lda(p.v + off + c);
                a.w_raw[e] = lda(p.w_raw + off + c);
                a.a_raw[e] = lda(p.a_raw + off + c);
                if (!p.layer0) {
                    a.vg_raw[e] = lda(p.vg_raw + off + c);
                    a.vf[e] = lda(p.v_first + off + c);
                }
            }
        };
        // reference/rwkv7.py:284-297 for one (sequence, head): vectors of the recurrence into `o`
        auto glue = [&](int n, const Act& a, HeadVec& o) {
            const int it = item_of(n), b = it / p.H, h = it - b * p.H;
            const size_t off = (size_t)b * p.D + h * 64;
            float kk0[2], av[2];
            float ssq = 0.f, rkr = 0.f;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e, gc = h * 64 + c;
                const float rr = a.r[e], kr = a.k[e];
                float vv = a.v[e];
                const float aa = rh(sigmoidf_(rh(__half2float(p.a0[gc]) + a.a_raw[e])));
                kk0[e] = rh(kr * __half2float(p.k_k[gc]));
                ssq = fmaf(kk0[e], kk0[e], ssq);
                const float k2 = rh(kr * rh(1.f + rh(rh(aa - 1.f) * __half2float(p.k_a[gc]))));
                if (p.layer0) {
                    p.v_first[off + c] = __float2half_rn(vv);
                } else {
                    const float vg = rh(sigmoidf_(rh(__half2float(p.v0[gc]) + a.vg_raw[e])));
                    vv = rh(vv + rh(rh(a.vf[e] - vv) * vg));
                }
                const float wd = __expf(-0.606531f * sigmoidf_(rh(__half2float(p.w0[gc]) + a.w_raw[e])));
                o.r[c] = rr; o.w[c] = wd; o.k[c] = k2; o.v[c] = vv;
                av[e] = aa;
                rkr += rh(rh(rr * k2) * __half2float(p.r_k[gc]));
            }
            ssq = warp_sum(ssq);
            rkr = rh(warp_sum(rkr));
            const float nrm = fmaxf(rh(sqrtf(ssq)), 1e-12f);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e;
                const float kk = rh(kk0[e] / nrm);
                o.a[c] = -kk;
                o.b[c] = rh(kk * av[e]);
            }
            if (lane == 0) o.rkr = rkr;
        };
        Act act;
        if (n_mine > 0) {
            fetch(0, act);
            glue(0, act, vec[0]);
            bar_arrive_id(1, HB_THREADS);
        }
        for (int n = 0; n < n_mine; ++n) {
            if (n + 1 < n_mine) {
                fetch(n + 1, act);
                glue(n + 1, act, vec[(n + 1) & 1]);
                bar_arrive_id(1 + ((n + 1) & 1), HB_THREADS);
            }
            bar_sync_id(3 + (n & 1), HB_THREADS);   // item n: state consumed, read-out in sy
            if (lane == 0 && n + HB_STAGES < n_mine) load_state_of(n + HB_STAGES);
            // group norm over the head's 64 channels (eps 64e-5), bonus, gate (reference/rwkv7.py:297-299)
            const int it = item_of(n), b = it / p.H, h = it - b * p.H;
            const size_t off = (size_t)b * p.D + h * 64;
            const HeadVec& cv = vec[n & 1];
            const float y0 = sy[n & 1][lane], y1 = sy[n & 1][lane + 32];
            const float mean = warp_sum(y0 + y1) * (1.f / 64.f);
            const float d0 = y0 - mean, d1 = y1 - mean;
            const float var = warp_sum(d0 * d0 + d1 * d1) * (1.f / 64.f);
            const float rstd = rsqrtf(var + 64e-5f);
            const float rkr = cv.rkr;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = lane + 32 * e, gc = h * 64 + c;
                float o = rh((e ? d1 : d0) * rstd * __half2float(p.lnx_w[gc]) + __half2float(p.lnx_b[gc]));
                o = rh(o + rh(rkr * cv.v[c]));
                p.out[off + c] = __float2half_rn(o * lda(p.g + off + c));
            }
            __syncwarp();
        }
    } else {
        const int i = tid >> 2, q = tid & 3;
        if (p.use_pdl) pdl_wait();   // the stores below must not pass the preceding kernel either
        for (int n = 0; n < n_mine; ++n) {
            const int s = n % HB_STAGES;
            if (!*reinterpret_cast<volatile int*>(&s_failed) && !mbar_wait_bounded(&full[s], (uint32_t)(n / HB_STAGES) & 1u, 1u << 16)) {
                *reinterpret_cast<volatile int*>(&s_failed) = 1;
                atomicOr(&g_device_status, DEV_WAIT_HEAD);
            }
            const float* srow = reinterpret_cast<const float*>(dsm + s * HB_STATE_BYTES) + i * 64;
            float4 st[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) st[e] = *reinterpret_cast<const float4*>(srow + 16 * ((e + i) & 3) + 4 * q);
            bar_sync_id(1 + (n & 1), HB_THREADS);
            const HeadVec& cv = vec[n & 1];
            float sa = 0.f;
            float4 a4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                a4[e] = *reinterpret_cast<const float4*>(cv.a + 16 * ((e + i) & 3) + 4 * q);
                sa = fmaf(a4[e].x, st[e].x, sa); sa = fmaf(a4[e].y, st[e].y, sa);
                sa = fmaf(a4[e].z, st[e].z, sa); sa = fmaf(a4[e].w, st[e].w, sa);
            }
            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
            sa += __shfl_xor_sync(0xffffffffu, sa, 2);
            const float v_i = cv.v[i];
            float y = 0.f;
            float* gout = p.state + (size_t)item_of(n) * 4096 + i * 64;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c0 = 16 * ((e + i) & 3) + 4 * q;
                const float4 w4 = *reinterpret_cast<const float4*>(cv.w + c0), k4 = *reinterpret_cast<const float4*>(cv.k + c0);
                const float4 b4 = *reinterpret_cast<const float4*>(cv.b + c0), r4 = *reinterpret_cast<const float4*>(cv.r + c0);
                float4 o;
                o.x = fmaf(st[e].x, w4.x, fmaf(k4.x, v_i, sa * b4.x)); y = fmaf(o.x, r4.x, y);
                o.y = fmaf(st[e].y, w4.y, fmaf(k4.y, v_i, sa * b4.y)); y = fmaf(o.y, r4.y, y);
                o.z = fmaf(st[e].z, w4.z, fmaf(k4.z, v_i, sa * b4.z)); y = fmaf(o.z, r4.z, y);
                o.w = fmaf(st[e].w, w4.w, fmaf(k4.w, v_i, sa * b4.w)); y = fmaf(o.w, r4.w, y);
                st_cs16(gout + c0, o);
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (q == 0) sy[n & 1][i] = rh(y);
            bar_arrive_id(3 + (n & 1), HB_THREADS);
        }
    }
}

}  // namespace

int head_launch(const HeadParams& p, cudaStream_t stream) {
    AB_CHECK_ARG(p.B > 0 && p.T > 0 && p.H > 0 && p.D == p.H * HEAD, "head: bad shape B=%d T=%d D=%d H=%d", p.B, p.T, p.D, p.H);
    AB_CHECK_ARG(p.state && p.r && p.k && p.v && p.v_first && p.out, "head: null pointer");
    const bool ups = p.w2 != nullptr;
    AB_CHECK_ARG(ups || (p.w_raw && p.a_raw && p.g && (p.layer0 || p.vg_raw)), "head: adapter outputs missing");
    AB_CHECK_ARG(!ups || (p.B == 1 && p.T == 1), "head: in-kernel adapter up-projection is the batch-1 path");
    if (!ups && p.T == 1 && p.B * p.H >= 512) {
        // many sequences, one step each: persistent blocks with the state staged by bulk copies
        static int n_sm = 0;
        if (!n_sm) {
            int dev = 0, v = 0;
            AB_CUDA(cudaGetDevice(&dev));
            AB_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            AB_CUDA(cudaFuncSetAttribute(head_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HB_STAGES * HB_STATE_BYTES));
            n_sm = v;
        }
        AB_CHECK_ARG(((uintptr_t)p.state & 15) == 0, "head: state must be 16-byte aligned");
        const int n_items = p.B * p.H;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)min(n_items, 3 * n_sm));
        cfg.blockDim = dim3(HB_THREADS);
        cfg.dynamicSmemBytes = HB_STAGES * HB_STATE_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = p.use_pdl ? 1 : 0;
        AB_CUDA(cudaLaunchKernelEx(&cfg, head_batch_kernel, p, n_items));
        return OK;
    }
    size_t smem = 0;
    if (ups) {
        const int rtot = p.rw + p.ra + p.rv + p.rg;
        smem = (size_t)rtot * 128 + (size_t)((rtot + 3) & ~3) * 4 + 8 * 4 * 64 * 4;
    }
    static size_t max_smem = 0;
    if (!max_smem) {
        int dev = 0, m = 0;
        AB_CUDA(cudaGetDevice(&dev));
        AB_CUDA(cudaDeviceGetAttribute(&m, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        AB_CUDA(cudaFuncSetAttribute(head_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, m - 4096));
        max_smem = (size_t)m - 4096;
    }
    if (smem > max_smem) {
        set_error("head: adapter ranks need %zu bytes of shared memory (limit %zu)", smem, max_smem);
        return ERR_TOO_LARGE;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.B * p.H));
    cfg.blockDim = dim3(HT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.use_pdl ? 1 : 0;
    AB_CUDA(cudaLaunchKernelEx(&cfg, head_fused_kernel, p));
    return OK;
}

int wkv7_launch(int B, int T, int C, int H, float* state, const __half* r, const __half* w, const __half* k,
                const __half* v, const __half* a, const __half* b, __half* y, cudaStream_t stream) {
    AB_CHECK_ARG(B > 0 && T > 0 && H > 0 && C == H * HEAD, "wkv7: need C == H*64 (B=%d T=%d C=%d H=%d)", B, T, C, H);
    AB_CHECK_ARG(state && r && w && k && v && a && b && y, "wkv7: null pointer");
    AB_CHECK_ARG(((uintptr_t)state & 15) == 0, "wkv7: state must be 16-byte aligned");
    wkv7_kernel<<<B * H, HT, 0, stream>>>(T, C, H, state, r, w, k, v, a, b, y);
    AB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace ab
