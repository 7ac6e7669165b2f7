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
__global__ void __launch_bounds__(HT, 2) head_fused_kernel(const __grid_constant__ HeadParams p) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ HeadShared sh;
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, i = tid >> 2, q = tid & 3;
    const bool ups = p.w2 != nullptr;

    // ---- batch-1 path: pull this head's slices of the four up-projection matrices into smem.
    // They are weights, so this runs before the wait on the previous kernel.
    if (ups) head_ups_stage(p, h, tid, dsm);
    if (p.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }

    float* sbase = p.state + (size_t)bh * 4096;
    StateRow st;
    load_state(st, sbase, i, q);

    if (ups) {
        head_ups_compute(p, tid, dsm, sh, SyncBlock());
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
// around keeping it moving, and nothing on an item's critical path waits for a global load:
//   * warps 0-7 (256 threads) run the recurrence. The item's state arrives as ONE 16 KiB bulk copy into a ring of
//     HB_STAGES shared-memory stages (mbarrier, byte-counted) ahead of the item being worked on; the updated state
//     is written back into its stage and leaves as ONE 16 KiB bulk copy as well, so no warp ever waits for the
//     memory system to accept a store (register -> global stores made the step itself take 2.6 us per item).
//   * warp 8 ("pre") turns the projections of item n+1 into the vectors of the recurrence (k normalisation and
//     modulation, v residual gate, decay) while warps 0-7 are on item n; its inputs were fetched an item earlier.
//     Its lane 0 issues the first bulk copies; thread 0 issues the write-backs and the later loads.
//   * warp 9 ("post") turns the read-out of item n into the block output (group norm, bonus, gate).
// Thread (i = tid/4, q = tid%4) owns, of state row i, the four 16-byte chunks {4m + q, m = 0..3} and visits them in
// the order m = (e + i) % 4: a quarter-warp then reads eight different bank groups of the stage (no conflicts).
// Helper lanes own channels 2*lane and 2*lane+1 (one 32-bit load per vector).
#ifndef HB_STAGES_
#define HB_STAGES_ 4
#endif
#ifndef HB_BLOCKS_
#define HB_BLOCKS_ 3
#endif
constexpr int HB_STAGES = HB_STAGES_;
constexpr int HB_BLOCKS = HB_BLOCKS_;   // resident blocks per SM
constexpr int HB_THREADS = HT + 64;
constexpr int HB_STATE_BYTES = 64 * 64 * 4;

// Vectors of one recurrence step. r, k, a, b are fp16 values anyway (each is the result of an fp16-rounded op), so
// they are kept as fp16: every thread reads 16 elements of each per item, and the shared-memory pipe, not HBM, paces
// the step; 8-byte instead of 16-byte reads take half the wavefronts. The decay w is fp32.
struct HeadVec {
    float w[64], v[64];
    __half r[64], k[64], a[64], b[64];
};
__device__ __forceinline__ float4 ld_h4(const __half* p) {   // four consecutive fp16 -> float4
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
struct HeadPost {   // what the output stage needs from the input stage
    float v[64];
    float rkr;
    float pad[3];
};

__device__ __forceinline__ void bar_sync_id(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive_id(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n cp.async.bulk.commit_group;" ::"l"(dst),
                 "r"(smem_u32(src)), "r"(bytes)
                 : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// two adjacent fp16 channels; activations bypass L1 (written by another SM in an earlier kernel)
__device__ __forceinline__ float2 ld2a(const __half* p) { return __half22float2(__ldcg(reinterpret_cast<const __half2*>(p))); }
__device__ __forceinline__ float2 ld2p(const __half* p) { return __half22float2(__ldg(reinterpret_cast<const __half2*>(p))); }

__global__ void __launch_bounds__(HB_THREADS, HB_BLOCKS) head_batch_kernel(const __grid_constant__ HeadParams p, int n_items) {
    extern __shared__ __align__(128) unsigned char dsm[];   // HB_STAGES x 16 KiB
    __shared__ __align__(16) HeadVec vec[2];
    __shared__ __align__(16) HeadPost post[3];
    __shared__ float sy[4][64];
    __shared__ uint64_t full[HB_STAGES];
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_mine = ((int)blockIdx.x < n_items) ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    auto item_of = [&](int n) { return (int)blockIdx.x + n * (int)gridDim.x; };
    auto off_of = [&](int n) {   // element offset of the item's 64 channels in a [B, D] activation
        const int it = item_of(n), b = it / p.H, h = it - b * p.H;
        return (size_t)b * p.D + h * 64;
    };
    if (tid == 0) {
        for (int s = 0; s < HB_STAGES; ++s) mbar_init(&full[s], 1);
        fence_mbar_init();
        s_failed = 0;
    }
    __syncthreads();
    // Named barriers. 1, 2: the vectors of an even / odd item are ready (pre arrives, warps 0-7 wait).
    // 3, 4: the recurrence of an even / odd item is done (warps 0-7 arrive, pre and post wait).
    // 5: warps 0-7 have written an item's new state into its stage.
    constexpr int N_VEC = HT + 32, N_DONE = HT + 64;
    if (warp == 8) {
        auto load_state_of = [&](int n) {
            const int s = n % HB_STAGES;
            mbar_expect_tx(&full[s], HB_STATE_BYTES);
            (void)AB_BC(item_of(n) >= 0 && item_of(n) < n_items);   // checked build: recorded; the copy itself is not skipped (its barrier expects it)
            bulk_g2s(dsm + s * HB_STATE_BYTES, p.state + (size_t)item_of(n) * 4096, HB_STATE_BYTES, &full[s]);
        };
        // The state is requested BEFORE the wait for the preceding grid. That is safe because its last writer is this
        // same kernel one decode step earlier, hundreds of launches back, and programmatic launch cannot stack that
        // deep: a grid may start early only once EVERY block of its predecessor has started, and no block of any
        // grid of the step exits before its own wait has passed, i.e. before the grid in front of it is complete.
        // For this request to overtake that writer, all blocks of all launches in between would have to be resident
        // at once; the products between two head launches alone are hundreds of blocks that each fill an SM.
        if (lane == 0)
            for (int n = 0; n < HB_STAGES && n < n_mine; ++n) load_state_of(n);
        if (p.use_pdl) {
            pdl_wait();
            pdl_launch_dependents();
        }
        // Everything the input stage reads from global memory, activations and per-channel parameters alike, is
        // requested one item ahead and kept packed (two fp16 per register): the stage is on the critical path of the
        // block (item n+1 cannot start before it is done), so it must not wait for a load.
        struct Act { __half2 r, k, v, w_raw, a_raw, vg_raw, vf, a0, k_k, k_a, w0, r_k, v0; };
        auto ldh2a = [](const __half* q) { return __ldcg(reinterpret_cast<const __half2*>(q)); };
        auto ldh2p = [](const __half* q) { return __ldg(reinterpret_cast<const __half2*>(q)); };
        auto fetch = [&](int n, Act& a) {
            const size_t o = off_of(n) + 2 * lane;
            const int gc = (item_of(n) % p.H) * 64 + 2 * lane;
            a.r = ldh2a(p.r + o); a.k = ldh2a(p.k + o); a.v = ldh2a(p.v + o);
            a.w_raw = ldh2a(p.w_raw + o); a.a_raw = ldh2a(p.a_raw + o);
            a.a0 = ldh2p(p.a0 + gc); a.k_k = ldh2p(p.k_k + gc); a.k_a = ldh2p(p.k_a + gc);
            a.w0 = ldh2p(p.w0 + gc); a.r_k = ldh2p(p.r_k + gc);
            if (!p.layer0) { a.vg_raw = ldh2a(p.vg_raw + o); a.vf = ldh2a(p.v_first + o); a.v0 = ldh2p(p.v0 + gc); }
        };
        // reference/rwkv7.py:284-297 for one (sequence, head)
        auto glue = [&](int n, const Act& a, HeadVec& o, HeadPost& po) {
            const float2 fr = __half22float2(a.r), fk = __half22float2(a.k), fv = __half22float2(a.v);
            const float2 fwr = __half22float2(a.w_raw), far = __half22float2(a.a_raw);
            const float2 a0 = __half22float2(a.a0), k_k = __half22float2(a.k_k), k_a = __half22float2(a.k_a);
            const float2 w0 = __half22float2(a.w0), r_k = __half22float2(a.r_k);
            const float rr[2] = {fr.x, fr.y}, kr[2] = {fk.x, fk.y};
            float vv[2] = {fv.x, fv.y};
            const float a_raw[2] = {far.x, far.y}, w_raw[2] = {fwr.x, fwr.y};
            const float a0_[2] = {a0.x, a0.y}, kk_[2] = {k_k.x, k_k.y}, ka_[2] = {k_a.x, k_a.y};
            const float w0_[2] = {w0.x, w0.y}, rk_[2] = {r_k.x, r_k.y};
            if (p.layer0) {
                *reinterpret_cast<__half2*>(p.v_first + off_of(n) + 2 * lane) = __floats2half2_rn(vv[0], vv[1]);
            } else {
                const float2 v0 = __half22float2(a.v0), fvg = __half22float2(a.vg_raw), fvf = __half22float2(a.vf);
                const float v0_[2] = {v0.x, v0.y}, vg_raw[2] = {fvg.x, fvg.y}, vf[2] = {fvf.x, fvf.y};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float vg = rh(sigmoidf_(rh(v0_[e] + vg_raw[e])));
                    vv[e] = rh(vv[e] + rh(rh(vf[e] - vv[e]) * vg));
                }
            }
            float kk0[2], av[2];
            float ssq = 0.f, rkr = 0.f;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * lane + e;
                const float aa = rh(sigmoidf_(rh(a0_[e] + a_raw[e])));
                kk0[e] = rh(kr[e] * kk_[e]);
                ssq = fmaf(kk0[e], kk0[e], ssq);
                const float k2 = rh(kr[e] * rh(1.f + rh(rh(aa - 1.f) * ka_[e])));
                // decay in fp32 as on the reference's single-token path (reference/rwkv7.py:241)
                const float wd = __expf(-0.606531f * sigmoidf_(rh(w0_[e] + w_raw[e])));
                o.r[c] = __float2half_rn(rr[e]); o.w[c] = wd; o.k[c] = __float2half_rn(k2); o.v[c] = vv[e];
                po.v[c] = vv[e];
                av[e] = aa;
                rkr += rh(rh(rr[e] * k2) * rk_[e]);
            }
            ssq = warp_sum(ssq);
            rkr = rh(warp_sum(rkr));
            const float nrm = fmaxf(rh(sqrtf(ssq)), 1e-12f);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float kk = rh(kk0[e] / nrm);
                o.a[2 * lane + e] = __float2half_rn(-kk);
                o.b[2 * lane + e] = __float2half_rn(kk * av[e]);
            }
            if (lane == 0) po.rkr = rkr;
        };
        Act cur, nxt;
        if (n_mine > 0) {
            fetch(0, cur);
            if (n_mine > 1) fetch(1, nxt);
            glue(0, cur, vec[0], post[0]);
            bar_arrive_id(1, N_VEC);
            cur = nxt;
        }
        for (int n = 0; n + 1 < n_mine; ++n) {
            // cur = inputs of item n+1 (fetched an iteration ago); start on those of item n+2
            if (n + 2 < n_mine) fetch(n + 2, nxt);
            if (n > 0) {
                bar_sync_id(3 + ((n - 1) & 1), N_DONE);   // item n-1 is through: its vectors are free
            }
            glue(n + 1, cur, vec[(n + 1) & 1], post[(n + 1) % 3]);
            bar_arrive_id(1 + ((n + 1) & 1), N_VEC);
            cur = nxt;
        }
        // the barriers of the last items still expect this warp
        for (int n = max(n_mine - 1, 1); n <= n_mine; ++n) bar_sync_id(3 + ((n - 1) & 1), N_DONE);
    } else if (warp == 9) {
        if (p.use_pdl) pdl_wait();
        float2 g_cur = make_float2(0.f, 0.f), g_nxt = g_cur;
        if (n_mine > 0) g_cur = ld2a(p.g + off_of(0) + 2 * lane);
        for (int n = 0; n < n_mine; ++n) {
            if (n + 1 < n_mine) g_nxt = ld2a(p.g + off_of(n + 1) + 2 * lane);
            const int it = item_of(n), h = it % p.H, gc = h * 64 + 2 * lane;
            const float2 lw = ld2p(p.lnx_w + gc), lb = ld2p(p.lnx_b + gc);
            bar_sync_id(3 + (n & 1), N_DONE);
            // group norm over the head's 64 channels (eps 64e-5), bonus, gate (reference/rwkv7.py:297-299)
            const HeadPost& po = post[n % 3];
            const float2 y2 = *reinterpret_cast<const float2*>(&sy[n & 3][2 * lane]);
            const float mean = warp_sum(y2.x + y2.y) * (1.f / 64.f);
            const float d0 = y2.x - mean, d1 = y2.y - mean;
            const float var = warp_sum(d0 * d0 + d1 * d1) * (1.f / 64.f);
            const float rstd = rsqrtf(var + 64e-5f);
            const float rkr = po.rkr;
            const float2 v2 = *reinterpret_cast<const float2*>(&po.v[2 * lane]);
            float o0 = rh(d0 * rstd * lw.x + lb.x), o1 = rh(d1 * rstd * lw.y + lb.y);
            o0 = rh(o0 + rh(rkr * v2.x));
            o1 = rh(o1 + rh(rkr * v2.y));
            *reinterpret_cast<__half2*>(p.out + off_of(n) + 2 * lane) = __floats2half2_rn(o0 * g_cur.x, o1 * g_cur.y);
            g_cur = g_nxt;
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
            float* srow = reinterpret_cast<float*>(dsm + s * HB_STATE_BYTES) + i * 64;
            float4 st[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) st[e] = *reinterpret_cast<const float4*>(srow + 16 * ((e + i) & 3) + 4 * q);
            bar_sync_id(1 + (n & 1), N_VEC);
            const HeadVec& cv = vec[n & 1];
            float sa = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float4 a4 = ld_h4(cv.a + 16 * ((e + i) & 3) + 4 * q);
                sa = fmaf(a4.x, st[e].x, sa); sa = fmaf(a4.y, st[e].y, sa);
                sa = fmaf(a4.z, st[e].z, sa); sa = fmaf(a4.w, st[e].w, sa);
            }
            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
            sa += __shfl_xor_sync(0xffffffffu, sa, 2);
            const float v_i = cv.v[i];
            float y = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c0 = 16 * ((e + i) & 3) + 4 * q;
                const float4 w4 = *reinterpret_cast<const float4*>(cv.w + c0), k4 = ld_h4(cv.k + c0);
                const float4 b4 = ld_h4(cv.b + c0), r4 = ld_h4(cv.r + c0);
                float4 o;
                o.x = fmaf(st[e].x, w4.x, fmaf(k4.x, v_i, sa * b4.x)); y = fmaf(o.x, r4.x, y);
                o.y = fmaf(st[e].y, w4.y, fmaf(k4.y, v_i, sa * b4.y)); y = fmaf(o.y, r4.y, y);
                o.z = fmaf(st[e].z, w4.z, fmaf(k4.z, v_i, sa * b4.z)); y = fmaf(o.z, r4.z, y);
                o.w = fmaf(st[e].w, w4.w, fmaf(k4.w, v_i, sa * b4.w)); y = fmaf(o.w, r4.w, y);
                *reinterpret_cast<float4*>(srow + c0) = o;   // same chunk this thread read: nobody else touches it
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (q == 0) sy[n & 3][i] = rh(y);
            bar_arrive_id(3 + (n & 1), N_DONE);
            fence_proxy_async();   // the stage is about to be read by the bulk-copy unit
            bar_sync_id(5, HT);
            if (tid == 0) {
                bulk_s2g(p.state + (size_t)item_of(n) * 4096, dsm + s * HB_STATE_BYTES, HB_STATE_BYTES);
                // all write-backs but the newest have left shared memory: the previous item's stage can be refilled
                bulk_wait_read<1>();
                const int m = n - 1 + HB_STAGES;
                if (n >= 1 && m < n_mine) {
                    const int sm = m % HB_STAGES;
                    mbar_expect_tx(&full[sm], HB_STATE_BYTES);
                    bulk_g2s(dsm + sm * HB_STATE_BYTES, p.state + (size_t)item_of(m) * 4096, HB_STATE_BYTES, &full[sm]);
                }
            }
        }
        if (tid == 0) bulk_wait_all();   // every write-back has reached global memory before the block ends
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
        static PerDeviceOnce once;
        const DeviceProps* dp = nullptr;
        {
            const int s = once.run(&dp, [](DeviceProps&) -> int {
                return check_cuda(cudaFuncSetAttribute(head_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HB_STAGES * HB_STATE_BYTES),
                                  "cudaFuncSetAttribute(head_batch_kernel)");
            });
            if (s != OK) return s;
        }
        const int n_sm = dp->n_sm;
        AB_CHECK_ARG(((uintptr_t)p.state & 15) == 0, "head: state must be 16-byte aligned");
        const int n_items = p.B * p.H;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)min(n_items, HB_BLOCKS * n_sm));
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
        smem = head_ups_smem(p.rw + p.ra + p.rv + p.rg);
    }
    static PerDeviceOnce once_fused;
    const DeviceProps* dpf = nullptr;
    {
        const int s = once_fused.run(&dpf, [](DeviceProps& d) -> int {
            return check_cuda(cudaFuncSetAttribute(head_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d.smem_optin - 4096),
                              "cudaFuncSetAttribute(head_fused_kernel)");
        });
        if (s != OK) return s;
    }
    const size_t max_smem = dpf->smem_optin - 4096;
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
