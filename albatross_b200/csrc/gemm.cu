// Batched matrix products of the RWKV-7 batch path on the 5th-generation tensor cores (tcgen05 / TMEM),
// and the de-quantisation dump.
//
// Replaces the `[B,T,D] @ W` call sites of reference/rwkv7.py:283-288, :293, :300 (time-mix), :322-323
// (channel-mix) and :220 (vocabulary head) with weight-only int8 / NVFP4 / fp16 weights.
//
//   D[128 weight rows, N batch rows] (fp32, TMEM) += A[128, 64] (weights, fp16) * B[N, 64]^T (activations, fp16)
//
// The weights are the M side of the MMA so that every weight byte is read from HBM exactly once per
// N tile; the batch (up to 320 rows per block: an MMA of N = 192 and one for the rest) is the N side.
//   producer groups (G_NG groups of 4 warps; thread = one of the block's 128 weight rows): group g owns
//               k-steps g, g + G_NG, ... It brings the row's 64 inputs of a k-step in (cp.async ring of raw
//               quantised bytes; fp16 rows go straight to registers), de-quantises in registers (int8 ->
//               fp16 exactly; e2m1 x e4m3 block scale -> fp16 exactly) and writes them to tensor memory
//               (tcgen05.st: its 32 registers = 32 columns of its own TMEM lane), from where the MMA reads its
//               weight operand; shared memory carries only the activation tiles. (Compiled with G_A_TMEM_=0
//               the weights go to shared memory instead, K-major with the 128-byte swizzle.)
//               One warp per scheduler cannot hide the latencies of this
//               serial instruction stream; several groups on different k-steps can. Afterwards all groups
//               run the epilogue: tcgen05.ld of 32 columns of their 32 TMEM lanes, row / tensor scale,
//               activation or residual; the fp16 tile is laid out in shared memory and leaves through TMA stores
//               (a residual tile comes in through TMA loads); products with a ragged row pitch store directly;
//   next warp : one thread issues the TMA loads of the activation tile (tensor map over X, 128B swizzle);
//   last warp : allocates TMEM; one thread issues tcgen05.mma (kind::f16) and commits to mbarriers.
// Four-stage operand ring, all waits bounded (status word on expiry), TMEM freed on every path. Short grids with
// long K loops are split along K: every block of a tile finishes a share of its 32-row chunks, fetching the other
// blocks' fp32 partial sums of them from a scratch area with bulk copies and adding them in a fixed order. Launched with
// programmatic stream serialisation the kernel starts its weight stream before it waits for its predecessor.
#include <cuda.h>

#include <type_traits>

#include "gemm.cuh"
#include "gemv.cuh"

namespace ab {

namespace {

#ifndef G_NG_
#define G_NG_ 3
#endif
constexpr int G_NG = G_NG_;      // producer groups
constexpr int G_PROD = 128 * G_NG;
constexpr int GT = G_PROD + 128; // threads per block: producers + a warpgroup holding the TMA warp, the MMA warp and two idle warps
                                 // (register re-allocation works on whole, aligned warpgroups)
#ifndef G_A_TMEM_
#define G_A_TMEM_ 1
#endif
#ifndef G_STAGES_
#define G_STAGES_ 4
#endif
constexpr int G_STAGES = G_STAGES_;
constexpr bool G_A_TMEM = G_A_TMEM_ != 0;   // de-quantised weights go to tensor memory instead of shared memory
constexpr int G_A_COLS = 32;             // TMEM columns of one weight stage: 64 inputs as fp16 pairs
constexpr int G_BM = 128;        // weight rows per block
constexpr int G_BK = 64;         // inputs per k-step (128 bytes of fp16 = one swizzle row)
constexpr int G_A_BYTES = G_BM * G_BK * 2;
constexpr int G_RAW_BYTES = 56 * 1024;   // rings of raw (still quantised) weight k-steps filled by cp.async
constexpr int G_RAW_GROUP = (G_RAW_BYTES / G_NG) & ~1023;   // one ring per producer group
constexpr int G_REGS_PROD = 136, G_REGS_REST = 96;   // (136 - 128) * 384 producer threads <= (128 - 96) * 128 others
constexpr int G_MAX_OPS = 8;
constexpr int G_COUNTERS = 4096;         // split-K arrival counters at the start of the scratch area

// One matrix product of a grouped launch.
struct GemmProb {
    ab_mat w;
    const __half* resid;
    __half* y;
    int epi;
    int cta_base;     // first blockIdx.x of this product
    int ksplit;       // blocks that share one output tile along K
    int tile_base;    // first split-K tile id (counter / partial index)
    long long part_base;   // float offset of its split-K partial sums in the scratch area
    int tma_out;      // output (and residual) tiles go through shared memory and the TMA unit
    int recv_slots;   // split K: own chunks whose slices fit the receive area at a time
};
struct GemmGroup {
    GemmProb pr[G_MAX_OPS];
    int n_prob;
    int rows;       // batch rows (B*T)
    int n_tile;     // batch rows per block tile
    int n_first;    // batch rows of the first MMA of a k-substep (n_tile, or 192 when a second MMA takes the rest)
    int tma_rows;   // batch rows per TMA box
    int tmem_cols;
    int a_col0;     // first TMEM column of the weight stages (behind the accumulators)
    unsigned* counters;
    float* partials;
    int recv_off;   // split K: byte offset of the area the partial sums are fetched to, in the block's shared memory
};
struct GemmMaps {
    CUtensorMap m[G_MAX_OPS];   // activations X
    CUtensorMap y[G_MAX_OPS];   // outputs Y, boxes of 32 batch rows x 128 features
    CUtensorMap r[G_MAX_OPS];   // residuals, same boxes
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers (tcgen05 / TMA)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
                 "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_drain_reads() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// The same product with the weight operand read from tensor memory (128 lanes = weight rows, 8 columns = 16 inputs
// as fp16 pairs) instead of shared memory.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 registers of each of the warp's 32 lanes -> 32 consecutive TMEM columns of its 32 lanes.
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src, bool ok) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(ok ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(G_PROD) : "memory"); }
__device__ __forceinline__ void group_sync(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory"); }   // one producer group
constexpr int G_CHUNK_F32 = 32 * G_BM * 4;   // fp32 partial sums of 32 batch rows x 128 features

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem) {
    const uint32_t a = smem_u32(smem);
    uint64_t d = (uint64_t)((a >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset: unused with swizzled K-major tiles
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// De-quantise the 64 inputs of this thread's row from a landed ring slot into eight 16-byte chunks of fp16
// (chunk c = inputs 8c..8c+7). Invalid rows / inputs were zero-filled by the copy.
__device__ __forceinline__ void raw_dequant(int fmt, int r_local, const unsigned char* slot, uint4* out) {
    if (fmt == FMT_I8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 raw = *reinterpret_cast<const uint4*>(slot + q * 2048 + r_local * 16);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t h[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // int8 -> fp16 exactly: bytes b0, b1 into the mantissas of 1024 + (b ^ 0x80), then subtract 1152
                const uint32_t x = words[e] ^ 0x80808080u;
                const uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140), hi = __byte_perm(x, 0x64646464u, 0x4342);
                const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
                const __half2 l2 = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
                const __half2 h2 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
                h[2 * e] = *reinterpret_cast<const uint32_t*>(&l2);
                h[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            out[2 * q] = make_uint4(h[0], h[1], h[2], h[3]);
            out[2 * q + 1] = make_uint4(h[4], h[5], h[6], h[7]);
        }
    } else if (fmt == FMT_F16) {
#pragma unroll
        for (int c = 0; c < 8; ++c) out[c] = *reinterpret_cast<const uint4*>(slot + c * 2048 + r_local * 16);
    } else {
        const uint4 r0 = *reinterpret_cast<const uint4*>(slot + r_local * 16);
        const uint4 r1 = *reinterpret_cast<const uint4*>(slot + 2048 + r_local * 16);
        const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(slot + 4096 + r_local * 4);
        const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        // the four block scales of these 64 inputs, each duplicated into both halves of a half2
        const __half2 s01 = e4m3x2_to_half2(sc4 & 0xffffu), s23 = e4m3x2_to_half2(sc4 >> 16);
        const __half2 scs[4] = {__low2half2(s01), __high2half2(s01), __low2half2(s23), __high2half2(s23)};
#pragma unroll
        for (int c = 0; c < 8; ++c) {   // chunk c: 8 inputs = 4 bytes; scale block = c / 2
            uint32_t h[4];
            e2m1x8_to_half2x4(words[c], h);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&h[e]), scs[c >> 1]);   // exact in fp16
                h[e] = *reinterpret_cast<const uint32_t*>(&v);
            }
            out[c] = make_uint4(h[0], h[1], h[2], h[3]);
        }
    }
}

template <int EPI>
__device__ __forceinline__ float apply_epi_t(float o) {
    if (EPI == EPI_TANH) return tanhf(o);
    if (EPI == EPI_SIGMOID) return sigmoidf_(o);
    if (EPI == EPI_RELU2) { o = fmaxf(o, 0.f); return o * o; }
    return o;
}
__device__ __forceinline__ float apply_epi(int epi, float o) {
    switch (epi) {
        case EPI_TANH: return tanhf(o);
        case EPI_SIGMOID: return sigmoidf_(o);
        case EPI_RELU2: o = fmaxf(o, 0.f); return o * o;
        default: return o;
    }
}

// SPLIT: some product of the launch is split along K (the lean instance is compiled without that ending).
template <bool SPLIT>
__global__ void __launch_bounds__(GT, 1) gemm_tc_kernel(const __grid_constant__ GemmMaps maps,
                                                        const __grid_constant__ GemmGroup g) {
    extern __shared__ __align__(1024) unsigned char gsm[];
    __shared__ uint64_t full[G_STAGES], empty[G_STAGES], accum_bar, resid_bar, recv_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // ---- which product, which tile, which K split
    int pi = 0;
    while (pi + 1 < g.n_prob && (int)blockIdx.x >= g.pr[pi + 1].cta_base) ++pi;
    const GemmProb& pb = g.pr[pi];
    const int local = blockIdx.x - pb.cta_base;
    const int m_tile = local / pb.ksplit, z = local - m_tile * pb.ksplit;
    const int m0 = m_tile * G_BM;
    const int n0 = blockIdx.y * g.n_tile;
    const int total_ksteps = (pb.w.k + G_BK - 1) / G_BK;
    const int ks_begin = (int)((long long)total_ksteps * z / pb.ksplit);
    const int ks_end = (int)((long long)total_ksteps * (z + 1) / pb.ksplit);
    const int n_ksteps = ks_end - ks_begin;
    // Blocks walk K in rotated order: at any moment they read different columns of the (shared) activation
    // matrix, instead of all hitting the same few L2 lines.
    const int rot = (int)((blockIdx.x * 7u + blockIdx.y * 3u) % (unsigned)n_ksteps);
    auto kstep_of = [&](int i) { int k = i + rot; if (k >= n_ksteps) k -= n_ksteps; return ks_begin + k; };

    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
    const int b_bytes = g.n_tile * 128;
    unsigned char* smA = base;                                  // G_STAGES x 16 KB (unused when the weights go to TMEM)
    unsigned char* smB = base + (G_A_TMEM ? 0 : G_STAGES * G_A_BYTES);   // G_STAGES x n_tile x 128 B
    unsigned char* smRaw = smB + G_STAGES * b_bytes;            // raw weight ring

    if (tid == 0) {
        for (int s = 0; s < G_STAGES; ++s) {
            mbar_init(&full[s], 5);   // the four warps of the group that owns the k-step + the TMA thread's expect_tx
            mbar_init(&empty[s], 1);
        }
        mbar_init(&accum_bar, 1);
        mbar_init(&resid_bar, 1);
        mbar_init(&recv_bar, 1);
        fence_mbar_init();
        s_failed = 0;
    }
    if (warp == 4 * G_NG + 1) tmem_alloc(&tmem_base_s, (uint32_t)g.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    // Registers go where the work is: the producers' de-quantisation needs more than an even share, the two single-thread
    // warps and the idle ones far less. (Whole warpgroups execute these: warps 0-3, 4-7, 8-11 / 12-15.)
    if (warp < 4 * G_NG) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(G_REGS_PROD));
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(G_REGS_REST));
    // Under programmatic stream serialisation the next grid may start now; like this one it begins with its weight
    // stream (weights are never written) and waits for its predecessor before it touches activations or outputs.
    if (tid == 0) pdl_launch_dependents();

    // After the first wait that runs out, nobody waits any more: the block drains in bounded time.
    auto wait_ok = [&](uint64_t* bar, uint32_t parity) {
        if (mbar_try_wait(bar, parity)) return;   // the common case costs one instruction
        if (*reinterpret_cast<volatile int*>(&s_failed)) return;
        if (!mbar_wait_bounded(bar, parity, 1u << 16)) {
            *reinterpret_cast<volatile int*>(&s_failed) = 1;
            atomicOr(&g_device_status, DEV_WAIT_GEMM);
        }
    };

    if (warp < 4 * G_NG) {
        // ===== weight producers: thread = weight row of the tile, group = every G_NG-th k-step =====
        const int grp = warp >> 2, r_local = tid & 127;
        const int row = m0 + r_local;
        const int fmt = pb.w.fmt;
        const int n_out = pb.w.n_out;
        const bool row_ok = row < n_out;

        // de-quantised k-step -> operand stage (swizzled), then tell the MMA warp
        // (j = how many k-steps this group has done before; with as many groups as stages a group always fills the
        // same stage)
        auto put_stage = [&](int ks, int j, const uint4* cur) {
            const int s = G_NG == G_STAGES ? grp : ks % G_STAGES, f = G_NG == G_STAGES ? j : ks / G_STAGES;
            if (f > 0) wait_ok(&empty[s], (f - 1) & 1);
            if (G_A_TMEM) {
                tc_fence_after();   // the MMAs that read this stage are complete (their commit released it)
                // this thread's 64 inputs = 32 registers -> 32 columns of its own TMEM lane
                tc_st32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g.a_col0 + s * G_A_COLS),
                        reinterpret_cast<const uint32_t*>(cur));
                tc_fence_before();
            } else {
                unsigned char* dst = smA + s * G_A_BYTES + r_local * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + ((c ^ (r_local & 7)) << 4)) = cur[c];
                fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's async proxy
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);   // one arrival per warp of the owning group
        };

        if (fmt == FMT_F16) {
            // fp16 rows need no conversion: global -> registers one own k-step ahead -> operand stage
            const unsigned char* rowp = reinterpret_cast<const unsigned char*>(pb.w.w) + (row_ok ? (size_t)row * pb.w.k * 2 : 0);
            auto fetch = [&](int ks, uint4* dst) {
                const int k0 = kstep_of(ks) * G_BK;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    dst[c] = (row_ok && k0 + c * 8 < pb.w.k) ? ldg_nc16(rowp + (size_t)(k0 + c * 8) * 2) : make_uint4(0, 0, 0, 0);
            };
            uint4 nxt[8];
            if (grp < n_ksteps) fetch(grp, nxt);
            pdl_wait();
            int j = 0;
            for (int ks = grp; ks < n_ksteps; ks += G_NG, ++j) {
                uint4 cur[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) cur[c] = nxt[c];
                if (ks + G_NG < n_ksteps) fetch(ks + G_NG, nxt);
                put_stage(ks, j, cur);
            }
        } else {
            // One instance of the loop per weight format: ring depth, slot size and chunk counts are constants in it,
            // the ring slots are walked with wrapping counters and the row's base addresses are computed once.
            auto quant_loop = [&](auto fmt_c) {
                constexpr int F = decltype(fmt_c)::value;
                constexpr int rb = F == FMT_I8 ? 64 : 32, nq = rb / 16, epc = 16 * 64 / rb;
                constexpr int slot_bytes = rb * G_BM + (F == FMT_FP4 ? G_BM * 4 : 0);
                constexpr int depth = G_RAW_GROUP / slot_bytes > 6 ? 6 : G_RAW_GROUP / slot_bytes;   // own k-steps in flight
                static_assert(depth >= 1, "raw ring too small");
                unsigned char* ring = smRaw + grp * G_RAW_GROUP;
                const int K = pb.w.k;
                const unsigned char* wrow = reinterpret_cast<const unsigned char*>(pb.w.w) + (row_ok ? (size_t)row * K * rb / 64 : 0);
                const unsigned char* srow = reinterpret_cast<const unsigned char*>(pb.w.scale) + (row_ok && F == FMT_FP4 ? (size_t)row * K / 16 : 0);
                // chunk-major slot: chunk q of row r at q * 2048 + r * 16 (conflict-free read-back); NVFP4 block scales follow
                auto issue = [&](int ks_abs, unsigned char* slot) {
                    const int k0 = ks_abs * G_BK;
#pragma unroll
                    for (int q = 0; q < nq; ++q)
                        cp_async_16(slot + q * 2048 + r_local * 16, wrow + (size_t)ks_abs * rb + q * 16,
                                    row_ok && k0 + q * epc < K && AB_BC(ks_abs >= 0 && (size_t)ks_abs * rb + q * 16 + 16 <= (size_t)K * rb / 64));
                    if (F == FMT_FP4) cp_async_4(slot + nq * 2048 + r_local * 4, srow + (size_t)ks_abs * 4, row_ok && k0 < K);
                };
#pragma unroll
                for (int j = 0; j < depth - 1; ++j) {
                    const int ks = grp + j * G_NG;
                    if (ks < n_ksteps) issue(kstep_of(ks), ring + j * slot_bytes);
                    cp_async_commit();
                }
                pdl_wait();
                int j = 0, wslot = depth - 1, rslot = 0;
                for (int ks = grp; ks < n_ksteps; ks += G_NG, ++j) {
                    const int ks_a = ks + (depth - 1) * G_NG;
                    if (ks_a < n_ksteps) issue(kstep_of(ks_a), ring + wslot * slot_bytes);
                    if (++wslot == depth) wslot = 0;
                    cp_async_commit();
                    cp_async_wait<depth - 1>();   // all but the newest depth-1 groups have landed: k-step ks is there
                    uint4 cur[8];
                    raw_dequant(F, r_local, ring + rslot * slot_bytes, cur);
                    if (++rslot == depth) rslot = 0;
                    put_stage(ks, j, cur);
                }
            };
            if (fmt == FMT_I8) quant_loop(std::integral_constant<int, FMT_I8>());
            else quant_loop(std::integral_constant<int, FMT_FP4>());
        }

        // ===== epilogue: thread = output feature (TMEM lane); groups take turns on chunks of 32 batch rows =====
        wait_ok(&accum_bar, 0);
        tc_fence_after();
        float scale = 1.f;
        if (row_ok) scale = fmt == FMT_I8 ? reinterpret_cast<const float*>(pb.w.scale)[row] : pb.w.tscale;
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const int n_valid = min(g.n_tile, g.rows - n0);
        const int n_chunks = (n_valid + 31) / 32;
        const int epi = pb.epi;

        // finished sums of 32 batch rows of this thread's feature -> fp16, stored straight to Y: the 32 lanes of a
        // warp write 32 consecutive features (64 bytes) of one batch row per instruction
        auto emit32 = [&](int ci, const float* v) {
            const int c0 = ci * 32;
            const size_t off = (size_t)(n0 + c0) * n_out + row;
            __half* yp = pb.y + off;
            if (!row_ok) return;
            if (epi == EPI_RESID) {
                const __half* rp = pb.resid + off;
#pragma unroll
                for (int h8 = 0; h8 < 32; h8 += 8) {   // eight loads in flight, then eight stores
                    __half rs[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) rs[i] = c0 + h8 + i < n_valid ? rp[(size_t)(h8 + i) * n_out] : __half(0.f);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (c0 + h8 + i < n_valid)
                            yp[(size_t)(h8 + i) * n_out] = __hadd(rs[i], __float2half_rn(v[h8 + i] * scale));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (c0 + i < n_valid && AB_BC(row < n_out && n0 + c0 + i < g.rows)) yp[(size_t)i * n_out] = __float2half_rn(apply_epi(epi, rh(v[i] * scale)));
            }
        };

        // Preferred way out: the finished tile is laid out in shared memory as [batch row][128 features] fp16 (the
        // operand stages are idle by now) and leaves through the TMA unit in full lines; the unit clips rows and
        // features beyond the matrix. A residual tile comes in the same way and is updated in place.
        __half* stg = reinterpret_cast<__half*>(smA);
        const bool staged = pb.tma_out != 0;
        auto stage32 = [&](int ci, const float* v) {
            __half* t = stg + (size_t)ci * 32 * G_BM + r_local;
            auto body = [&](auto E) {
                constexpr int EP = decltype(E)::value;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (EP == EPI_RESID) t[i * G_BM] = __hadd(t[i * G_BM], __float2half_rn(v[i] * scale));
                    else t[i * G_BM] = __float2half_rn(apply_epi_t<EP>(rh(v[i] * scale)));
                }
            };
            switch (epi) {
                case EPI_TANH: body(std::integral_constant<int, EPI_TANH>()); break;
                case EPI_SIGMOID: body(std::integral_constant<int, EPI_SIGMOID>()); break;
                case EPI_RELU2: body(std::integral_constant<int, EPI_RELU2>()); break;
                case EPI_RESID: body(std::integral_constant<int, EPI_RESID>()); break;
                default: body(std::integral_constant<int, EPI_NONE>()); break;
            }
        };
        // A staged chunk leaves at once, while the group works on its next chunk: the group's first thread hands it
        // to the TMA unit as soon as all four warps have written their part.
        auto emit = [&](int ci, const float* v) {
            if (!staged) { emit32(ci, v); return; }
            stage32(ci, v);
            fence_proxy_async();
            group_sync(grp);
            if (r_local == 0) {
                tma_store_2d(&maps.y[pi], m0, n0 + ci * 32, stg + (size_t)ci * 32 * G_BM);
                bulk_commit();
            }
        };
        // With split K every block of a tile finishes the chunks ci = z, z + ksplit, ... of it.
        auto my_chunk = [&](int ci) { return pb.ksplit == 1 || ci % pb.ksplit == z; };
        // residual tiles on their way in
        auto fetch_resid = [&](bool wait = true) {
            if (!(staged && epi == EPI_RESID)) return;
            if (tid == 0) {
                int n_mine = 0;
                for (int ci = 0; ci < n_chunks; ++ci) n_mine += my_chunk(ci) ? 1 : 0;
                mbar_expect_tx(&resid_bar, (uint32_t)(n_mine * 32 * G_BM * 2));
                for (int ci = 0; ci < n_chunks; ++ci)
                    if (my_chunk(ci)) tma_load_2d(stg + (size_t)ci * 32 * G_BM, &maps.r[pi], m0, n0 + ci * 32, &resid_bar);
            }
            if (wait) wait_ok(&resid_bar, 0);
        };
        auto flush = [&]() {
            if (staged && r_local == 0) bulk_drain_reads();   // the shared memory must outlive the unit's reads
        };

        if (!SPLIT || pb.ksplit == 1) {
            fetch_resid();
            for (int ci = grp; ci < n_chunks; ci += G_NG) {
                uint32_t raw[32];
                tc_ld32(lane_addr + (uint32_t)(ci * 32), raw);
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                emit(ci, v);
            }
            flush();
        } else {
            // Split K: chunk ci of the tile is finished by block ci % ksplit. Every block parks the partial sums of
            // the other blocks' chunks in the scratch area; once all blocks of the tile have done so, each fetches
            // the slices of its own chunks with bulk copies (all in flight at once) into the idle operand stages and
            // sums them in slice order (deterministic), its own slice coming from TMEM. The blocks of a tile wait
            // for one another: a split grid never has more blocks than the GPU has SMs and every block holds a
            // whole SM, so all of them are resident. The wait is bounded all the same.
            const int nz = pb.ksplit;
            const int tile = pb.tile_base + m_tile * gridDim.y + blockIdx.y;
            const size_t tile_floats = (size_t)g.n_tile * G_BM;
            float* tile0 = g.partials + pb.part_base + ((size_t)(m_tile * gridDim.y + blockIdx.y) * nz) * tile_floats;
            float* mine = tile0 + (size_t)z * tile_floats;
            fetch_resid(false);
            for (int ci = grp; ci < n_chunks; ci += G_NG) {
                if (ci % nz == z) continue;
                uint32_t raw[32];
                tc_ld32(lane_addr + (uint32_t)(ci * 32), raw);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (ci * 32 + i < g.n_tile) __stcg(mine + (size_t)(ci * 32 + i) * G_BM + r_local, __uint_as_float(raw[i]));
            }
            __threadfence();
            epi_sync();
            bool ok = true;
            if (tid == 0) {
                atomicAdd(&g.counters[tile], 1u);
                uint32_t it = 0;
                while (ld_acquire_gpu(&g.counters[tile]) < (unsigned)nz) {
                    if (++it > (1u << 21)) {
                        ok = false;
                        atomicOr(&g_device_status, DEV_WAIT_GEMM);
                        break;
                    }
                }
                // the partial sums were written by ordinary stores of other blocks; the bulk copies read them
                asm volatile("fence.proxy.async;" ::: "memory");
            }
            if (staged && epi == EPI_RESID) wait_ok(&resid_bar, 0);
            unsigned char* recv = base + g.recv_off;
            const int n_own = z < n_chunks ? (n_chunks - z + nz - 1) / nz : 0;   // chunks z, z + nz, ...
            const int per_round = pb.recv_slots;   // own chunks whose slices fit the receive area at a time
            for (int k0 = 0, round = 0; k0 < n_own; k0 += per_round, ++round) {
                const int k1 = min(k0 + per_round, n_own);
                if (round > 0) epi_sync();   // everybody has read the slices of the round before
                if (tid == 0) {
                    uint32_t total = 0;
                    for (int kk = k0; kk < k1; ++kk)
                        total += (uint32_t)(nz - 1) * (uint32_t)(min(32, g.n_tile - (z + kk * nz) * 32) * G_BM * 4);
                    mbar_expect_tx(&recv_bar, ok ? total : 0u);
                    for (int kk = k0; ok && kk < k1; ++kk) {
                        const int ci = z + kk * nz;
                        const uint32_t bytes = (uint32_t)(min(32, g.n_tile - ci * 32) * G_BM * 4);
                        for (int zz = 0; zz < nz; ++zz) {
                            if (zz == z) continue;
                            bulk_g2s(recv + (size_t)((kk - k0) * (nz - 1) + (zz < z ? zz : zz - 1)) * G_CHUNK_F32,
                                     tile0 + (size_t)zz * tile_floats + (size_t)ci * 32 * G_BM, bytes, &recv_bar);
                        }
                    }
                }
                wait_ok(&recv_bar, (uint32_t)(round & 1));
                for (int kk = k0; kk < k1; ++kk) {
                    if (kk % G_NG != grp) continue;
                    const int ci = z + kk * nz;
                    uint32_t raw[32];
                    tc_ld32(lane_addr + (uint32_t)(ci * 32), raw);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                    for (int zz = 0; zz < nz; ++zz) {
                        if (zz == z) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(raw[i]);
                        } else {
                            const float* src = reinterpret_cast<const float*>(recv + (size_t)((kk - k0) * (nz - 1) + (zz < z ? zz : zz - 1)) * G_CHUNK_F32) + r_local;
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += src[i * G_BM];
                        }
                    }
                    emit(ci, v);
                }
            }
            flush();
            // the last block to leave puts the counter back to zero for the next launch
            if (tid == 0) {
                const unsigned old = atomicAdd(&g.counters[tile], 1u);
                if (old == 2u * (unsigned)nz - 1u) g.counters[tile] = 0;
            }
        }
        tc_fence_before();
    } else if (warp == 4 * G_NG) {
        // ===== activation tiles by TMA =====
        if (lane == 0) {
            const CUtensorMap* map = &maps.m[pi];
            pdl_wait();
            for (int ks = 0; ks < n_ksteps; ++ks) {
                const int s = ks % G_STAGES, f = ks / G_STAGES;
                if (f > 0) wait_ok(&empty[s], (f - 1) & 1);
                mbar_expect_tx(&full[s], (uint32_t)b_bytes);
                for (int r = 0; r < g.n_tile; r += g.tma_rows)
                    tma_load_2d(smB + s * b_bytes + r * 128, map, kstep_of(ks) * G_BK, n0 + r, &full[s]);
            }
        }
    } else if (warp == 4 * G_NG + 1) {
        // ===== MMA issue =====
        if (lane == 0) {
            // One thread feeds the tensor core, so its instruction stream is kept short: descriptors are built
            // once, a stage or a 16-input step further is an add to the (address >> 4) field.
            // An MMA is at most 256 batch rows wide and runs in steps of 64 of them: a 320-row tile is issued as
            // 192 + 128 on separate TMEM columns (160 + 160 would cost as much as 192 + 192).
            const bool two = g.n_first < g.n_tile;
            const uint32_t idesc = umma_idesc_f16(g.n_first), idesc1 = umma_idesc_f16(two ? g.n_tile - g.n_first : 16);
            const uint64_t da0 = umma_desc_sw128(smA), db0 = umma_desc_sw128(smB);
            const uint64_t a_stage = (uint64_t)(G_A_BYTES >> 4), b_stage = (uint64_t)(b_bytes >> 4);
            const uint64_t b_half = (uint64_t)((g.n_first * 128) >> 4);
            const uint32_t d1 = tmem_base + (uint32_t)g.n_first;
            // unrolled over the stages: stage index, descriptors and barrier addresses are compile-time offsets
            uint32_t parity = 0;
            for (int ks0 = 0; ks0 < n_ksteps; ks0 += G_STAGES, parity ^= 1u) {
#pragma unroll
                for (int s = 0; s < G_STAGES; ++s) {
                    const int ks = ks0 + s;
                    if (ks >= n_ksteps) break;
                    const uint64_t da = da0 + (uint64_t)s * a_stage, db = db0 + (uint64_t)s * b_stage;
                    wait_ok(&full[s], parity);
                    tc_fence_after();
                    const uint32_t acc0 = ks > 0 ? 1u : 0u;
                    // advancing 16 inputs = 32 bytes inside the swizzle row: +2 in the (address >> 4) field
                    if (G_A_TMEM) {
                        const uint32_t ta = tmem_base + (uint32_t)(g.a_col0 + s * G_A_COLS);
#pragma unroll
                        for (int k4 = 0; k4 < G_BK / 16; ++k4) {   // 16 inputs = 8 columns of the weight stage
                            const uint32_t acc = k4 ? 1u : acc0;
                            tc_mma_f16_ts(tmem_base, ta + (uint32_t)(8 * k4), db + (uint64_t)(2 * k4), idesc, acc);
                            if (two) tc_mma_f16_ts(d1, ta + (uint32_t)(8 * k4), db + b_half + (uint64_t)(2 * k4), idesc1, acc);
                        }
                    } else {
                        tc_mma_f16(tmem_base, da, db, idesc, acc0);
                        if (two) tc_mma_f16(d1, da, db + b_half, idesc1, acc0);
#pragma unroll
                        for (int k4 = 1; k4 < G_BK / 16; ++k4) {
                            tc_mma_f16(tmem_base, da + (uint64_t)(2 * k4), db + (uint64_t)(2 * k4), idesc, 1u);
                            if (two) tc_mma_f16(d1, da + (uint64_t)(2 * k4), db + b_half + (uint64_t)(2 * k4), idesc1, 1u);
                        }
                    }
                    tc_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
                }
            }
            tc_commit(&accum_bar);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 4 * G_NG + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)g.tmem_cols);
    }
}

// In-register de-quantisation exactly as the product kernels do it, written out as fp32.
__global__ void dequant_kernel(ab_mat m, float* __restrict__ out) {
    const size_t total = (size_t)m.n_out * m.k;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(idx / m.k), col = (int)(idx % m.k);
        float v;
        if (m.fmt == FMT_I8) {
            v = (float)reinterpret_cast<const signed char*>(m.w)[idx] * reinterpret_cast<const float*>(m.scale)[row];
            if (m.col_scale) v *= m.col_scale[col];
        } else if (m.fmt == FMT_FP4) {
            const uint32_t byte = reinterpret_cast<const unsigned char*>(m.w)[idx >> 1];
            const float2 pr = __half22float2(e2m1x2_to_half2(byte));
            const float q = (col & 1) ? pr.y : pr.x;
            const float sb = e4m3_to_float(reinterpret_cast<const unsigned char*>(m.scale)[(size_t)row * (m.k / 16) + col / 16]);
            v = (q * sb) * m.tscale;
        } else {
            v = __half2float(reinterpret_cast<const __half*>(m.w)[idx]);
        }
        out[idx] = v;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        AB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres));
        AB_CHECK_ARG(ptr && qres == cudaDriverEntryPointSuccess, "gemm: cuTensorMapEncodeTiled is not available");
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    *out = fn;
    return OK;
}

}  // namespace

int check_mat(const ab_mat& m, const char* what) {
    AB_CHECK_ARG(m.fmt == FMT_F16 || m.fmt == FMT_I8 || m.fmt == FMT_FP4, "%s: unknown weight format %d", what, m.fmt);
    AB_CHECK_ARG(m.w && m.n_out > 0 && m.k > 0, "%s: empty matrix", what);
    AB_CHECK_ARG(m.fmt == FMT_F16 || m.scale, "%s: scales missing", what);
    AB_CHECK_ARG(m.fmt != FMT_FP4 || m.k % 32 == 0, "%s: NVFP4 needs k %% 32 == 0", what);
    return OK;
}

namespace {

struct GroupShape {
    int n_tile, n_first, tma_rows, tmem_cols, n_tiles_y;
    int ksplit[G_MAX_OPS];
    int grid_x;
    long long part_floats;
    int n_split_tiles;
};

// Shared memory of a block (beyond the 1 KB alignment slack): operand stages + raw weight rings.
size_t block_smem(int n_tile) {
    if (!G_A_TMEM) return (size_t)G_STAGES * (G_A_BYTES + (size_t)n_tile * 128) + G_RAW_BYTES;
    // activation stages + raw rings, and some more for the epilogue (output staging, split-K slices), up to 224 KB
    const size_t need = (size_t)G_STAGES * n_tile * 128 + G_RAW_BYTES, want = need + 48 * 1024;
    return want < 224 * 1024 ? want : (need > 224 * 1024 ? need : 224 * 1024);
}
// Split K: how many of its own chunks a block can fetch the other blocks' partial sums for at a time. They land
// in the operand stages behind the output staging area.
int split_recv_slots(int n_tile, int ks) {
    const int n_chunks = (n_tile + 31) / 32;
    const size_t stage_bytes = (size_t)n_chunks * 32 * G_BM * 2;
    const size_t avail = block_smem(n_tile) - stage_bytes;
    const int own_max = (n_chunks + ks - 1) / ks;
    const int fit = (int)(avail / ((size_t)(ks - 1) * G_CHUNK_F32));
    return fit < own_max ? fit : own_max;
}

GroupShape group_shape(const GemmOp* ops, int n, int rows, int n_sm) {
    GroupShape gs = {};
    if (rows <= 256) { gs.n_tile = (rows + 15) & ~15; gs.n_first = gs.tma_rows = gs.n_tile; }
    else if (rows <= 320) { gs.n_tile = (rows + 31) & ~31; gs.n_first = 192; gs.tma_rows = gs.n_tile % 64 ? 32 : 64; }
    else { gs.n_tile = gs.n_first = gs.tma_rows = 256; }
    gs.tmem_cols = 32;
    const int a_cols = G_A_TMEM ? G_STAGES * G_A_COLS : 0;   // weight stages behind the accumulators
    while (gs.tmem_cols < ((gs.n_tile + 31) & ~31) + a_cols) gs.tmem_cols *= 2;
    gs.n_tiles_y = (rows + gs.n_tile - 1) / gs.n_tile;
    int base_ctas = 0, slow_ctas = 0;
    for (int i = 0; i < n; ++i) {
        const int c = (ops[i].w.n_out + G_BM - 1) / G_BM * gs.n_tiles_y;
        base_ctas += c;
        if (ops[i].w.fmt == FMT_F16 && ops[i].w.k >= 32 * G_BK) slow_ctas += c;
    }
    for (int i = 0; i < n; ++i) {
        const int ksteps = (ops[i].w.k + G_BK - 1) / G_BK;
        int ks = 1;
        if (base_ctas > 0 && base_ctas < (100 * n_sm) / 148 && ksteps >= 32) {   // too few tiles to fill the GPU: split the long K loops
            ks = n_sm / base_ctas;
            if (ks > 8) ks = 8;
            if (ks > ksteps / 8) ks = ksteps / 8;
            if (ks < 1) ks = 1;
        } else if (base_ctas < n_sm && slow_ctas > 0 && ops[i].w.fmt == FMT_F16 && ksteps >= 32) {
            // A nearly full grid whose fp16 products (twice to four times the bytes per k-step of the quantised
            // ones, fetched only two k-steps ahead) would finish last: the idle SMs take slices of their K loops.
            ks = 1 + (n_sm - base_ctas) / slow_ctas;
            if (ks > 8) ks = 8;
            if (ks > ksteps / 8) ks = ksteps / 8;
            if (ks < 1) ks = 1;
        }
        while (ks > 1 && split_recv_slots(gs.n_tile, ks) < 1) --ks;   // the slices of one chunk must fit the receive area
        gs.ksplit[i] = ks;
        const int m_tiles = (ops[i].w.n_out + G_BM - 1) / G_BM;
        gs.grid_x += m_tiles * ks;
        if (ks > 1) {
            gs.part_floats += (long long)m_tiles * gs.n_tiles_y * ks * gs.n_tile * G_BM;
            gs.n_split_tiles += m_tiles * gs.n_tiles_y;
        }
    }
    return gs;
}

}  // namespace

// SMs of the current device (148 on B200); the split-K decisions depend on it.
int current_sm_count() {
    static PerDeviceOnce once;
    const DeviceProps* dp = nullptr;
    if (once.run(&dp, [](DeviceProps&) -> int { return OK; }) != OK || !dp || dp->n_sm <= 0) return 148;
    return dp->n_sm;
}

size_t gemm_group_scratch_bytes(const GemmOp* ops, int n, int rows) {
    if (!ops || n < 1 || n > G_MAX_OPS || rows <= 0) return 0;
    for (int i = 0; i < n; ++i)
        if (ops[i].w.n_out <= 0 || ops[i].w.k <= 0) return 0;
    const GroupShape gs = group_shape(ops, n, rows, current_sm_count());
    return (size_t)G_COUNTERS * 4 + (size_t)gs.part_floats * 4 + 256;
}
size_t gemm_scratch_bytes(const ab_mat& m, int rows) {
    GemmOp op = {};
    op.w = m;
    return gemm_group_scratch_bytes(&op, 1, rows);
}

int gemm_group_launch(const GemmOp* ops, int n, int rows, void* scratch, cudaStream_t stream, bool pdl) {
    AB_CHECK_ARG(ops && n >= 1 && n <= G_MAX_OPS && rows > 0, "gemm: bad group (n=%d rows=%d)", n, rows);
    for (int i = 0; i < n; ++i) {   // shapes first: the grid arithmetic below divides by tile counts
        const int s = check_mat(ops[i].w, "gemm");
        if (s != OK) return s;
    }
    const int n_sm = current_sm_count();
    GroupShape gs = group_shape(ops, n, rows, n_sm);
    AB_CHECK_ARG(gs.n_split_tiles <= G_COUNTERS, "gemm: too many split-K tiles");
    if (gs.n_split_tiles > 0 && gs.grid_x * gs.n_tiles_y > n_sm) {
        // the blocks of a split tile wait for one another, so all of them must be resident (one block per SM); a
        // split grid that would not be is launched without the split instead
        GemmOp unsplit[G_MAX_OPS];
        for (int i = 0; i < n; ++i) unsplit[i] = ops[i];
        gs = group_shape(unsplit, n, rows, 0);   // no SMs to fill: every product keeps its whole K loop
    }
    AB_CHECK_ARG(gs.part_floats == 0 || (scratch && ((uintptr_t)scratch & 15) == 0), "gemm: split-K needs a 16-byte aligned scratch area");
    EncodeTiledFn encode;
    int st = get_encode_fn(&encode);
    if (st != OK) return st;

    GemmGroup g = {};
    GemmMaps maps;
    g.n_prob = n; g.rows = rows; g.n_tile = gs.n_tile; g.n_first = gs.n_first; g.tma_rows = gs.tma_rows; g.tmem_cols = gs.tmem_cols;
    g.a_col0 = (gs.n_tile + 31) & ~31;
    g.recv_off = (gs.n_tile + 31) / 32 * 32 * G_BM * 2;
    g.counters = reinterpret_cast<unsigned*>(scratch);
    g.partials = scratch ? reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + (size_t)G_COUNTERS * 4) : nullptr;
    int cta = 0, tile = 0;
    long long part = 0;
    for (int i = 0; i < n; ++i) {
        const GemmOp& op = ops[i];
        const ab_mat& m = op.w;
        st = check_mat(m, "gemm");
        if (st != OK) return st;
        AB_CHECK_ARG(op.x && op.y, "gemm: null activation pointer");
        AB_CHECK_ARG(op.epi >= EPI_NONE && op.epi <= EPI_RESID && (op.epi != EPI_RESID || op.resid), "gemm: bad epilogue");
        AB_CHECK_ARG(m.col_scale == nullptr, "gemm: per-input-column scales are a batch-1 feature");
        AB_CHECK_ARG(m.k % 16 == 0 && ((uintptr_t)op.x & 15) == 0 && ((uintptr_t)m.w & 15) == 0, "gemm: k %% 16 and 16-byte alignment needed");
        AB_CHECK_ARG(m.fmt != FMT_FP4 || (m.k % 64 == 0 && ((uintptr_t)m.scale & 3) == 0), "gemm: NVFP4 needs k %% 64 == 0");
        GemmProb& pb = g.pr[i];
        pb.w = m; pb.resid = op.resid; pb.y = op.y; pb.epi = op.epi;
        pb.cta_base = cta; pb.ksplit = gs.ksplit[i]; pb.tile_base = tile; pb.part_base = part;
        pb.recv_slots = pb.ksplit > 1 ? split_recv_slots(gs.n_tile, pb.ksplit) : 0;
        const int m_tiles = (m.n_out + G_BM - 1) / G_BM;
        cta += m_tiles * pb.ksplit;
        if (pb.ksplit > 1) {
            tile += m_tiles * gs.n_tiles_y;
            part += (long long)m_tiles * gs.n_tiles_y * pb.ksplit * gs.n_tile * G_BM;
        }
        const cuuint64_t gdim[2] = {(cuuint64_t)m.k, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)m.k * 2};
        const cuuint32_t box[2] = {(cuuint32_t)G_BK, (cuuint32_t)gs.tma_rows};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = encode(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(op.x), gdim, gstride, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            set_error("gemm: cuTensorMapEncodeTiled failed with %d (rows=%d k=%d)", (int)cr, rows, m.k);
            return ERR_CUDA;
        }
        // output / residual tiles through the TMA unit when the row pitch and the pointers allow it
        pb.tma_out = (m.n_out % 8 == 0 && m.n_out >= G_BM && ((uintptr_t)op.y & 15) == 0 &&
                      (op.epi != EPI_RESID || ((uintptr_t)op.resid & 15) == 0)) ? 1 : 0;
        maps.y[i] = maps.m[i];
        maps.r[i] = maps.m[i];
        if (pb.tma_out) {
            const cuuint64_t odim[2] = {(cuuint64_t)m.n_out, (cuuint64_t)rows};
            const cuuint64_t ostride[1] = {(cuuint64_t)m.n_out * 2};
            const cuuint32_t obox[2] = {(cuuint32_t)G_BM, 32};
            CUresult c2 = encode(&maps.y[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, op.y, odim, ostride, obox, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (c2 == CUDA_SUCCESS && op.epi == EPI_RESID)
                c2 = encode(&maps.r[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(op.resid), odim, ostride, obox,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (c2 != CUDA_SUCCESS) {
                set_error("gemm: cuTensorMapEncodeTiled (output) failed with %d (rows=%d n_out=%d)", (int)c2, rows, m.n_out);
                return ERR_CUDA;
            }
        }
    }
    for (int i = n; i < G_MAX_OPS; ++i) { maps.m[i] = maps.m[0]; maps.y[i] = maps.m[0]; maps.r[i] = maps.m[0]; }

    const size_t smem = 1024 + block_smem(gs.n_tile);
    {
        static PerDeviceOnce once;
        const int s = once.run(nullptr, [](DeviceProps& d) -> int {
            // the largest dynamic size the device allows (the kernels' static shared memory is under 1 KB)
            AB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d.smem_optin - 1024));
            AB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d.smem_optin - 1024));
            return OK;
        });
        if (s != OK) return s;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(gs.grid_x, gs.n_tiles_y);
    cfg.blockDim = dim3(GT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    if (gs.n_split_tiles > 0) AB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true>, maps, g));
    else AB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false>, maps, g));
    return OK;
}

int gemm_launch(const ab_mat& m, int rows, const __half* x, __half* y, int epi, const __half* resid, void* scratch,
                cudaStream_t stream, bool pdl) {
    GemmOp op = {};
    op.w = m; op.x = x; op.y = y; op.epi = epi; op.resid = resid;
    return gemm_group_launch(&op, 1, rows, scratch, stream, pdl);
}

int dequant_launch(const ab_mat& m, float* out, cudaStream_t stream) {
    int s = check_mat(m, "dequant");
    if (s != OK) return s;
    AB_CHECK_ARG(out, "dequant: null output");
    dequant_kernel<<<1184, 256, 0, stream>>>(m, out);
    AB_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace ab

// ---------------------------------------------------------------------------------------------
// Batched product with built-in scratch: the split-K counters and partial tiles live in a fixed array of this
// module instead of a caller-supplied buffer, so the call neither takes nor makes a device allocation.
// ---------------------------------------------------------------------------------------------
namespace ab {
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[AB_GEMM_STATIC_SCRATCH_BYTES];

constexpr int STATIC_MAX_DEVICES = AB_MAX_DEVICES;
std::mutex g_static_mu;
void* g_static_ptrs[STATIC_MAX_DEVICES] = {};

// Address of the array on the current device, looked up once per device (under a lock: the first calls of two host
// threads may coincide); the counters are cleared on `stream` when a device is first used (the kernels need them at
// zero and leave them at zero).
int static_scratch(void** out, cudaStream_t stream) {
    int dev = 0;
    AB_CUDA(cudaGetDevice(&dev));
    AB_CHECK_ARG(dev >= 0 && dev < STATIC_MAX_DEVICES, "ab_gemm_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptrs[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            set_error("ab_gemm_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return ERR_CUDA;
        }
        AB_CUDA(cudaMemsetAsync(ptr, 0, (size_t)G_COUNTERS * 4, stream));
        g_static_ptrs[dev] = ptr;
    }
    *out = g_static_ptrs[dev];
    return OK;
}

}  // namespace

// Puts the arrival counters of the built-in scratch area of the current device back to zero (nothing to do if the
// device has not used it yet). The kernels leave them at zero themselves, except when a bounded wait gave up or a
// launch was aborted half-way; then every later split-K product through ab_gemm_static would read stale counts.
int static_scratch_reset(cudaStream_t stream) {
    int dev = 0;
    AB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return OK;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptrs[dev]) AB_CUDA(cudaMemsetAsync(g_static_ptrs[dev], 0, (size_t)G_COUNTERS * 4, stream));
    return OK;
}

namespace {
}  // namespace
}  // namespace ab

extern "C" int ab_gemm_static(const ab_mat* m, int rows, const void* x, void* y, int epi, const void* resid, void* stream) {
    using namespace ab;
    AB_CHECK_ARG(m && x && y, "ab_gemm_static: null pointer");
    AB_CHECK_ARG(epi >= EPI_NONE && epi <= EPI_RESID && (epi != EPI_RESID || resid), "ab_gemm_static: bad epilogue");
    AB_CHECK_ARG(rows > 0, "ab_gemm_static: rows must be positive");
    int st = check_mat(*m, "ab_gemm_static");
    if (st != OK) return st;
    const size_t need = gemm_scratch_bytes(*m, rows);
    if (need > (size_t)AB_GEMM_STATIC_SCRATCH_BYTES) {
        set_error("ab_gemm_static: this product needs %zu bytes of split-K scratch, the built-in area holds %zu "
                  "(n_out=%d k=%d rows=%d); use ab_gemm with a caller-supplied scratch buffer",
                  need, (size_t)AB_GEMM_STATIC_SCRATCH_BYTES, m->n_out, m->k, rows);
        return ERR_TOO_LARGE;
    }
    void* scratch = nullptr;
    st = static_scratch(&scratch, (cudaStream_t)stream);
    if (st != OK) return st;
    return gemm_launch(*m, rows, (const __half*)x, (__half*)y, epi, (const __half*)resid, scratch, (cudaStream_t)stream);
}

extern "C" int ab_gemm_static_reset(void* stream) { return ab::static_scratch_reset((cudaStream_t)stream); }

// Test hook: reads (write == 0) or overwrites (write != 0) arrival counter `index` of the built-in scratch area of the
// current device, through `value_host`. Synchronises the device.
extern "C" int ab_gemm_static_debug_counter(int index, int write, uint32_t* value_host) {
    using namespace ab;
    AB_CHECK_ARG(value_host && index >= 0 && index < G_COUNTERS, "ab_gemm_static_debug_counter: bad argument");
    void* scratch = nullptr;
    const int st = static_scratch(&scratch, nullptr);
    if (st != OK) return st;
    AB_CUDA(cudaDeviceSynchronize());
    uint32_t* p = reinterpret_cast<uint32_t*>(scratch) + index;
    if (write) AB_CUDA(cudaMemcpy(p, value_host, 4, cudaMemcpyHostToDevice));
    else AB_CUDA(cudaMemcpy(value_host, p, 4, cudaMemcpyDeviceToHost));
    return OK;
}

