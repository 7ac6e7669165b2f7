// Batched matrix products of the RWKV-7 batch path on the 5th-generation tensor cores (tcgen05 / TMEM),
// and the de-quantisation dump.
//
// Replaces the `[B,T,D] @ W` call sites of reference/rwkv7.py:283-288, :293, :300 (time-mix), :322-323
// (channel-mix) and :220 (vocabulary head) with weight-only int8 / NVFP4 / fp16 weights.
//
//   D[128 weight rows, N batch rows] (fp32, TMEM) += A[128, 64] (weights, fp16) * B[N, 64]^T (activations, fp16)
//
// The weights are the M side of the MMA so that every weight byte is read from HBM exactly once per
// N tile; the batch (up to 320 rows per block: two MMAs of N = 160) is the N side.
//   warps 0-3 : read this block's 128 weight rows straight from global memory (64 inputs per row and
//               k-step), de-quantise in registers (int8 -> fp16 exactly; e2m1 x e4m3 block scale -> fp16
//               exactly) and store them K-major with the 128-byte swizzle the MMA expects; afterwards
//               they run the epilogue: tcgen05.ld of their 32 TMEM lanes, row / tensor scale, activation
//               or residual, fp16 stores that are contiguous along the output features;
//   warp 4    : one thread issues the TMA loads of the activation tile (tensor map over X, 128B swizzle);
//   warp 5    : allocates TMEM; one thread issues tcgen05.mma (kind::f16) and commits to mbarriers.
// Three-stage ring, all mbarrier waits bounded (status word on expiry), TMEM freed on every path.
#include <cuda.h>

#include "gemm.cuh"
#include "gemv.cuh"

namespace ab {

namespace {

constexpr int GT = 192;          // threads per block
constexpr int G_STAGES = 3;
constexpr int G_BM = 128;        // weight rows per block
constexpr int G_BK = 64;         // inputs per k-step (128 bytes of fp16 = one swizzle row)
constexpr int G_A_BYTES = G_BM * G_BK * 2;

struct GemmParams {
    ab_mat w;
    const __half* resid;
    __half* y;
    int rows;       // batch rows (B*T)
    int n_tile;     // batch rows per block tile
    int n_inst;     // MMAs per k-substep (1, or 2 when n_tile > 256)
    int epi;
    int tmem_cols;
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
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

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

// De-quantise 64 inputs of one weight row into eight 16-byte chunks of fp16 (chunk c = inputs 8c..8c+7).
__device__ __forceinline__ void dequant_row64(const ab_mat& w, int row, int k0, uint4* out) {
    const int K = w.k;
    if (row >= w.n_out) {
#pragma unroll
        for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
        return;
    }
    if (w.fmt == FMT_I8) {
        const signed char* src = reinterpret_cast<const signed char*>(w.w) + (size_t)row * K + k0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (k0 + q * 16 < K) raw = __ldg(reinterpret_cast<const uint4*>(src + q * 16));
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t h[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int b0 = (int)(signed char)(words[e] & 0xff), b1 = (int)(signed char)((words[e] >> 8) & 0xff);
                const int b2 = (int)(signed char)((words[e] >> 16) & 0xff), b3 = (int)(signed char)(words[e] >> 24);
                h[2 * e] = pack_h2((float)b0, (float)b1);
                h[2 * e + 1] = pack_h2((float)b2, (float)b3);
            }
            out[2 * q] = make_uint4(h[0], h[1], h[2], h[3]);
            out[2 * q + 1] = make_uint4(h[4], h[5], h[6], h[7]);
        }
    } else if (w.fmt == FMT_F16) {
        const __half* src = reinterpret_cast<const __half*>(w.w) + (size_t)row * K + k0;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            out[c] = (k0 + c * 8 < K) ? __ldg(reinterpret_cast<const uint4*>(src + c * 8)) : make_uint4(0, 0, 0, 0);
    } else {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(w.w) + ((size_t)row * K + k0) / 2;
        const unsigned char* ssrc = reinterpret_cast<const unsigned char*>(w.scale) + ((size_t)row * K + k0) / 16;
        const bool in = k0 < K;   // NVFP4 matrices have K % 64 == 0
        const uint4 r0 = in ? __ldg(reinterpret_cast<const uint4*>(src)) : make_uint4(0, 0, 0, 0);
        const uint4 r1 = in ? __ldg(reinterpret_cast<const uint4*>(src + 16)) : make_uint4(0, 0, 0, 0);
        const uint32_t sc4 = in ? __ldg(reinterpret_cast<const uint32_t*>(ssrc)) : 0u;
        const uint32_t words[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {   // chunk c: 8 inputs = 4 bytes; scale block = c / 2
            const __half2 s2 = e4m3x2_to_half2((sc4 >> (8 * (c >> 1))) & 0xffu);
            const __half2 sc = __half2half2(__low2half(s2));
            uint32_t h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 v = __hmul2(e2m1x2_to_half2((words[c] >> (8 * e)) & 0xffu), sc);   // exact in fp16
                h[e] = *reinterpret_cast<const uint32_t*>(&v);
            }
            out[c] = make_uint4(h[0], h[1], h[2], h[3]);
        }
    }
}

__global__ void __launch_bounds__(GT, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                        const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(1024) unsigned char gsm[];
    __shared__ uint64_t full_a[G_STAGES], full_b[G_STAGES], empty[G_STAGES], accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
    const int b_bytes = p.n_tile * 128;
    unsigned char* smA = base;                                  // G_STAGES x 16 KB
    unsigned char* smB = base + G_STAGES * G_A_BYTES;           // G_STAGES x n_tile x 128 B
    const int n_inst_cols = p.n_tile / p.n_inst;
    const int m0 = blockIdx.x * G_BM;
    const int n0 = blockIdx.y * p.n_tile;
    const int n_ksteps = (p.w.k + G_BK - 1) / G_BK;

    if (tid == 0) {
        for (int s = 0; s < G_STAGES; ++s) {
            mbar_init(&full_a[s], 128);
            mbar_init(&full_b[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&accum_bar, 1);
        fence_mbar_init();
        s_failed = 0;
    }
    if (warp == 5) tmem_alloc(&tmem_base_s, (uint32_t)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // After the first wait that runs out, nobody waits any more: the block drains in bounded time.
    auto wait_ok = [&](uint64_t* bar, uint32_t parity) {
        if (*reinterpret_cast<volatile int*>(&s_failed)) return;
        if (!mbar_wait_bounded(bar, parity, 1u << 16)) {
            *reinterpret_cast<volatile int*>(&s_failed) = 1;
            atomicOr(&g_device_status, DEV_WAIT_GEMM);
        }
    };
    if (warp < 4) {
        // ===== weight producers: thread = weight row of the tile =====
        const int row = m0 + tid;
        uint4 cur[8];
        dequant_row64(p.w, row, 0, cur);
        for (int ks = 0; ks < n_ksteps; ++ks) {
            const int s = ks % G_STAGES, f = ks / G_STAGES;
            uint4 nxt[8];
            if (ks + 1 < n_ksteps) dequant_row64(p.w, row, (ks + 1) * G_BK, nxt);   // next k-step's loads in flight
            if (f > 0) wait_ok(&empty[s], (f - 1) & 1);
            unsigned char* dst = smA + s * G_A_BYTES + tid * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + ((c ^ (tid & 7)) << 4)) = cur[c];
            fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's async proxy
            mbar_arrive(&full_a[s]);
#pragma unroll
            for (int c = 0; c < 8; ++c) cur[c] = nxt[c];
        }
        // ===== epilogue: thread = output feature (TMEM lane), loop over batch columns =====
        wait_ok(&accum_bar, 0);
        tc_fence_after();
        const bool row_ok = row < p.w.n_out;
        float scale = 1.f;
        if (row_ok) scale = p.w.fmt == FMT_I8 ? reinterpret_cast<const float*>(p.w.scale)[row] : p.w.tscale;
        for (int c0 = 0; c0 < p.n_tile; c0 += 16) {
            if (n0 + c0 >= p.rows) break;   // warp-uniform
            uint32_t v[16];
            tc_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
            if (row_ok) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int b = n0 + c0 + i;
                    if (b < p.rows) {
                        float o = rh(__uint_as_float(v[i]) * scale);
                        switch (p.epi) {
                            case EPI_TANH: o = tanhf(o); break;
                            case EPI_SIGMOID: o = sigmoidf_(o); break;
                            case EPI_RELU2: o = fmaxf(o, 0.f); o = o * o; break;
                            case EPI_RESID: o = __half2float(p.resid[(size_t)b * p.w.n_out + row]) + o; break;
                            default: break;
                        }
                        p.y[(size_t)b * p.w.n_out + row] = __float2half_rn(o);
                    }
                }
            }
        }
        tc_fence_before();
    } else if (warp == 4) {
        // ===== activation tiles by TMA =====
        if (lane == 0) {
            for (int ks = 0; ks < n_ksteps; ++ks) {
                const int s = ks % G_STAGES, f = ks / G_STAGES;
                if (f > 0) wait_ok(&empty[s], (f - 1) & 1);
                mbar_expect_tx(&full_b[s], (uint32_t)b_bytes);
                for (int j = 0; j < p.n_inst; ++j)
                    tma_load_2d(smB + s * b_bytes + j * n_inst_cols * 128, &tmap_x, ks * G_BK, n0 + j * n_inst_cols, &full_b[s]);
            }
        }
    } else {
        // ===== MMA issue =====
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(n_inst_cols);
            for (int ks = 0; ks < n_ksteps; ++ks) {
                const int s = ks % G_STAGES, f = ks / G_STAGES;
                wait_ok(&full_a[s], f & 1);
                wait_ok(&full_b[s], f & 1);
                tc_fence_after();
                const uint64_t da = umma_desc_sw128(smA + s * G_A_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < G_BK / 16; ++k4)
                    for (int j = 0; j < p.n_inst; ++j) {
                        const uint64_t db = umma_desc_sw128(smB + s * b_bytes + j * n_inst_cols * 128);
                        // advancing 16 inputs = 32 bytes inside the swizzle row: +2 in the (address >> 4) field
                        tc_mma_f16(tmem_base + (uint32_t)(j * n_inst_cols), da + (uint64_t)(2 * k4), db + (uint64_t)(2 * k4),
                                   idesc, (ks > 0 || k4 > 0) ? 1u : 0u);
                    }
                tc_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
            }
            tc_commit(&accum_bar);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
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

size_t gemm_scratch_bytes(const ab_mat&, int) { return 256; }

int gemm_launch(const ab_mat& m, int rows, const __half* x, __half* y, int epi, const __half* resid, void*,
                cudaStream_t stream) {
    int st = check_mat(m, "gemm");
    if (st != OK) return st;
    AB_CHECK_ARG(rows > 0 && x && y, "gemm: bad argument");
    AB_CHECK_ARG(m.col_scale == nullptr, "gemm: per-input-column scales are a batch-1 feature");
    AB_CHECK_ARG(m.k % 16 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)m.w & 15) == 0, "gemm: k %% 16 and 16-byte alignment needed");
    AB_CHECK_ARG(m.fmt != FMT_FP4 || (m.k % 64 == 0 && ((uintptr_t)m.scale & 3) == 0), "gemm: NVFP4 needs k %% 64 == 0");

    GemmParams p = {};
    p.w = m; p.resid = resid; p.y = y; p.rows = rows; p.epi = epi;
    if (rows <= 256) { p.n_tile = (rows + 15) & ~15; p.n_inst = 1; }
    else if (rows <= 320) { p.n_tile = (rows + 31) & ~31; p.n_inst = 2; }
    else { p.n_tile = 256; p.n_inst = 1; }
    p.tmem_cols = 32;
    while (p.tmem_cols < p.n_tile) p.tmem_cols *= 2;
    const int n_inst_cols = p.n_tile / p.n_inst;

    EncodeTiledFn encode;
    st = get_encode_fn(&encode);
    if (st != OK) return st;
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)m.k, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)m.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)G_BK, (cuuint32_t)n_inst_cols};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_error("gemm: cuTensorMapEncodeTiled failed with %d (rows=%d k=%d)", (int)cr, rows, m.k);
        return ERR_CUDA;
    }

    const size_t smem = 1024 + (size_t)G_STAGES * (G_A_BYTES + (size_t)p.n_tile * 128);
    static size_t smem_set = 0;
    if (smem > smem_set) {
        AB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        smem_set = smem;
    }
    const dim3 grid((m.n_out + G_BM - 1) / G_BM, (rows + p.n_tile - 1) / p.n_tile);
    gemm_tc_kernel<<<grid, GT, smem, stream>>>(tmap, p);
    AB_CUDA(cudaGetLastError());
    return OK;
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
