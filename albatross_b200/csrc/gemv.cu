// Batch-1 weight-streaming matrix-vector product for sm_100a, one launch per group of matrices.
//
// Replaces the reference's fp16 `x @ W` GEMV call sites at batch 1
// (reference/rwkv7.py:230-235, :240, :250 time-mix; :308-309 channel-mix; :156 vocabulary head).
// The device code lives in gemv_body.cuh; this file holds the stand-alone kernel and its launcher.
#include "gemv_body.cuh"

namespace ab {

namespace {

struct GemvLaunchShape {
    int Kn, with_dx, Kq;
};
__host__ __device__ inline GemvLaunchShape gemv_shape(const GemvParams& p) {
    GemvLaunchShape sh = {0, 0, 0};
    if (p.emb || p.x) sh.Kn = p.K;
    for (int s = 0; s < p.nseg; ++s) {
        if (p.seg[s].mix) sh.with_dx = 1;
        if (p.seg[s].K > sh.Kq) sh.Kq = p.seg[s].K;
    }
    return sh;
}

__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_stream_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const GemvLaunchShape sh = gemv_shape(p);
    const GemvLayout L = gemv_layout(p.stages, sh.Kn, sh.with_dx, sh.Kq);
    const GemvSmem m = gemv_smem(smem, L, p.stages);
    if (tid == 0) gemv_init_barriers(m);
    __syncthreads();

    if (warp == GEMV_WARPS) {
        // weights do not depend on the previous kernel: the producer does not wait for it
        if (lane < GEMV_WARPS) {
            ProducerState ps = {0, 0, 0, false};
            gemv_produce(p, m, ps, lane, blockIdx.x, gridDim.x, policy_evict_first());
        }
        return;
    }
    if (p.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }
    ConsumerState cs = {0, 0, false};
    gemv_consume(p, m, cs, tid, blockIdx.x, gridDim.x);
}

}  // namespace

int gemv_check(GemvParams& p) {
    AB_CHECK_ARG(p.nseg >= 1 && p.nseg <= GEMV_MAX_SEG, "gemv: nseg %d out of range", p.nseg);
    const bool shared_in = p.emb || p.x;
    AB_CHECK_ARG(!shared_in || (p.K >= 16 && p.K % 16 == 0 && p.K <= 32768), "gemv: K=%d must be a multiple of 16 in [16, 32768]", p.K);
    for (int s = 0; s < p.nseg; ++s) {
        GemvSeg& g = p.seg[s];
        if (!g.x && g.K == 0) g.K = p.K;
        AB_CHECK_ARG(g.x || shared_in, "gemv: segment %d has no input", s);
        AB_CHECK_ARG(g.x || g.K == p.K, "gemv: segment %d: K differs from the shared input", s);
        AB_CHECK_ARG(!(g.x && g.mix), "gemv: segment %d: token-shift lerp needs the shared input", s);
        AB_CHECK_ARG(g.K >= 16 && g.K % 16 == 0 && g.K <= 32768, "gemv: segment %d: K=%d must be a multiple of 16 in [16, 32768]", s, g.K);
        AB_CHECK_ARG(g.w && g.out && g.n_rows > 0, "gemv: segment %d has a null pointer or no rows", s);
        AB_CHECK_ARG(((uintptr_t)g.w & 15) == 0, "gemv: segment %d weights not 16-byte aligned", s);
        AB_CHECK_ARG(!g.x || ((uintptr_t)g.x & 15) == 0, "gemv: segment %d input not 16-byte aligned", s);
        AB_CHECK_ARG(g.fmt == FMT_F16 || g.scale, "gemv: segment %d needs scales", s);
        AB_CHECK_ARG(g.fmt != FMT_FP4 || (((uintptr_t)g.scale & 15) == 0 && g.K % 256 == 0),
                     "gemv: segment %d: NVFP4 needs 16-byte aligned block scales and K %% 256 == 0", s);
        AB_CHECK_ARG(g.epi != EPI_RESID || g.resid, "gemv: segment %d residual missing", s);
        AB_CHECK_ARG(!g.mix || p.x_prev, "gemv: segment %d: token-shift state missing", s);
    }
    return OK;
}

int gemv_groups(const GemvParams& p) {
    int groups = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const int R = gemv_rows_per_group(p.seg[s].fmt, p.seg[s].K);
        groups += (p.seg[s].n_rows + R - 1) / R;
    }
    return groups;
}

int gemv_launch(const GemvParams& p_in, cudaStream_t stream) {
    GemvParams p = p_in;
    int st = gemv_check(p);
    if (st != OK) return st;
    if (p.stages <= 0) p.stages = 2;
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
    const GemvLaunchShape sh = gemv_shape(p);
    size_t smem = gemv_layout(p.stages, sh.Kn, sh.with_dx, sh.Kq).total;
    while (smem > max_smem && p.stages > 1) {
        --p.stages;
        smem = gemv_layout(p.stages, sh.Kn, sh.with_dx, sh.Kq).total;
    }
    AB_CHECK_ARG(smem <= max_smem, "gemv: K=%d needs %zu bytes of shared memory", sh.Kq, smem);
    const int grid = max(1, min(n_sm, gemv_groups(p)));

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
