// Batch-1 weight-streaming matrix-vector product for sm_100a, one launch per group of matrices.
//
// Replaces the reference's fp16 `x @ W` GEMV call sites at batch 1
// (reference/rwkv7.py:230-235, :240, :250 time-mix; :308-309 channel-mix; :156 vocabulary head).
// The device code lives in gemv_body.cuh; this file holds the stand-alone kernel and its launcher.
#include <algorithm>
#include <vector>

#include "gemv_body.cuh"

namespace ab {

struct GemvLaunchShape {
    int Kn, with_dx, xq_bytes;
};
// Shared-memory needs of a launch: the prepared inputs of all its segments (a block touches a subset).
GemvLaunchShape gemv_shape(const GemvParams& p) {
    GemvLaunchShape sh = {0, 0, 0};
    if (p.emb || p.x) sh.Kn = p.K;
    for (int s = 0; s < p.nseg; ++s) {
        if (p.seg[s].mix) sh.with_dx = 1;
        sh.xq_bytes += gemv_xq_bytes(p.seg[s].K);
    }
    return sh;
}

namespace {

__global__ void __launch_bounds__(GEMV_THREADS, 1)
gemv_stream_kernel(const __grid_constant__ GemvParams p, const int Kn, const int with_dx, const int xq_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ BlockPlan bp;
    const GemvSmem m = gemv_smem(smem, gemv_layout(Kn, with_dx, xq_bytes));
    if (threadIdx.x == 0) compute_plan(p, blockIdx.x, gridDim.x, bp);
    __syncthreads();
    int pre_phase = -1;
    if (p.use_pdl) {
        // Launched with programmatic stream serialisation the block may run before its predecessor has finished.
        // Weights are never written, so every warp's first slice starts its way into shared memory now; inputs and
        // outputs are touched only behind the wait.
        const int warp = threadIdx.x >> 5;
        if (warp < bp.n_items) {
            prefetch_item(make_item(p, bp, warp), threadIdx.x & 31, m.pref + warp * (GEMV_ROWS * GEMV_SLICE_BYTES));
            pre_phase = 0;
        }
        pdl_wait();
        pdl_launch_dependents();
    }
    gemv_consume(p, bp, m, threadIdx.x, blockIdx.x, 0, pre_phase, nullptr, nullptr, -1);
}

}  // namespace

int gemv_check(GemvParams& p) {
    AB_CHECK_ARG(p.nseg >= 1 && p.nseg <= GEMV_MAX_SEG, "gemv: nseg %d out of range", p.nseg);
    const bool shared_in = p.emb || p.x;
    AB_CHECK_ARG(!p.emb || (p.token && p.emb_rows > 0), "gemv: embedding input needs a token pointer and the table's row count");
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
        AB_CHECK_ARG(g.fmt != FMT_FP4 || g.K % 32 == 0, "gemv: segment %d: NVFP4 needs K %% 32 == 0", s);
        AB_CHECK_ARG(g.epi != EPI_RESID || g.resid, "gemv: segment %d residual missing", s);
        AB_CHECK_ARG(!g.mix || p.x_prev, "gemv: segment %d: token-shift state missing", s);
    }
    return OK;
}

int gemv_groups(const GemvParams& p) {
    int groups = 0;
    for (int s = 0; s < p.nseg; ++s) groups += gemv_groups_of(p.seg[s].n_rows);
    return groups;
}

// Rows and partial sums of one block must fit the epilogue's one-thread-per-row scheme and the partial area.
int gemv_check_partials(const GemvParams& p, int grid) {
    long long total = 0;
    for (int s = 0; s < p.nseg; ++s)
        total += (long long)gemv_groups_of(p.seg[s].n_rows) * gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
    const long long per_block = (total + grid - 1) / grid;
    long long rows = 0, floats = 0;
    for (int s = 0; s < p.nseg; ++s) {   // worst case: the block's whole share falls into this segment
        const long long unit = gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
        long long groups = per_block / unit + 2;
        if (groups > gemv_groups_of(p.seg[s].n_rows)) groups = gemv_groups_of(p.seg[s].n_rows);
        rows = std::max(rows, groups * GEMV_ROWS + 8 * GEMV_ROWS);
        floats = std::max(floats, (groups + 8) * GEMV_ROWS * gemv_slices(p.seg[s].fmt, p.seg[s].K));
    }
    if (rows > GEMV_MAX_ROWS_PER_BLOCK || floats > GEMV_PART_FLOATS) {
        set_error("gemv: %lld rows / %lld partial sums per block exceed the limits (%d / %d)", rows, floats,
                  GEMV_MAX_ROWS_PER_BLOCK, GEMV_PART_FLOATS);
        return ERR_TOO_LARGE;
    }
    return OK;
}

int gemv_launch(const GemvParams& p_in, cudaStream_t stream) {
    GemvParams p = p_in;
    int st = gemv_check(p);
    if (st != OK) return st;
    static PerDeviceOnce once;
    static size_t static_smem = 0;
    const DeviceProps* dp = nullptr;
    st = once.run(&dp, [](DeviceProps& d) -> int {
        cudaFuncAttributes fa;
        AB_CUDA(cudaFuncGetAttributes(&fa, gemv_stream_kernel));
        static_smem = fa.sharedSizeBytes;
        AB_CUDA(cudaFuncSetAttribute(gemv_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(d.smem_optin - fa.sharedSizeBytes)));
        return (int)OK;
    });
    if (st != OK) return st;
    const int n_sm = dp->n_sm;
    const size_t max_smem = dp->smem_optin - static_smem;
    const GemvLaunchShape sh = gemv_shape(p);
    const size_t smem = gemv_layout(sh.Kn, sh.with_dx, sh.xq_bytes).total;
    AB_CHECK_ARG(smem <= max_smem, "gemv: launch needs %zu bytes of shared memory (limit %zu)", smem, max_smem);
    const int grid = std::max(1, std::min(n_sm, gemv_groups(p)));
    st = gemv_check_partials(p, grid);
    if (st != OK) return st;

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
    AB_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel, p, sh.Kn, sh.with_dx, sh.xq_bytes));
    return OK;
}

}  // namespace ab

// Host-side self-check of the block partition (no GPU needed): every row group of every segment is owned by exactly
// one block, a block's share of a segment is one contiguous run, and the per-block counts stay inside the kernel's
// limits. Returns OK or ERR_BAD_ARG with a message; `max_items` / `max_cost_spread_pct` (optional) report the largest
// item count of a block and how far the most loaded block is above the mean cost, in percent.
extern "C" int ab_gemv_plan_selftest(const int32_t* fmt, const int32_t* n_rows, const int32_t* k, int nseg, int n_blocks,
                                     int32_t* max_items, int32_t* max_cost_spread_pct) {
    using namespace ab;
    AB_CHECK_ARG(fmt && n_rows && k && nseg >= 1 && nseg <= GEMV_MAX_SEG && n_blocks >= 1, "plan selftest: bad argument");
    GemvParams p = {};
    p.nseg = nseg;
    for (int s = 0; s < nseg; ++s) {
        AB_CHECK_ARG(n_rows[s] > 0 && k[s] > 0 && fmt[s] >= FMT_F16 && fmt[s] <= FMT_FP4, "plan selftest: bad segment %d", s);
        p.seg[s].fmt = fmt[s]; p.seg[s].n_rows = n_rows[s]; p.seg[s].K = k[s];
    }
    std::vector<int> next(nseg, 0);
    long long total_cost = 0, worst = 0;
    int items_max = 0;
    for (int b = 0; b < n_blocks; ++b) {
        BlockPlan bp;
        compute_plan(p, b, n_blocks, bp);
        long long cost = 0;
        int items = 0, rows = 0;
        for (int s = 0; s < nseg; ++s) {
            const SegPlan& q = bp.sp[s];
            AB_CHECK_ARG(q.n_groups >= 0, "plan selftest: negative share (block %d segment %d)", b, s);
            if (q.n_groups > 0)
                AB_CHECK_ARG(q.lo == next[s], "plan selftest: block %d segment %d starts at group %d, expected %d", b, s, q.lo, next[s]);
            if (q.n_groups > 0) next[s] = q.lo + q.n_groups;
            AB_CHECK_ARG(q.npc * q.chunk == q.nks && q.item_base == items && q.row_base == rows,
                         "plan selftest: inconsistent item layout (block %d segment %d)", b, s);
            items += q.n_groups * q.npc;
            rows += q.n_groups * GEMV_ROWS;
            cost += (long long)q.n_groups * gemv_group_cost(fmt[s], k[s]);
        }
        AB_CHECK_ARG(items == bp.n_items && rows == bp.n_rows, "plan selftest: totals of block %d do not add up", b);
        items_max = std::max(items_max, items);
        worst = std::max(worst, cost);
        total_cost += cost;
    }
    for (int s = 0; s < nseg; ++s)
        AB_CHECK_ARG(next[s] == gemv_groups_of(n_rows[s]), "plan selftest: segment %d covered up to group %d of %d", s, next[s],
                     gemv_groups_of(n_rows[s]));
    if (max_items) *max_items = items_max;
    if (max_cost_spread_pct) {
        const double mean = (double)total_cost / n_blocks;
        *max_cost_spread_pct = mean > 0 ? (int)((worst / mean - 1.0) * 100.0 + 0.5) : 0;
    }
    return OK;
}
