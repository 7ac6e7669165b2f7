// Batched matrix products of the RWKV-7 batch path and the de-quantisation dump.
#include "gemm.cuh"
#include "gemv.cuh"

namespace ab {

namespace {

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
    int s = check_mat(m, "gemm");
    if (s != OK) return s;
    AB_CHECK_ARG(rows > 0 && x && y, "gemm: bad argument");
    for (int r = 0; r < rows; ++r) {
        GemvParams p = {};
        p.nseg = 1;
        p.K = m.k;
        p.x = x + (size_t)r * m.k;
        GemvSeg& g = p.seg[0];
        g.w = m.w; g.scale = m.scale; g.col_scale = m.col_scale; g.tscale = m.tscale;
        g.fmt = m.fmt; g.epi = epi; g.n_rows = m.n_out; g.K = m.k;
        g.out = y + (size_t)r * m.n_out;
        g.resid = resid ? resid + (size_t)r * m.n_out : nullptr;
        s = gemv_launch(p, stream);
        if (s != OK) return s;
    }
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
