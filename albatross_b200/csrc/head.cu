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

}  // namespace

int head_launch(const HeadParams& p, cudaStream_t stream) {
    AB_CHECK_ARG(p.B > 0 && p.T > 0 && p.H > 0 && p.D == p.H * HEAD, "head: bad shape B=%d T=%d D=%d H=%d", p.B, p.T, p.D, p.H);
    AB_CHECK_ARG(p.state && p.r && p.k && p.v && p.v_first && p.out, "head: null pointer");
    const bool ups = p.w2 != nullptr;
    AB_CHECK_ARG(ups || (p.w_raw && p.a_raw && p.g && (p.layer0 || p.vg_raw)), "head: adapter outputs missing");
    AB_CHECK_ARG(!ups || (p.B == 1 && p.T == 1), "head: in-kernel adapter up-projection is the batch-1 path");
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
