// Persistent batch-1 decode kernel: one launch runs every phase of one token.
//
// The reference's single-token path (reference/rwkv7.py:128-157) is ~190 dependent steps, each far
// shorter than a kernel boundary. Here one block per SM stays resident for the whole token:
//   * the producer warp of each block walks the phase list and streams that block's share of every
//     weight matrix through the shared-memory rings without ever waiting for another block (weights
//     do not depend on activations), so HBM stays busy across phase boundaries;
//   * consumer warps run the phases (matrix-vector products with fused prologue / epilogue, and the
//     per-head WKV-7 step) and meet at a grid-wide barrier between phases: a monotonically
//     increasing counter in global memory, arrive = fence + atomic add, wait = bounded acquire spin.
// Every wait is bounded; on expiry the block sets the device status word and stops waiting.
#include <cooperative_groups.h>

#include "decode.cuh"
#include "gemv_body.cuh"
#include "head_body.cuh"

namespace ab {

namespace {

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Barrier among the consumer threads of all blocks. Returns false once a wait has run out.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int tid, bool& failed) {
    __shared__ int s_ok;
    cons_sync();
    if (tid == 0) {
        int ok = 1;
        if (!failed) {
            __threadfence();
            atomicAdd(counter, 1u);
            uint32_t it = 0;
            while (ld_acquire_u32(counter) < target) {
                if (++it > (1u << 22)) {
                    ok = 0;
                    atomicOr(&g_device_status, DEV_WAIT_HEAD);
                    break;
                }
                __nanosleep(20);
            }
            __threadfence();
        } else {
            ok = 0;
        }
        s_ok = ok;
    }
    cons_sync();
    if (!s_ok) failed = true;
    return !failed;
}

__global__ void __launch_bounds__(GEMV_THREADS, 1) decode_kernel(const DecodeProgram* __restrict__ prog) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ HeadShared hsh;
    // phase descriptors are staged in shared memory: the inner loops read them constantly
    __shared__ __align__(16) DecodePhase cons_ph;
    __shared__ __align__(16) GemvParams prod_g;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bid = blockIdx.x, nb = gridDim.x;
    const int n_phases = prog->n_phases;
    const GemvLayout L = gemv_layout(prog->stages, prog->Kn, 1, prog->Kq);
    const GemvSmem m = gemv_smem(smem, L, prog->stages);
    if (tid == 0) gemv_init_barriers(m);
    __syncthreads();

    if (warp == GEMV_WARPS) {
        if (lane < GEMV_WARPS) {
            ProducerState ps = {0, 0, 0, false};
            const uint64_t policy = policy_evict_first();
            for (int i = 0; i < n_phases && !ps.dead; ++i) {
                const DecodePhase& ph = prog->phases[i];
                if (ph.type != PHASE_GEMV) continue;
                __syncwarp(0xffffu);
                for (int j = lane; j < (int)(sizeof(GemvParams) / 16); j += GEMV_WARPS)
                    reinterpret_cast<uint4*>(&prod_g)[j] = reinterpret_cast<const uint4*>(&ph.g)[j];
                __syncwarp(0xffffu);
                gemv_produce(prod_g, m, ps, lane, bid, nb, policy);
            }
        }
        return;
    }

    ConsumerState cs = {0, 0, false};
    bool failed = false;
    for (int i = 0; i < n_phases; ++i) {
        for (int j = tid; j < (int)(sizeof(DecodePhase) / 16); j += NT_CONS)
            reinterpret_cast<uint4*>(&cons_ph)[j] = reinterpret_cast<const uint4*>(&prog->phases[i])[j];
        cons_sync();
        const DecodePhase& ph = cons_ph;
        if (prog->timeline && bid == 0 && tid == 0) prog->timeline[2 * i] = global_ns();
        if (ph.type == PHASE_GEMV) {
            gemv_consume(ph.g, m, cs, tid, bid, nb);
        } else {
            const HeadParams& hp = ph.h;
            for (int h = bid; h < hp.H; h += nb) {   // block-uniform
                if (tid < HT) {
                    float* sbase = hp.state + (size_t)h * 4096;
                    StateRow st;
                    load_state(st, sbase, tid >> 2, tid & 3);
                    head_steps(hp, 0, h, tid, st, hsh, false, SyncNamed256());
                    store_state(st, sbase, tid >> 2, tid & 3);
                    if (hp.copy_src && tid < 32)
                        reinterpret_cast<__half2*>(hp.copy_dst + h * 64)[tid] =
                            __ldcg(reinterpret_cast<const __half2*>(hp.copy_src + h * 64) + tid);
                    SyncNamed256()();
                }
            }
        }
        if (prog->timeline && bid == 0 && tid == 0) prog->timeline[2 * i + 1] = global_ns();
        if (i + 1 < n_phases) grid_barrier(prog->barrier, (unsigned)(i + 1) * nb, tid, failed);
        if (failed) cs.failed = true;
    }
}

}  // namespace

size_t decode_program_bytes(int n_layer) {
    return sizeof(DecodeProgram) + (sizeof(DecodePhase) + 16) * (size_t)(6 * n_layer + 1) + 256;
}

int decode_launch(const DecodeProgram* prog_dev, unsigned* barrier_dev, int stages, int Kn, int Kq, cudaStream_t stream) {
    static int n_sm = 0;
    static size_t max_smem = 0;
    if (!n_sm) {
        int dev = 0, v = 0, m = 0, coop = 0;
        AB_CUDA(cudaGetDevice(&dev));
        AB_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        AB_CUDA(cudaDeviceGetAttribute(&m, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        AB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        AB_CHECK_ARG(coop, "decode: device does not support cooperative launch");
        cudaFuncAttributes fa;
        AB_CUDA(cudaFuncGetAttributes(&fa, decode_kernel));
        max_smem = (size_t)m - fa.sharedSizeBytes;
        n_sm = v;
    }
    const size_t smem = gemv_layout(stages, Kn, 1, Kq).total;
    AB_CHECK_ARG(smem <= max_smem, "decode: needs %zu bytes of shared memory (limit %zu)", smem, max_smem);
    static size_t smem_set = 0;
    if (smem > smem_set) {
        AB_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        smem_set = smem;
    }
    int per_sm = 0;
    AB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_kernel, GEMV_THREADS, smem));
    AB_CHECK_ARG(per_sm >= 1, "decode: kernel does not fit on an SM");
    AB_CUDA(cudaMemsetAsync(barrier_dev, 0, 4, stream));
    void* args[] = {(void*)&prog_dev};
    AB_CUDA(cudaLaunchCooperativeKernel((const void*)decode_kernel, dim3(n_sm), dim3(GEMV_THREADS), args, smem, stream));
    return OK;
}

}  // namespace ab
