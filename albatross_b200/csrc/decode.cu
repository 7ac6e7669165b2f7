// Persistent batch-1 decode kernel: one launch runs every phase of one token.
//
// The reference's single-token path (reference/rwkv7.py:128-157) is ~190 dependent steps, each far
// shorter than a kernel boundary. Here one block per SM stays resident for the whole token:
//   * every warp runs the phases (matrix-vector products with fused prologue / epilogue, and the
//     per-head WKV-7 step); weights stream HBM -> registers with 128-bit loads;
//   * blocks meet at a grid-wide barrier between phases: a monotonically increasing counter in
//     global memory, arrive = release-add, wait = four staggered pollers with bounded acquire spins;
//   * requesting the next phase's weights early (L2 prefetch, cp.async of each warp's first slice before or while
//     the block waits at the barrier) exists as options and is off: all of it measured slower, because the requests
//     sit in front of the small loads of the next phase's input vector, which are the critical path.
// Every wait is bounded; on expiry the block sets the device status word and stops waiting.
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
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Barrier among all blocks. `failed` becomes (and stays) true once a wait has run out.
// `while_waiting` runs in every thread after the block has announced its arrival and before thread 0 starts to
// poll: work that does not depend on other blocks (requests for the next phase's first weights) goes there, so that
// it neither delays the arrival nor shares the memory pipeline with the loads that follow the barrier.
template <class F>
__device__ __forceinline__ void grid_barrier(unsigned* counter, unsigned target, int tid, bool& failed, F while_waiting) {
    __shared__ volatile int s_done, s_ok;
    cons_sync();   // every thread of the block has issued its writes of this phase
    if (tid == 0) {
        s_done = 0;
        s_ok = failed ? 0 : 1;
        if (!failed) red_release_add(counter, 1u);
    }
    while_waiting();
    // Four pollers (lane 0 of warps 0-3), a fifth of a round trip apart: the block notices the last arrival a
    // fraction of an L2 round trip after it happened instead of up to a whole one.
    cons_sync();
    if ((tid & 31) == 0 && tid < 128 && !failed) {
        if (tid) __nanosleep((unsigned)(tid >> 5) * 160u);
        uint32_t it = 0;
        while (!s_done) {
            if (ld_acquire_u32(counter) >= target) break;
            if (++it > (1u << 23)) {
                s_ok = 0;
                atomicOr(&g_device_status, DEV_WAIT_HEAD);
                break;
            }
        }
        s_done = 1;
    }
    cons_sync();
    if (!s_ok) failed = true;
}

__device__ __forceinline__ void stage_phase(DecodePhase* dst, const DecodePhase* src, int tid) {
    for (int j = tid; j < (int)(sizeof(DecodePhase) / 16); j += NT_CONS)
        reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(src)[j];
}

// The per-head phase of one network block. Its own function (not inlined) so that the register allocation of the
// matrix-vector phases, which run at the kernel's register cap, does not have to make room for it.
__device__ __noinline__ void head_phase(const HeadParams& hp, int bid, int nb, int tid, unsigned char* smem, unsigned char* pref,
                                        const __half* xn, HeadShared& hsh, uint32_t epoch, unsigned long long* htl) {
    // adapter up-projections inside the phase: block h needs only the 64 channels of head h, so the
    // matrix-vector phase (and the grid barrier) that would produce them for everybody is not needed
    const bool ups = hp.w2 != nullptr;
    // Dataflow mode (pair_mode): no barrier among all blocks came before this phase. Block 2h runs head h; its
    // inputs (the head's r / k / v rows, the adapter hidden vectors) are tagged words and the loads wait for
    // them one by one. Everybody else goes straight on to the next phase.
    const bool pair = hp.pair_mode != 0;
    const bool mine = !pair || (bid < 2 * hp.H && (bid & 1) == 0);
    for (int h = pair ? (bid >> 1) : bid; mine && h < hp.H; h += pair ? hp.H : nb) {   // block-uniform
        if (tid < HT) {
            unsigned char* dsm = pair ? pref : smem;   // pair mode: staged during the phase before
            if (ups && !pair) head_ups_stage(hp, h, tid, dsm);   // the matrix-vector buffers are idle in this phase
            float* sbase = hp.state + (size_t)h * 4096;
            StateRow st;
            load_state(st, sbase, tid >> 2, tid & 3);   // last written a token ago: in flight while the inputs arrive
            const HeadTags tg = {hp.tag_in != 0, tag_of(epoch, hp.tag_in), tag_of(epoch, hp.tag_out)};
            if (ups) head_ups_compute(hp, tid, dsm, hsh, SyncNamed256(), tg, htl);
            if (htl) htl[2] = global_ns();
            head_steps(hp, 0, h, tid, st, hsh, ups, SyncNamed256(), tg, (pair && ups) ? head_par_area(hp, dsm) : nullptr);
            if (htl) htl[3] = global_ns();
            store_state(st, sbase, tid >> 2, tid & 3);
            // token-shift state hand-over. Pair mode: the normalised input of the phase before is still in this
            // block's shared memory (every block prepared it), so no other block's global write is read here.
            if (hp.copy_dst && tid < 32)
                reinterpret_cast<__half2*>(hp.copy_dst + h * 64)[tid] =
                    pair ? reinterpret_cast<const __half2*>(xn + h * 64)[tid]
                         : __ldcg(reinterpret_cast<const __half2*>(hp.copy_src + h * 64) + tid);
            SyncNamed256()();
        }
    }
}

__global__ void __launch_bounds__(GEMV_THREADS, 1) decode_kernel(const DecodeProgram* __restrict__ prog) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ HeadShared hsh;
    // phase descriptors are staged three phases ahead in a ring of four; block plans one matrix-vector phase ahead
    __shared__ __align__(16) DecodePhase phs[4];
    __shared__ __align__(16) BlockPlan plans[4];   // staged like the descriptors, indexed by phase & 3
    const int tid = threadIdx.x;
    const int bid = blockIdx.x, nb = gridDim.x;
    const int n_phases = prog->n_phases;
    const GemvSmem m = gemv_smem(smem, gemv_layout(prog->Kn, 1, prog->xq_bytes));

    const BlockPlan* my_plans = prog->plans + bid;   // plan of phase i: my_plans[i * nb]
    auto stage_plan = [&](int i) {
        for (int j = tid; j < (int)(sizeof(BlockPlan) / 16); j += NT_CONS)
            reinterpret_cast<uint4*>(&plans[i & 3])[j] = reinterpret_cast<const uint4*>(&my_plans[(size_t)i * nb])[j];
    };
    for (int i = 0; i < 3 && i < n_phases; ++i) {
        stage_phase(&phs[i], &prog->phases[i], tid);
        stage_plan(i);
    }
    __syncthreads();

    const uint32_t epoch = prog->epoch;   // tag base of this token (dataflow mode)
    // this block's time stamps: [2 * n] phase start / end, then [4 * n] inside the phase; timeline_block < 0: every block
    // records, into consecutive areas of timeline_stride entries
    auto tl_base = [&]() -> unsigned long long* {
        if (!prog->timeline) return nullptr;
        if (prog->timeline_block < 0) return prog->timeline + (size_t)bid * prog->timeline_stride;
        return bid == prog->timeline_block ? prog->timeline : nullptr;
    };
    bool failed = false;
    int pre_phase = -1;
    unsigned n_barriers = 0;
    for (int i = 0; i < n_phases; ++i) {
        // Descriptor and plan of phase i + 3 are copied asynchronously (a synchronous copy stalls every warp for a
        // memory round trip at the top of every phase). This thread's copies of the earlier iterations are complete
        // after the wait; the block barrier at the end of the iteration publishes them, two phases before their use.
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (i + 3 < n_phases) {
            const unsigned char* src_ph = reinterpret_cast<const unsigned char*>(&prog->phases[i + 3]);
            unsigned char* dst_ph = reinterpret_cast<unsigned char*>(&phs[(i + 3) & 3]);
            for (int j = tid; j < (int)(sizeof(DecodePhase) / 16); j += NT_CONS)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_ph + 16 * j)), "l"(src_ph + 16 * j) : "memory");
            const unsigned char* src_pl = reinterpret_cast<const unsigned char*>(&my_plans[(size_t)(i + 3) * nb]);
            unsigned char* dst_pl = reinterpret_cast<unsigned char*>(&plans[(i + 3) & 3]);
            for (int j = tid; j < (int)(sizeof(BlockPlan) / 16); j += NT_CONS)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_pl + 16 * j)), "l"(src_pl + 16 * j) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        const DecodePhase& ph = phs[i & 3];
        if (tid == 0 && tl_base()) tl_base()[2 * i] = global_ns();
        if (ph.type == PHASE_GEMV) {
            const int j = ph.next_gemv;
            const bool pre = j >= 0 && prog->smem_prefetch;
            gemv_consume(ph.g, plans[i & 3], m, tid, bid, i, pre_phase, pre ? &phs[j & 3].g : nullptr,
                         pre ? &plans[j & 3] : nullptr, j,
                         tl_base() ? tl_base() + 2 * n_phases + 4 * i : nullptr,
                         // the first-slice prefetch uses the area that the phase before a paired head phase stages into
                         (i + 1 < n_phases && phs[(i + 1) & 3].type == PHASE_HEAD && phs[(i + 1) & 3].h.pair_mode) ? 0 : prog->early_slice,
                         [&]() {
                             if (ph.no_barrier == 2 && tid < HT && bid < 2 * phs[(i + 1) & 3].h.H && (bid & 1) == 0) {
                                 // "fused heads": this block runs head bid / 2 right after the phase. Its slices of the
                                 // four adapter up-projection matrices (weights: no dependency) move into the idle
                                 // prefetch area while the phase's own weights stream; requested any earlier they would
                                 // sit in front of the loads of the phase's input vector. The head's per-channel
                                 // parameters and its state (last touched a token ago) are pulled towards the SM as well.
                                 const HeadParams& nh = phs[(i + 1) & 3].h;
                                 const int h = bid >> 1;
                                 head_ups_stage(nh, h, tid, m.pref);
                                 head_par_stage(nh, h, tid, m.pref);
                                 asm volatile("cp.async.commit_group;" ::: "memory");
                                 if (tid < 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(nh.state + (size_t)h * 4096 + tid * 32));
                             }
                         }, epoch, prog->l2_prefetch_bytes + (prog->early_slice ? GEMV_WARPS * GEMV_ROWS * GEMV_SLICE_BYTES : 0), prog->l2_prefetch2_bytes);
            // The memory system idles from the moment the blocks run out of weights until the next phase's inputs have
            // crossed the chip and been prepared. One thread asks for the head of this block's share of the next
            // matrix-vector phase to be moved HBM -> L2 in that window (no data returns to the SM: the request does not
            // sit in front of the loads that wait for the inputs).
            if (tid == 32 && j >= 0 && prog->l2_prefetch_bytes > 0) prefetch_share(phs[j & 3].g, plans[j & 3], 0, prog->l2_prefetch_bytes);
        } else {
            head_phase(ph.h, bid, nb, tid, smem, m.pref, m.xn, hsh, epoch,
                       (tid == 0 && tl_base()) ? tl_base() + 2 * n_phases + 4 * i : nullptr);
        }
        if (tid == 0 && tl_base()) tl_base()[2 * i + 1] = global_ns();
        if (i + 1 < n_phases) {
            if (ph.no_barrier) {
                // a block barrier only: either the same block produces and consumes, or (dataflow mode) the phase's
                // outputs are tagged words that their readers wait for; the block's shared memory is free for the next phase
                cons_sync();
            } else {
                const int j = ph.type == PHASE_GEMV ? ph.next_gemv : -1;
                grid_barrier(prog->barrier, (unsigned)(++n_barriers) * nb, tid, failed, [&]() {
                    // the warp's first work item of the next matrix-vector phase starts its way into shared memory
                    if (prog->barrier_prefetch && j >= 0 && pre_phase != j) {
                        const GemvParams& q = phs[j & 3].g;
                        const BlockPlan& np_ = plans[j & 3];
                        const int w = tid >> 5;
                        if (w < np_.n_items)
                            prefetch_item(make_item(q, np_, w), tid & 31, m.pref + w * (GEMV_ROWS * GEMV_SLICE_BYTES));
                        pre_phase = j;
                    }
                });
            }
        }
    }
    // Every block has read the tag base by now (block 0 could not have finished the last phase otherwise).
    if (bid == 0 && tid == 0) const_cast<DecodeProgram*>(prog)->epoch = epoch + (uint32_t)n_phases;
}

}  // namespace

size_t decode_plans_offset(int n_phases) {
    return (sizeof(DecodeProgram) + sizeof(DecodePhase) * (size_t)n_phases + 255) & ~(size_t)255;
}
size_t decode_timeline_offset(int n_phases, int n_blocks) {
    return (decode_plans_offset(n_phases) + sizeof(BlockPlan) * (size_t)n_phases * n_blocks + 255) & ~(size_t)255;
}
size_t decode_program_bytes(int n_layer, int n_blocks) {
    const int n_phases = 6 * n_layer + 1;
    return decode_timeline_offset(n_phases, n_blocks) + 48 * (size_t)n_phases * n_blocks + 256;
}

int decode_launch(const DecodeProgram* prog_dev, unsigned* barrier_dev, int Kn, int xq_bytes, cudaStream_t stream) {
    static PerDeviceOnce once;
    static size_t static_smem = 0;
    const DeviceProps* dp = nullptr;
    {
        const int s = once.run(&dp, [](DeviceProps& d) -> int {
            int dev = 0, coop = 0;
            AB_CUDA(cudaGetDevice(&dev));
            AB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
            AB_CHECK_ARG(coop, "decode: device does not support cooperative launch");
            cudaFuncAttributes fa;
            AB_CUDA(cudaFuncGetAttributes(&fa, decode_kernel));
            static_smem = fa.sharedSizeBytes;
            // the largest dynamic size the device allows next to the kernel's static shared memory, set once
            AB_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(d.smem_optin - fa.sharedSizeBytes)));
            return (int)OK;
        });
        if (s != OK) return s;
    }
    const int n_sm = dp->n_sm;
    const size_t max_smem = dp->smem_optin - static_smem;
    const size_t smem = gemv_layout(Kn, 1, xq_bytes).total;
    AB_CHECK_ARG(smem <= max_smem, "decode: needs %zu bytes of shared memory (limit %zu)", smem, max_smem);
    int per_sm = 0;
    AB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_kernel, GEMV_THREADS, smem));
    AB_CHECK_ARG(per_sm >= 1, "decode: kernel does not fit on an SM");
    AB_CUDA(cudaMemsetAsync(barrier_dev, 0, 4, stream));
    void* args[] = {(void*)&prog_dev};
    AB_CUDA(cudaLaunchCooperativeKernel((const void*)decode_kernel, dim3(n_sm), dim3(GEMV_THREADS), args, smem, stream));
    return OK;
}

}  // namespace ab
