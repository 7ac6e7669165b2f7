// Shared device/host helpers for the sm_100a kernels of the RWKV-7 decode path.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace ab {

// ---------------------------------------------------------------------------------------------
// Status codes returned by every extern "C" entry point (0 = success).
// ---------------------------------------------------------------------------------------------
enum Status : int {
    OK = 0,
    ERR_BAD_ARG = -1,      // null pointer, misaligned pointer, unsupported shape
    ERR_CUDA = -2,         // a CUDA runtime call failed; see ab_last_error()
    ERR_TOO_LARGE = -3,    // size exceeds a compiled-in limit
    ERR_DEVICE_WAIT = -4,  // a bounded device-side wait ran out (reported through the status word)
};

void set_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

#define AB_CHECK_ARG(cond, ...)                 \
    do {                                        \
        if (!(cond)) {                          \
            ab::set_error(__VA_ARGS__);         \
            return ab::ERR_BAD_ARG;             \
        }                                       \
    } while (0)

#define AB_CUDA(call)                                        \
    do {                                                     \
        int _s = ab::check_cuda((call), #call);              \
        if (_s != ab::OK) return _s;                         \
    } while (0)

// One-time set-up of a launcher (function attributes, device properties) is per DEVICE, not per process: a process
// may drive several GPUs, and cudaFuncSetAttribute applies to the current one only. `run` executes `f` the first time
// it is called with a given device current (under a lock: host threads may launch concurrently) and remembers success.
constexpr int AB_MAX_DEVICES = 64;
struct DeviceProps {
    int n_sm = 0;
    size_t smem_optin = 0;
};
struct PerDeviceOnce {
    std::mutex mu;
    bool done[AB_MAX_DEVICES] = {};
    DeviceProps props[AB_MAX_DEVICES];
    template <class F>
    int run(const DeviceProps** out, F f) {
        int dev = 0;
        AB_CUDA(cudaGetDevice(&dev));
        AB_CHECK_ARG(dev >= 0 && dev < AB_MAX_DEVICES, "device index %d not supported (at most %d devices per process)", dev, AB_MAX_DEVICES);
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            int v = 0, m = 0;
            AB_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            AB_CUDA(cudaDeviceGetAttribute(&m, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            props[dev].n_sm = v;
            props[dev].smem_optin = (size_t)m;
            const int s = f(props[dev]);
            if (s != OK) return s;
            done[dev] = true;
        }
        if (out) *out = &props[dev];
        return OK;
    }
};

// Device-side status word: kernels OR a bit in when a bounded wait gives up.
// The host reads it with ab_device_status().
static __device__ unsigned int g_device_status = 0;
constexpr unsigned int DEV_WAIT_GEMV = 1u;
constexpr unsigned int DEV_WAIT_GEMM = 2u;
constexpr unsigned int DEV_WAIT_HEAD = 4u;
constexpr unsigned int DEV_BOUNDS = 16u;     // bounds-checked build only: a computed index fell outside its array (the access was skipped)
constexpr unsigned int DEV_BAD_TOKEN = 8u;   // a token id outside [0, vocab) reached a kernel (it was clamped, not followed)

#ifndef TAG_POLL_NS_VALUE
#define TAG_POLL_NS_VALUE 100u
#endif
constexpr unsigned TAG_POLL_NS = TAG_POLL_NS_VALUE;   // pause between two looks at a tagged word that is not there yet

// Bounds-checked build (-DAB_BOUNDS_CHECK, `python -m albatross_b200.build --bounds-check`): the stand-in for a memory
// checker where none can be run. AB_BC(cond) is `true` in the normal build and costs nothing; in the checked build it
// evaluates the range condition of the access it guards, and when the condition fails it records DEV_BOUNDS in the status
// word and yields false, so that the access is skipped instead of made: `if (AB_BC(i < n)) a[i] = v;`.
#ifdef AB_BOUNDS_CHECK
#define AB_BC(cond) ((cond) ? true : (atomicOr(&ab::g_device_status, ab::DEV_BOUNDS), false))
#else
#define AB_BC(cond) true
#endif

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `ns` before it reports "not yet":
// polling in a tight loop floods the shared-memory pipe that the math loads need.
__device__ __forceinline__ bool mbar_try_wait_park(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller records an error) instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t max_iters = (1u << 20)) {
    for (uint32_t i = 0; i < max_iters; ++i) {
        if (mbar_try_wait_park(bar, parity, 2000u)) return true;
        if (i > 4) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 1-D bulk (TMA) copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Same with an L2 eviction-priority hint (weights are streamed once: evict first).
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Programmatic dependent launch: wait for the preceding grid in the stream / let the next one start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 4-way int8 dot products. a: signed bytes; b: signed (ss) or unsigned (su) bytes.
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One byte holding two e2m1 codes (low nibble first) -> half2.
__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
    uint32_t out;
    asm("{\n .reg .b8 lo, hi;\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n mov.b16 {lo, hi}, t;\n cvt.rn.f16x2.e2m1x2 %0, lo;\n}"
        : "=r"(out)
        : "r"(byte));
    return *reinterpret_cast<__half2*>(&out);
}
// Four bytes = eight e2m1 codes -> four half2 (byte i -> out[i], low nibble first): one unpack, four converts.
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t word, uint32_t* out) {
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
        : "r"(word));
}
// Two e4m3 codes (16 bits) -> half2.
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t two) {
    uint32_t out;
    asm("{\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n cvt.rn.f16x2.e4m3x2 %0, t;\n}" : "=r"(out) : "r"(two));
    return *reinterpret_cast<__half2*>(&out);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
    return __low2float(e4m3x2_to_half2(code & 0xffu));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// fp16 rounding points: the reference computes its glue in fp16 tensors, so each torch op rounds.
__device__ __forceinline__ float rh(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + __expf(-v)); }

constexpr int HEAD = 64;

}  // namespace ab
