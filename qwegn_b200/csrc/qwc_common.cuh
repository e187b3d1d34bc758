// Shared definitions for the sm_100a quantized-matmul kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qwc.h"

struct qwc_hal {
    int device;
    int sm_count;
    int max_smem_optin;
    int32_t* status;  // device: [0] first error code written by a kernel, [1] detail
    void* encode_tiled;  // driver entry point cuTensorMapEncodeTiled (null if unavailable)
    int static_weights;  // the caller promised that weight banks are never written by in-flight work (see qwc_hal_set_static_weights)
};

// Error reporting (thread-local message, status code returned).
int qwc_fail(int code, const char* fmt, ...);
void qwc_clear_error();
#define QWC_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) return qwc_fail(QWC_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// Tuning knobs read from the environment exist only in builds made with -DQWC_TUNING (parameter sweeps); the shipped
// library takes every choice from the shape of the call.
#ifdef QWC_TUNING
#include <cstdlib>
inline int tune_env(const char* name, int fallback) {
    const char* v = getenv(name);
    return v ? atoi(v) : fallback;
}
#else
inline int tune_env(const char*, int fallback) { return fallback; }
#endif

#ifdef __CUDACC__
// Launch with programmatic stream serialization (see pdl_enter): the kernel must call pdl_enter() (or the two
// griddepcontrol instructions) before it touches global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t qwc_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Argument checks shared by the doors (qwc_api.cu): every refusal a later launch could make, without launching.
int qwc_check_view(const qwc_weight_view* w);
int qwc_gemm_check(const qwc_hal* hal, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx, void* y, int32_t y_dtype,
                   int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace, size_t workspace_bytes);
int qwc_gemm_args_check_stream(const qwc_hal* hal, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx, void* y,
                               int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace,
                               size_t workspace_bytes);

// The three containers this library decodes.
enum QwcFmt : int { FMT_HQ4_G32_M5 = 0, FMT_HQ8_G32 = 1, FMT_HQ4_G64 = 2, FMT_UNSUPPORTED = -1 };
// Fewest tokens the tensor-core path takes, per format (measured crossover against the streaming kernel).
inline int qwc_tc_min_tokens(int fmt) { return fmt == FMT_HQ8_G32 ? 8 : 9; }

inline int qwc_fmt_of(const qwc_weight_view& w) {
    if (w.kind == QWC_KIND_HQ4_G32_M5) return FMT_HQ4_G32_M5;
    if (w.kind == QWC_KIND_ROTATED_HQ && w.bits == 8 && w.group == 32) return FMT_HQ8_G32;
    if (w.kind == QWC_KIND_ROTATED_HQ && w.bits == 4 && w.group == 64) return FMT_HQ4_G64;
    return FMT_UNSUPPORTED;
}

// Per-format byte geometry.  A "unit" is 32 consecutive k (one FWHT block, one pair of k16 MMAs).
template <int FMT> struct FmtTraits;
template <> struct FmtTraits<FMT_HQ4_G32_M5> {
    static constexpr int kBlockBytes = 20, kGroup = 32, kUnitsPerBlock = 1;
};
template <> struct FmtTraits<FMT_HQ8_G32> {
    static constexpr int kBlockBytes = 36, kGroup = 32, kUnitsPerBlock = 1;
};
template <> struct FmtTraits<FMT_HQ4_G64> {
    static constexpr int kBlockBytes = 36, kGroup = 64, kUnitsPerBlock = 2;
};

// Kernel status codes written to qwc_hal::status[0].
enum { QWC_DEV_OK = 0, QWC_DEV_WAIT_FULL_TIMEOUT = 101, QWC_DEV_WAIT_EMPTY_TIMEOUT = 102,
       QWC_DEV_WAIT_MMA_TIMEOUT = 103, QWC_DEV_WAIT_TMEM_TIMEOUT = 104, QWC_DEV_WAIT_PEER_TIMEOUT = 105, QWC_DEV_NONFINITE_WEIGHT = 201 };

#ifdef __CUDACC__

__device__ __forceinline__ float qwc_inv_sqrt32() { return __uint_as_float(0x3E3504F3u); }

// One FWHT-32 stage across lanes: lane holds v, partner lane = lane ^ mask.
__device__ __forceinline__ float fwht_xor_stage(float v, int lane_mask, bool upper) {
    float o = __shfl_xor_sync(0xFFFFFFFFu, v, lane_mask);
    return upper ? __fsub_rn(o, v) : __fadd_rn(v, o);
}

// Programmatic dependent launch, used between the kernels of one operator chain: a kernel lets its successor be
// scheduled at once (the successor's launch latency and set-up then overlap this kernel) and waits for its predecessor
// -- the whole grid, memory flushed -- before its first global access.  Both are no-ops in an ordinary launch.  The wait
// comes before any early return, so that "this grid completed" always implies "the grid before it completed".
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- mbarrier / bulk-copy helpers (all waits bounded) ----------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Suspend-time hint of try_wait (ns): the waiting thread sleeps in hardware until the phase completes instead of
// spinning through the issue slots; measured to matter (spinning waiters slowed the tensor-core kernel by 15 %).
#ifndef QWC_TRY_WAIT_HINT_NS
#define QWC_TRY_WAIT_HINT_NS 20000
#endif
#ifndef QWC_RELAXED_SLEEP_NS
#define QWC_RELAXED_SLEEP_NS 512
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
#if QWC_TRY_WAIT_HINT_NS > 0
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(static_cast<uint32_t>(QWC_TRY_WAIT_HINT_NS))
        : "memory");
#else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
#endif
    return ok != 0;
}
// Non-blocking test of a phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Device wall clock in nanoseconds (the bounded waits measure elapsed time, not poll counts).
__device__ __forceinline__ uint64_t qwc_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// How long a wait may last before the kernel gives up, sets its status word and winds down.  A healthy pipeline
// never waits longer than a few microseconds; the limit only has to be far above that and short enough that a stuck
// kernel frees the GPU quickly.
#ifndef QWC_WAIT_LIMIT_NS
#define QWC_WAIT_LIMIT_NS 1000000000ull
#endif
// Bounded wait: true when the phase completed; false when QWC_WAIT_LIMIT_NS passed or another role of the CTA raised
// `abort_flag` (so that after one role fails the others leave at once instead of running out their own limits).  The
// clock is first read after 32 failed polls and then every 32nd poll (a poll may itself sleep up to the suspend hint):
// reading it on every miss put a timer read on the pipeline's critical path.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag = nullptr) {
    if (mbar_test(bar, parity)) return true;   // the phase is often complete already: skip the suspending form
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 31u) {
            if (abort_flag != nullptr && *abort_flag) return false;
            const uint64_t now = qwc_globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > QWC_WAIT_LIMIT_NS) return false;
        }
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
}
// Bounded wait for the roles whose waits are long (an epilogue waiting for a whole main loop, a producer waiting for
// a free stage): sleeps between polls from the first miss on, so that the waiting warps leave the issue slots to the
// warps that do the decoding.  Same limit and abort rule as mbar_wait.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, const volatile int* abort_flag = nullptr) {
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 31u) {
            if (abort_flag != nullptr && *abort_flag) return false;
            const uint64_t now = qwc_globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > QWC_WAIT_LIMIT_NS) return false;
        }
        __nanosleep(i < 16 ? QWC_RELAXED_SLEEP_NS / 4 : QWC_RELAXED_SLEEP_NS);
    }
}
// Bounded wait until a CTA-scope counter in shared memory (published with a release store) exceeds `q`.
__device__ __forceinline__ uint32_t ld_acquire_cta_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_counter_above(const uint32_t* ctr, uint32_t q, const volatile int* abort_flag) {
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (ld_acquire_cta_u32(ctr) > q) return true;
        if ((i & 63u) == 63u) {
            if (abort_flag != nullptr && *abort_flag) return false;
            const uint64_t now = qwc_globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > QWC_WAIT_LIMIT_NS) return false;
        }
        __nanosleep(i < 64 ? 20 : 200);
    }
}
// 1-D bulk async copy global -> this CTA's shared memory, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

#endif  // __CUDACC__
