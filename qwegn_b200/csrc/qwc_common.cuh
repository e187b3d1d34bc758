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

// The three containers this library decodes.
enum QwcFmt : int { FMT_HQ4_G32_M5 = 0, FMT_HQ8_G32 = 1, FMT_HQ4_G64 = 2, FMT_UNSUPPORTED = -1 };

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
// Bounded wait: gives up after ~2^22 polls (several seconds at worst) and reports false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;   // the phase is often complete already: skip the suspending form
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}
// Bounded wait for the roles whose waits are long (an epilogue waiting for a whole main loop, a producer waiting for
// a free stage): sleeps between polls from the first miss on, so that the waiting warps leave the issue slots to the
// warps that do the decoding.  Gives up after ~1 s.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 21); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(i < 16 ? 128 : 512);
    }
    return false;
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
