// qwc_gemm_static_scratch: the decode / verify matmul door for callers that cannot hand the library a scratch
// buffer.
//
// Some hosts of this library are not allowed to allocate device memory at the point where they call it: an operator
// plugged into an engine whose arena was sized and frozen at load time (the reference's own rule is that nothing on
// the per-token path allocates), a thread that must not take the device-wide synchronisation cudaMalloc can imply,
// or code running under a memory budget that was fully handed out before the first token.  For the one case where
// the small-M door needs scratch (9..16 tokens whose staged activations do not fit in shared memory, so K is
// processed in slices and the raw f32 sums are carried between the slices), this entry point supplies that scratch
// itself from a fixed array that lives in the library's device image.
//
// The array is a file-scope __device__ array of kScratchBytes (2 MiB): every GPU that loads the library holds it
// until the process exits.  Host code must not pass the array's name to a kernel (on the host the name is only a
// handle of the symbol); the device address is looked up once per device with cudaGetSymbolAddress, with that device
// current, and that pointer is what the kernel receives.
//
// Rules for callers:
//  * The first call on a device performs the address lookup.  Make that first call outside any stream capture.
//  * The device of `hal` must be current on the calling thread.
//  * A call whose scratch need exceeds 2 MiB (tokens x weight rows x 4 bytes) is refused with QWC_ERR_BAD_SHAPE.
//  * All calls on a device share the one array and it keeps whatever the previous call left in it.  Nothing needs
//    clearing: the first K slice of a call overwrites every element a later slice reads.  Two calls that may run on
//    the GPU at the same time (different streams, or different threads) would overwrite each other's sums: run them
//    on one stream or order them yourself.
//  * This entry point calls no cudaMalloc, cudaFree or other allocating routine.
#include <mutex>

#include "qwc_common.cuh"

int qwc_launch_gemv(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, int64_t, void*, int, int64_t,
                    int, int, void*, size_t);
size_t qwc_gemv_workspace_bytes(const qwc_weight_view*, int64_t);

namespace {

constexpr size_t kScratchBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device (looked up once per device).
int scratch_address(const qwc_hal* hal, void** out) {
    if (hal->device < 0 || hal->device >= kMaxDevices) return qwc_fail(QWC_ERR_CUDA, "device index %d is out of range", hal->device);
    int current = -1;
    QWC_CUDA_TRY(cudaGetDevice(&current));
    if (current != hal->device)
        return qwc_fail(QWC_ERR_CUDA, "device %d must be current on this thread (device %d is)", hal->device, current);
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_ptr[hal->device] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return qwc_fail(QWC_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        g_scratch_ptr[hal->device] = p;
    }
    *out = g_scratch_ptr[hal->device];
    return QWC_OK;
}

}  // namespace

extern "C" {

size_t qwc_static_scratch_capacity(void) { return kScratchBytes; }

int qwc_gemm_static_scratch(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const void* x_f16, int64_t m,
                            int64_t ldx, void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (m < 0 || m > 16) return qwc_fail(QWC_ERR_BAD_SHAPE, "this door serves 0..16 tokens, got m=%lld", (long long)m);
    if (int rc = qwc_check_view(w)) return rc;
    const size_t need = qwc_gemv_workspace_bytes(w, m);
    if (need > kScratchBytes)
        return qwc_fail(QWC_ERR_BAD_SHAPE,
                        "this call needs %zu bytes of scratch (tokens x weight rows x 4) but the built-in scratch holds %zu; "
                        "use qwc_gemm with a caller workspace",
                        need, kScratchBytes);
    void* scratch = nullptr;
    if (int rc = scratch_address(hal, &scratch)) return rc;
    // the same argument checks as qwc_gemm's streaming path, with the built-in array as the workspace
    if (int rc = qwc_gemm_args_check_stream(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, scratch, kScratchBytes)) return rc;
    if (m == 0) return QWC_OK;
    return qwc_launch_gemv(hal, static_cast<cudaStream_t>(stream), w, x_f16, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated,
                           scratch, kScratchBytes);
}

}  // extern "C"
