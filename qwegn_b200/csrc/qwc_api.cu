// C ABI of libqwcuda.so: context, weight-view validation, the dispatch table and the matmul door.
// Host logic mirrors the reference's Swift operator layer (Sources/Operators/QWGEMM/QWGemm.swift,
// QWGemmAQ.swift, QWGemmF32.swift; Sources/Foundation/QWAlloc/QWWeightView.swift): same refusals, same order
// (every check happens before the first launch).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "qwc_common.cuh"

int qwc_launch_dequant(const qwc_hal*, cudaStream_t, const qwc_weight_view*, void*, int, int);
int qwc_launch_fwht32_f16(const qwc_hal*, cudaStream_t, void*, int64_t);
int qwc_launch_quantize(const qwc_hal*, cudaStream_t, const float*, int64_t, int64_t, int, void*);
int qwc_launch_gemv(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, int64_t, void*, int,
                    int64_t, int, int, void*, size_t);
size_t qwc_gemv_workspace_bytes(const qwc_weight_view*, int64_t);
int qwc_launch_gemv_ar(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, int64_t, void*, int,
                       int64_t, int, int, void*, size_t, const qwc_allreduce_ctx*, bool dry = false);
bool qwc_gemm_tc_supported(const qwc_hal*, const qwc_weight_view*, int64_t, int);
size_t qwc_gemm_tc_workspace_bytes(const qwc_weight_view*, int64_t, int);
int qwc_launch_gemm_tc(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, int64_t, void*, int, int64_t,
                       int, int, void*, size_t);
int qwc_gemm_tc_check(const qwc_weight_view*, const void*, int64_t, int64_t, int, const void*, size_t);
int qwc_gemv_check(const qwc_hal*, const qwc_weight_view*, const void*, int64_t, int64_t, void*, int, int64_t, int, int, void*, size_t);

static thread_local char g_err[512] = "";

int qwc_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
void qwc_clear_error() { g_err[0] = 0; }

extern "C" {

const char* qwc_last_error(void) { return g_err; }

int qwc_hal_create(int device, qwc_hal** out) {
    qwc_clear_error();
    if (!out) return qwc_fail(QWC_ERR_BAD_SHAPE, "qwc_hal_create: out is null");
    *out = nullptr;
    int count = 0;
    QWC_CUDA_TRY(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return qwc_fail(QWC_ERR_CUDA, "device %d out of range (%d visible)", device, count);
    QWC_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    QWC_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return qwc_fail(QWC_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    qwc_hal* h = new (std::nothrow) qwc_hal();
    if (!h) return qwc_fail(QWC_ERR_CUDA, "out of host memory");
    h->device = device;
    h->sm_count = prop.multiProcessorCount;
    h->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    h->encode_tiled = nullptr;
    h->static_weights = 0;
    {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            h->encode_tiled = fn;
        (void)cudaGetLastError();
    }
    cudaError_t e = cudaMalloc(&h->status, 4 * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 4 * sizeof(int32_t));
    if (e != cudaSuccess) {
        delete h;
        return qwc_fail(QWC_ERR_CUDA, "status word: %s", cudaGetErrorString(e));
    }
    *out = h;
    return QWC_OK;
}

void qwc_hal_destroy(qwc_hal* hal) {
    if (!hal) return;
    cudaFree(hal->status);
    delete hal;
}

int qwc_hal_device_status(qwc_hal* hal, int32_t* status_out) {
    qwc_clear_error();
    if (!hal || !status_out) return qwc_fail(QWC_ERR_BAD_SHAPE, "null argument");
    QWC_CUDA_TRY(cudaDeviceSynchronize());
    QWC_CUDA_TRY(cudaMemcpy(status_out, hal->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
    return QWC_OK;
}

int qwc_sm_count(const qwc_hal* hal) { return hal ? hal->sm_count : 0; }

int qwc_hal_set_static_weights(qwc_hal* hal, int32_t enabled) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    hal->static_weights = enabled != 0;
    return QWC_OK;
}

int64_t qwc_block_bytes(int32_t kind, int32_t bits, int32_t group) {
    if (kind == QWC_KIND_HQ4_G32_M5) return 20;
    if (kind == QWC_KIND_ROTATED_HQ) return static_cast<int64_t>(group) * bits / 8 + 4;
    return 0;
}

// QWWeightView.init? (QWWeightView.swift:108-152): k % group == 0 and the bank must hold n * (k/group) blocks.
int qwc_weight_view_init(qwc_weight_view* view, const void* blocks, size_t bank_bytes, int64_t n, int64_t k,
                         int32_t kind, int32_t bits, int32_t group) {
    qwc_clear_error();
    if (!view) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "view is null");
    if (kind == QWC_KIND_HQ4_G32_M5) {
        bits = 4;
        group = 32;
    } else if (kind == QWC_KIND_ROTATED_HQ) {
        const bool bits_ok = bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8;
        const bool group_ok = group == 32 || group == 64 || group == 128 || group == 256;
        if (!bits_ok || !group_ok) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "rotatedHQ(%d, %d) is not a container of the family", bits, group);
    } else {
        return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unknown container kind %d", kind);
    }
    if (n <= 0 || k <= 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "empty bank (n=%lld k=%lld)", (long long)n, (long long)k);
    if (k % group != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "k=%lld is not a multiple of group %d", (long long)k, group);
    const int64_t need = n * (k / group) * qwc_block_bytes(kind, bits, group);
    if (bank_bytes < static_cast<size_t>(need))
        return qwc_fail(QWC_ERR_BAD_WEIGHTS, "bank holds %zu bytes, view needs %lld", bank_bytes, (long long)need);
    if (!blocks) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "blocks is null");
    if (reinterpret_cast<uintptr_t>(blocks) % 4 != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "blocks must be 4-byte aligned");
    view->blocks = blocks;
    view->n = n;
    view->k = k;
    view->kind = kind;
    view->bits = bits;
    view->group = group;
    return QWC_OK;
}

// QWGemmShape.family + QWGemm.plan (QWGemm.swift:24-33, 92-133) with the live thresholds of the shipped engine
// (the families follow the reference: GEMV at M = 1, batched verify for 2 <= M < 16, tensor GEMM from 16 tokens on,
// QWGemmF32.swift:413-440; the backend is this library's: the tensor-core kernel from 9 tokens on, 8 for HQ8_G32).
int qwc_gemm_plan(int64_t m, int64_t n, int64_t k, int32_t kind, int32_t bits, int32_t group, int32_t epilogue,
                  int64_t vocab, qwc_plan* out) {
    qwc_clear_error();
    if (!out) return qwc_fail(QWC_ERR_BAD_SHAPE, "plan out is null");
    memset(out, 0, sizeof(*out));
    if (m <= 0 || n <= 0 || k <= 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "m, n, k must be positive");
    int fam;
    if (m == 1 && vocab > 0 && n == vocab) fam = QWC_FAMILY_F2_LMHEAD_GEMV;
    else if (m == 1) fam = QWC_FAMILY_F1_DECODE_GEMV;
    else if (m >= 512) fam = QWC_FAMILY_F3_PREFILL_GEMM;
    else if (m <= 8) fam = QWC_FAMILY_F5_SKINNY_GEMM;
    else fam = QWC_FAMILY_F4_BLOCKED_GEMM;
    out->family = fam;
    out->epilogue = epilogue;
    qwc_weight_view v{nullptr, n, k, kind, bits, group};
    if (kind == QWC_KIND_HQ4_G32_M5) { v.bits = 4; v.group = 32; }
    const int fmt = qwc_fmt_of(v);
    if (fmt == FMT_UNSUPPORTED || k % v.group != 0 || epilogue < QWC_EPI_NONE || epilogue > QWC_EPI_SILU_PAIR_FWHT) {
        out->backend = QWC_BACKEND_BLOCKED;
        return QWC_OK;
    }
    const int64_t row_bytes = (k / v.group) * qwc_block_bytes(v.kind, v.bits, v.group);
    const char* fname = fmt == FMT_HQ4_G32_M5 ? "hq4g32m5" : (fmt == FMT_HQ8_G32 ? "hq8g32" : "hq4g64");
    if (row_bytes % 16 != 0) {
        out->backend = QWC_BACKEND_ROWWISE;
        out->threads_per_cta = 256;
        snprintf(out->kernel, sizeof(out->kernel), "qwc_gemv_rowwise_%s", fname);
    } else if (m >= qwc_tc_min_tokens(fmt) && (epilogue == QWC_EPI_NONE || (n % 2 == 0 && (n / 2) % 64 == 0)) && k % (fmt == FMT_HQ4_G64 ? 256 : 128) == 0) {
        out->backend = QWC_BACKEND_TCGEN05;
        out->threads_per_cta = 24 * 32;
        snprintf(out->kernel, sizeof(out->kernel), "qwc_gemm_ts_%s_128x%dx64", fname, m <= 64 ? 64 : (m <= 128 ? 128 : 192));
    } else {
        out->backend = QWC_BACKEND_STREAM_MMA;
        out->threads_per_cta = 17 * 32;
        snprintf(out->kernel, sizeof(out->kernel), "qwc_gemv_stream_%s_m%d", fname, m <= 8 ? 8 : 16);
    }
    return QWC_OK;
}

int qwc_fwht32_f16(qwc_hal* hal, qwc_stream stream, void* x_f16, int64_t count) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (count < 0 || count % 32 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "count=%lld is not a multiple of 32", (long long)count);
    if (count > 0 && !x_f16) return qwc_fail(QWC_ERR_BAD_SHAPE, "x is null");
    return qwc_launch_fwht32_f16(hal, static_cast<cudaStream_t>(stream), x_f16, count);
}

}  // extern "C"

// Library-internal (C++ linkage, declared in qwc_common.cuh).
int qwc_check_view(const qwc_weight_view* w) {
    if (!w || !w->blocks) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "weight view is null");
    if (w->n <= 0 || w->k <= 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "empty weight view");
    if (qwc_fmt_of(*w) == FMT_UNSUPPORTED)
        return qwc_fail(QWC_ERR_BAD_WEIGHTS, "no kernel for container kind %d bits %d group %d (supported: HQ4_G32_M5, HQ8_G32, HQ4_G64)",
                        w->kind, w->bits, w->group);
    if (w->k % w->group != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "k=%lld is not a multiple of group %d", (long long)w->k, w->group);
    if (reinterpret_cast<uintptr_t>(w->blocks) % 4 != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "blocks must be 4-byte aligned");
    if (w->n >= (int64_t(1) << 31) || w->k >= (int64_t(1) << 31)) return qwc_fail(QWC_ERR_BAD_SHAPE, "n, k must fit 31 bits");
    return QWC_OK;
}

extern "C" {

int qwc_dequant(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, void* out, int32_t out_dtype,
                int32_t standard_domain) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (int rc = qwc_check_view(w)) return rc;
    if (!out) return qwc_fail(QWC_ERR_BAD_SHAPE, "out is null");
    if (out_dtype != QWC_F16 && out_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "out dtype must be f16 or f32");
    return qwc_launch_dequant(hal, static_cast<cudaStream_t>(stream), w, out, out_dtype, standard_domain);
}

int qwc_quantize(qwc_hal* hal, qwc_stream stream, const float* w_f32, int64_t n, int64_t k, int32_t kind, int32_t bits,
                 int32_t group, void* blocks_out) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    qwc_weight_view v{blocks_out, n, k, kind, bits, group};
    if (kind == QWC_KIND_HQ4_G32_M5) { v.bits = 4; v.group = 32; }
    if (int rc = qwc_check_view(&v)) return rc;
    if (!w_f32) return qwc_fail(QWC_ERR_BAD_SHAPE, "w is null");
    return qwc_launch_quantize(hal, static_cast<cudaStream_t>(stream), w_f32, n, k, qwc_fmt_of(v), blocks_out);
}

size_t qwc_gemm_workspace_bytes(const qwc_hal* hal, const qwc_weight_view* w, int64_t m, int32_t epilogue,
                                int32_t x_is_rotated) {
    if (!hal || !w || w->k <= 0 || w->group <= 0 || qwc_fmt_of(*w) == FMT_UNSUPPORTED) return 0;
    if (qwc_gemm_tc_supported(hal, w, m, epilogue)) return qwc_gemm_tc_workspace_bytes(w, m, x_is_rotated);
    return qwc_gemv_workspace_bytes(w, m);
}

}  // extern "C"

// Every argument check of the matmul door in one place, shared by qwc_gemm, qwc_gemm_static_scratch and qwc_gemm_f32 so
// that none of them can drift: QWC_OK means that a launch with these arguments cannot be refused any more.  The order
// follows QWGemm.encode (QWGemm.swift:135-283): weights, shape, geometry, then scratch.
static int gemm_args_common(const qwc_hal* hal, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx, void* y,
                            int32_t y_dtype, int64_t ldy, int32_t epilogue) {
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (int rc = qwc_check_view(w)) return rc;
    if (m < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "m=%lld is negative", (long long)m);
    if (m == 0) return QWC_OK;
    if (!x_f16 || !y) return qwc_fail(QWC_ERR_BAD_SHAPE, "x or y is null");
    if (y_dtype != QWC_F16 && y_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "y dtype must be f16 or f32");
    if (epilogue < QWC_EPI_NONE || epilogue > QWC_EPI_SILU_PAIR_FWHT) return qwc_fail(QWC_ERR_BAD_SHAPE, "unknown epilogue %d", epilogue);
    int64_t n_out = w->n;
    if (epilogue != QWC_EPI_NONE) {
        // QWGemm.encode refuses an odd packed gate||up bank (QWGemm.swift:135-283: badWeights).
        if (w->n % 2 != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "silu-pair needs an even row count, got n=%lld", (long long)w->n);
        n_out = w->n / 2;
        if (epilogue == QWC_EPI_SILU_PAIR_FWHT && n_out % 32 != 0)
            return qwc_fail(QWC_ERR_BAD_GEOMETRY, "fused FWHT needs n/2 %% 32 == 0, got %lld", (long long)n_out);
    }
    if (ldx < w->k) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx=%lld < k=%lld", (long long)ldx, (long long)w->k);
    if (ldy < n_out) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldy=%lld < output width %lld", (long long)ldy, (long long)n_out);
    if (reinterpret_cast<uintptr_t>(x_f16) % 2 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "x must be 2-byte aligned");
    if (reinterpret_cast<uintptr_t>(y) % (y_dtype == QWC_F16 ? 2 : 4) != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "y is not aligned to its element size");
    return QWC_OK;
}

int qwc_gemm_check(const qwc_hal* hal, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx, void* y,
                   int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace, size_t workspace_bytes) {
    if (int rc = gemm_args_common(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue)) return rc;
    if (m == 0) return QWC_OK;
    if (qwc_gemm_tc_supported(hal, w, m, epilogue)) return qwc_gemm_tc_check(w, x_f16, ldx, m, x_is_rotated, workspace, workspace_bytes);
    return qwc_gemv_check(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, workspace, workspace_bytes);
}

// The same for a caller that always takes the streaming kernel (the scratch-free door).
int qwc_gemm_args_check_stream(const qwc_hal* hal, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx, void* y,
                               int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace,
                               size_t workspace_bytes) {
    if (int rc = gemm_args_common(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue)) return rc;
    if (m == 0) return QWC_OK;
    return qwc_gemv_check(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, workspace, workspace_bytes);
}

extern "C" {

int qwc_gemm(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx,
             void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace,
             size_t workspace_bytes) {
    qwc_clear_error();
    if (int rc = qwc_gemm_check(hal, w, x_f16, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, workspace, workspace_bytes)) return rc;
    if (m == 0) return QWC_OK;
    if (qwc_gemm_tc_supported(hal, w, m, epilogue))
        return qwc_launch_gemm_tc(hal, static_cast<cudaStream_t>(stream), w, x_f16, m, ldx, y, y_dtype, ldy, epilogue,
                                  x_is_rotated, workspace, workspace_bytes);
    return qwc_launch_gemv(hal, static_cast<cudaStream_t>(stream), w, x_f16, m, ldx, y, y_dtype, ldy, epilogue,
                           x_is_rotated, workspace, workspace_bytes);
}

int qwc_gemm_allreduce(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx,
                       void* y, int32_t y_dtype, int64_t ldy, int32_t x_is_rotated, const qwc_allreduce_ctx* ctx) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (int rc = qwc_check_view(w)) return rc;
    if (!ctx) return qwc_fail(QWC_ERR_BAD_SHAPE, "all-reduce context is null");
    if (ctx->world < 2 || ctx->world > 8 || ctx->rank < 0 || ctx->rank >= ctx->world)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "rank %d / world %d: the fused form takes 2..8 ranks", ctx->rank, ctx->world);
    if (m <= 0) return m == 0 ? QWC_OK : qwc_fail(QWC_ERR_BAD_SHAPE, "m is negative");
    if (!x_f16 || !y) return qwc_fail(QWC_ERR_BAD_SHAPE, "x or y is null");
    if (y_dtype != QWC_F16 && y_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "y dtype must be f16 or f32");
    if (ldx < w->k || ldy < w->n) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx / ldy too small");
    const int64_t row_bytes = (w->k / w->group) * qwc_block_bytes(w->kind, w->bits, w->group);
    if (m > 8 || row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(w->blocks) % 16 != 0 || qwc_gemv_workspace_bytes(w, m) != 0)
        return qwc_fail(QWC_ERR_BLOCKED, "the fused all-reduce takes m <= 8, 16-byte bank rows and one K slice");
    for (int r = 0; r < ctx->world; ++r)
        if (!ctx->inbox[r] || reinterpret_cast<uintptr_t>(ctx->inbox[r]) % 8 != 0)
            return qwc_fail(QWC_ERR_BAD_SHAPE, "inbox %d is null or not 8-byte aligned", r);
    if (ctx->inbox_floats < 2 * static_cast<int64_t>(ctx->world) * m * w->n || ctx->inbox_floats % 2 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "inbox too small: an even number of at least %lld floats is needed (two per slot)",
                        (long long)(2 * static_cast<int64_t>(ctx->world) * m * w->n));
    if (ctx->epoch_state == nullptr && ctx->epoch == 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "call number 0 marks an empty slot: count from 1");
    return qwc_launch_gemv_ar(hal, static_cast<cudaStream_t>(stream), w, x_f16, m, ldx, y, y_dtype, ldy, QWC_EPI_NONE, x_is_rotated,
                              nullptr, 0, ctx);
}

// ---- peer-visible device memory (load-time helpers of the tensor- and expert-parallel doors) -------------------------
// One process drives one GPU; the fused collectives store into the other ranks' buffers directly.  A rank allocates its
// buffer here, hands the 64-byte handle to its peers by whatever channel the host has (the Python mirror uses
// torch.distributed), and every peer maps it.  Allocation and mapping happen once, before the first encode call.
int qwc_peer_alloc(qwc_hal* hal, size_t bytes, void** ptr_out, void* handle_out_64) {
    qwc_clear_error();
    if (!hal || !ptr_out || !handle_out_64 || bytes == 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "qwc_peer_alloc: bad argument");
    *ptr_out = nullptr;
    QWC_CUDA_TRY(cudaSetDevice(hal->device));
    void* p = nullptr;
    QWC_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return qwc_fail(QWC_ERR_CUDA, "qwc_peer_alloc: %s", cudaGetErrorString(e));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    memcpy(handle_out_64, &h, 64);
    *ptr_out = p;
    return QWC_OK;
}

int qwc_peer_open(qwc_hal* hal, const void* handle_64, void** ptr_out) {
    qwc_clear_error();
    if (!hal || !handle_64 || !ptr_out) return qwc_fail(QWC_ERR_BAD_SHAPE, "qwc_peer_open: bad argument");
    QWC_CUDA_TRY(cudaSetDevice(hal->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64, 64);
    QWC_CUDA_TRY(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return QWC_OK;
}

int qwc_peer_close(qwc_hal* hal, void* ptr) {
    qwc_clear_error();
    if (!hal || !ptr) return QWC_OK;
    QWC_CUDA_TRY(cudaSetDevice(hal->device));
    QWC_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return QWC_OK;
}

int qwc_peer_free(qwc_hal* hal, void* ptr) {
    qwc_clear_error();
    if (!hal || !ptr) return QWC_OK;
    QWC_CUDA_TRY(cudaSetDevice(hal->device));
    QWC_CUDA_TRY(cudaFree(ptr));
    return QWC_OK;
}

}  // extern "C"
