// The f32-activation matmul door: the CUDA twin of the reference's encodeHQ4F32V4 / encodeHQ4F32BM
// (Sources/Operators/QWGEMM/QWGemmF32.swift:143-199, 309-350; kernel bodies
// Sources/QWMetal/include/qw_gemm_f32_common.metalh:15-29, 59-225) and of its f32 rotation encodeH32F32
// (QWGemmF32.swift:46-54).  Activations arrive as f32 rows in the rotated (Walsh-Hadamard) basis -- or in the standard
// basis, then they are rotated here in f32 -- and are rounded ONCE to f16 for the tensor-core dot products (the
// weights decode to f16-exact values, accumulation is f32).  The elementwise epilogues of the reference's f32 GEMV
// (0 none, 1 silu(y/scale), 2 sigmoid(y), 3 silu(y/scale) then FWHT-32 along n) run as one small kernel after the
// matmul.  Three launches at most: stage, matmul, epilogue.
#include "qwc_common.cuh"

namespace {

// 8 consecutive f32 per thread; a quad of threads holds one aligned 32-element block.
__global__ void __launch_bounds__(256) qwc_f32_stage_kernel(const float* __restrict__ x, int64_t ldx, __half* __restrict__ y,
                                                            int k8, int64_t total, int rotate) {
    const int lane = threadIdx.x & 31, t4 = lane & 3;
    // Let a matmul launched with programmatic stream serialization start its weight prefetch now; it still waits for
    // this whole grid (and its stores) before it reads the staged activations.  A no-op for ordinary launches.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // When this kernel was itself launched that way: wait for the grid before it (which may have produced x, or may
    // still be reading the staging buffer of the previous call).  Returns at once for an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the loop bound is per warp (i - lane), so that all 32 lanes reach the shuffles together
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i - lane < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const bool ok = i < total;
        const int64_t row = ok ? i / k8 : 0;
        const int c = ok ? static_cast<int>(i - row * k8) : 0;
        const float4* src = reinterpret_cast<const float4*>(x + row * ldx + static_cast<int64_t>(c) * 8);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (ok) { a = src[0]; b = src[1]; }
        float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (rotate) {
#pragma unroll
            for (int hh = 1; hh < 8; hh <<= 1)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((j & hh) == 0) {
                        const float u = f[j], v = f[j + hh];
                        f[j] = __fadd_rn(u, v);
                        f[j + hh] = __fsub_rn(u, v);
                    }
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = fwht_xor_stage(f[j], 1, (t4 & 1) != 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = fwht_xor_stage(f[j], 2, (t4 & 2) != 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(f[j], qwc_inv_sqrt32());
        }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        if (ok) reinterpret_cast<uint4*>(y)[i] = o;
    }
}

// y[r, c] = epi(t[r, c]): 1 silu(t/scale), 2 sigmoid(t), 3 silu(t/scale) then FWHT-32 along c (one warp per aligned
// 32 columns; n % 32 == 0 then).  qwg_apply_v4_epi_f32 and the BM epilogue, qw_gemm_f32_common.metalh:15-20, 131-133.
template <typename OutT>
__global__ void __launch_bounds__(256) qwc_f32_epilogue_kernel(const float* __restrict__ t, int64_t ldt, OutT* __restrict__ y,
                                                               int64_t ldy, int n, int64_t total, int epi, float scale) {
    const int lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // as in the stage kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i - lane < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const bool ok = i < total;
        const int64_t row = ok ? i / n : 0;
        const int c = ok ? static_cast<int>(i - row * n) : 0;
        float v = ok ? t[row * ldt + c] : 0.0f;
        if (epi == 1 || epi == 3) {
            const float z = v / scale;
            v = z / (1.0f + expf(-z));
        } else if (epi == 2) {
            v = 1.0f / (1.0f + expf(-v));
        }
        if (epi == 3) {
#pragma unroll
            for (int msk = 1; msk < 32; msk <<= 1) v = fwht_xor_stage(v, msk, (lane & msk) != 0);
            v = __fmul_rn(v, qwc_inv_sqrt32());
        }
        if (ok) {
            if constexpr (sizeof(OutT) == 2) y[row * ldy + c] = __float2half_rn(v);
            else y[row * ldy + c] = v;
        }
    }
}

size_t f32_align(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace

// Workspace: [x as f16, m * k][f32 matmul output m * n when an epilogue follows][the f16 door's own workspace].
extern "C" size_t qwc_gemm_f32_workspace_bytes(const qwc_hal* hal, const qwc_weight_view* w, int64_t m, int32_t epilogue) {
    if (!hal || !w || m <= 0) return 0;
    size_t b = f32_align(static_cast<size_t>(m) * w->k * 2);
    if (epilogue != 0) b += f32_align(static_cast<size_t>(m) * w->n * 4);
    return b + qwc_gemm_workspace_bytes(hal, w, m, QWC_EPI_NONE, 1);
}

extern "C" int qwc_gemm_f32(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const float* x_f32, int64_t m,
                            int64_t ldx, void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, float scale,
                            int32_t x_is_rotated, void* workspace, size_t workspace_bytes) {
    qwc_clear_error();
    if (!hal || !w) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal or weight view is null");
    if (int rc0 = qwc_check_view(w)) return rc0;
    if (m <= 0 || !x_f32 || !y) return qwc_fail(QWC_ERR_BAD_SHAPE, "f32 matmul: m=%lld and the buffers must be non-null", (long long)m);
    if (epilogue < 0 || epilogue > 3) return qwc_fail(QWC_ERR_BAD_SHAPE, "f32 matmul: epilogue %d (0 none, 1 silu, 2 sigmoid, 3 silu+fwht)", epilogue);
    if (y_dtype != QWC_F16 && y_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "y must be f16 or f32");
    if (w->k % 32 != 0 || ldx < w->k || ldx % 4 != 0 || reinterpret_cast<uintptr_t>(x_f32) % 16 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "f32 matmul: K %% 32 == 0 and 16-byte aligned x rows required");
    if (ldy < w->n) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldy=%lld < n", (long long)ldy);
    if (epilogue == 3 && w->n % 32 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "silu+fwht epilogue needs n %% 32 == 0");   // QWGemmF32.swift:86
    if ((epilogue == 1 || epilogue == 3) && !(scale != 0.0f)) return qwc_fail(QWC_ERR_BAD_SHAPE, "silu epilogue needs a non-zero scale");
    const size_t need = qwc_gemm_f32_workspace_bytes(hal, w, m, epilogue);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "f32 matmul workspace: %zu bytes (256-byte aligned) needed, %zu given", need, workspace_bytes);
    auto st = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    __half* x16 = reinterpret_cast<__half*>(ws);
    size_t off = f32_align(static_cast<size_t>(m) * w->k * 2);
    float* tmp = nullptr;
    if (epilogue != 0) { tmp = reinterpret_cast<float*>(ws + off); off += f32_align(static_cast<size_t>(m) * w->n * 4); }
    // every refusal of the f16 door (weight view, geometry, its share of the workspace) before the stage kernel runs
    if (int rc0 = qwc_gemm_check(hal, w, x16, m, w->k, epilogue == 0 ? y : static_cast<void*>(tmp), epilogue == 0 ? y_dtype : QWC_F32,
                                 epilogue == 0 ? ldy : w->n, QWC_EPI_NONE, 1, ws + off, workspace_bytes - off))
        return rc0;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    {
        const int k8 = static_cast<int>(w->k / 8);
        const int64_t total = m * k8;
        int64_t blocks = (total + 255) / 256;
        if (blocks > cap) blocks = cap;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(blocks));
        cfg.blockDim = dim3(256);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = hal->static_weights ? 1 : 0;   // the decode-loop promise: kernels may be launched ahead of their predecessors' end
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_f32_stage_kernel, x_f32, ldx, x16, k8, total, x_is_rotated ? 0 : 1));
    }
    int rc;
    if (epilogue == 0) rc = qwc_gemm(hal, stream, w, x16, m, w->k, y, y_dtype, ldy, QWC_EPI_NONE, 1, ws + off, workspace_bytes - off);
    else rc = qwc_gemm(hal, stream, w, x16, m, w->k, tmp, QWC_F32, w->n, QWC_EPI_NONE, 1, ws + off, workspace_bytes - off);
    if (rc != QWC_OK || epilogue == 0) return rc;
    const int64_t total = m * w->n;
    int64_t blocks = (total + 255) / 256;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = hal->static_weights ? 1 : 0;
    const float* tmp_c = tmp;
    const int64_t ldt = w->n;
    const int n_i = static_cast<int>(w->n);
    if (y_dtype == QWC_F16)
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_f32_epilogue_kernel<__half>, tmp_c, ldt, static_cast<__half*>(y), ldy, n_i, total,
                                        static_cast<int>(epilogue), scale));
    else
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_f32_epilogue_kernel<float>, tmp_c, ldt, static_cast<float*>(y), ldy, n_i, total,
                                        static_cast<int>(epilogue), scale));
    return QWC_OK;
}
