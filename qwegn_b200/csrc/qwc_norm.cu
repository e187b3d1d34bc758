// RMSNorm with the rotated (Walsh-Hadamard) f16 output the quantized matmuls consume: the CUDA twin of the
// reference's qwg_rmsnorm / qwg_rmsnorm_residual (Sources/QWMetal/mlp_norm_rope/qwnorm.metal:27-79, 249-259; host
// doors encodeRMSNormFast / encodeRMSNormResidualFast, Sources/Runtime/QWEngine/Driver/EncodeKernels.swift:339-404).
//   y = f16( fwht32( s * rsqrt(mean(s^2) + eps) * (1 + gamma) ) ),   s = x, or s = f16(x + residual) (stored back)
// f32 sum of squares, f32 products, f32 butterflies, one rounding to f16 at the store ("plus-one law": gamma is stored
// raw).  This is the step before every GEMM of the reference's engine: with it the matmuls are called with
// x_is_rotated = 1 and do not rotate activations themselves.
#include "qwc_common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace {

// One CTA per row; thread t owns the 16-byte chunks t, t + T, ... (8 halves each).  A quad of consecutive threads
// holds one aligned 32-element block, so the FWHT-32 is three in-lane butterfly stages plus two xor-shuffle stages.
constexpr int kNormMaxChunks = 4;   // chunks kept in registers per thread (hidden <= 8 * 4 * blockDim)

__global__ void __launch_bounds__(1024) qwc_rmsnorm_fwht_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma,
                                                                __half* __restrict__ y, __half* residual, int hidden, float eps,
                                                                int rotate) {
    __shared__ float s_part[32];
    __shared__ float s_rstd;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int chunks = hidden / 8;
    const int64_t row = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
    uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * hidden) : nullptr;
    uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);
    const uint4* gr = reinterpret_cast<const uint4*>(gamma);

    uint4 reg[kNormMaxChunks];
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
        const int u = tid + i * nthreads;
        if (u < chunks) {
            uint4 v = xr[u];
            if (rr) {
                const uint4 r = rr[u];
                __half2* a = reinterpret_cast<__half2*>(&v);
                const __half2* b = reinterpret_cast<const __half2*>(&r);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fa = __half22float2(a[j]), fb = __half22float2(b[j]);
                    a[j] = __floats2half2_rn(__fadd_rn(fa.x, fb.x), __fadd_rn(fa.y, fb.y));
                }
                rr[u] = v;   // residual += x, kept in f16 as the reference does
            }
            reg[i] = v;
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                acc = fmaf(f.x, f.x, acc);
                acc = fmaf(f.y, f.y, acc);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) s_part[warp] = acc;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (nthreads >> 5) ? s_part[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        if (lane == 0) s_rstd = rsqrtf(t / static_cast<float>(hidden) + eps);
    }
    __syncthreads();
    const float rstd = s_rstd;
    const int t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
        const int u = tid + i * nthreads;
        if (u < chunks) {   // uniform per warp: chunks and nthreads are multiples of 32
            const uint4 g = gr[u];
            const __half2* h = reinterpret_cast<const __half2*>(&reg[i]);
            const __half2* gh = reinterpret_cast<const __half2*>(&g);
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fv = __half22float2(h[j]), gv = __half22float2(gh[j]);
                f[2 * j] = __fmul_rn(__fmul_rn(fv.x, rstd), __fadd_rn(gv.x, 1.0f));
                f[2 * j + 1] = __fmul_rn(__fmul_rn(fv.y, rstd), __fadd_rn(gv.y, 1.0f));
            }
            if (rotate) {
#pragma unroll
                for (int hh = 1; hh < 8; hh <<= 1)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if ((j & hh) == 0) {
                            const float a = f[j], b = f[j + hh];
                            f[j] = __fadd_rn(a, b);
                            f[j + hh] = __fsub_rn(a, b);
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
            yr[u] = o;
        }
    }
}

// The explicit f32 -> f16 cast seam between the f32-emitting GEMV doors and the f16 engine storage
// (QWGemm.encodeCast, Sources/Operators/QWGEMM/QWGemm.swift:302-320): 8 elements per thread, round to nearest even.
__global__ void __launch_bounds__(256) qwc_cast_f32_to_f16_kernel(const float4* __restrict__ x, uint4* __restrict__ y, int64_t n8) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const float4 a = x[2 * i], b = x[2 * i + 1];
        uint4 o;
        __half2* h = reinterpret_cast<__half2*>(&o);
        h[0] = __floats2half2_rn(a.x, a.y);
        h[1] = __floats2half2_rn(a.z, a.w);
        h[2] = __floats2half2_rn(b.x, b.y);
        h[3] = __floats2half2_rn(b.z, b.w);
        y[i] = o;
    }
}

// Greedy head: token[row] = argmax over the vocabulary of logits[row, :] with the reference's key order
// (qwg_gemv_am_fold4 / qwg_head_argmax_fin: Sources/QWMetal/include/qw_gemm_f32_common.metalh:31-57,
// Sources/QWMetal/head_sampling/qwhead.metal:241-270; qw_sortable_f32_u32, include/qw_fastmath_safe.metalh:21-25):
// key = (sortable(value), ~column): NaN sorts lowest, +0 above -0, ties go to the lower column.
__device__ __forceinline__ uint32_t sortable_f32(float x) {
    const uint32_t u = __float_as_uint(x);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0u;
    return (u & 0x80000000u) ? ~u : (u ^ 0x80000000u);
}

// A cluster of kArgmaxCluster CTAs shares one row: CTA r scans columns [r * per, (r + 1) * per), the winners meet in
// the shared memory of CTA 0 of the cluster (distributed shared memory), which writes the token.
constexpr int kArgmaxCluster = 8;

__global__ void __launch_bounds__(1024) qwc_head_argmax_kernel(const float* __restrict__ logits, int64_t ld, int n_total,
                                                               int32_t* __restrict__ tokens) {
    __shared__ unsigned long long s_best[32];
    __shared__ unsigned long long s_cluster[kArgmaxCluster];
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = static_cast<int>(cluster.block_rank());
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + static_cast<int64_t>(blockIdx.y) * ld;
    const int per = (((n_total + kArgmaxCluster - 1) / kArgmaxCluster) + 3) & ~3;
    const int lo = min(n_total, crank * per), n = min(n_total, lo + per);
    unsigned long long best = 0ull;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    int c0 = lo;
    if (vec) {
        const int n4 = lo + ((n - lo) & ~3);
        for (int c = lo + tid * 4; c < n4; c += 4096) {
            const float4 v = *reinterpret_cast<const float4*>(row + c);
            const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const unsigned long long key = (static_cast<unsigned long long>(sortable_f32(f[i])) << 32) | static_cast<uint32_t>(~(c + i));
                best = key > best ? key : best;
            }
        }
        c0 = n4;
    }
    for (int c = c0 + tid; c < n; c += 1024) {
        const unsigned long long key = (static_cast<unsigned long long>(sortable_f32(row[c])) << 32) | static_cast<uint32_t>(~c);
        best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) s_best[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = s_best[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            best = other > best ? other : best;
        }
    }
    // Distributed shared memory may only be touched once the target CTA is known to be running: every CTA of the
    // cluster meets here first (with a short vocabulary the other ranks would otherwise reach the store at once).
    cluster.sync();
    if (warp == 0 && lane == 0) *cluster.map_shared_rank(&s_cluster[crank], 0) = best;
    cluster.sync();
    if (crank == 0 && tid == 0) {
        best = s_cluster[0];
#pragma unroll
        for (int r = 1; r < kArgmaxCluster; ++r) best = s_cluster[r] > best ? s_cluster[r] : best;
        tokens[blockIdx.y] = static_cast<int32_t>(~static_cast<uint32_t>(best & 0xFFFFFFFFull));
    }
}

}  // namespace

extern "C" int qwc_cast_f32_to_f16(qwc_hal* hal, qwc_stream stream, const float* x_f32, void* y_f16, int64_t count) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    // QWGemm.swift:308-311: the count must be positive and divide 8 (badWeights there)
    if (count <= 0 || count % 8 != 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "cast f32->f16: n=%lld must be positive and divide 8", (long long)count);
    if (!x_f32 || !y_f16) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    if ((reinterpret_cast<uintptr_t>(x_f32) | reinterpret_cast<uintptr_t>(y_f16)) % 16 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "buffers must be 16-byte aligned");
    const int64_t n8 = count / 8;
    int64_t blocks = (n8 + 255) / 256;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    qwc_cast_f32_to_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(x_f32), static_cast<uint4*>(y_f16), n8);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

extern "C" int qwc_head_argmax(qwc_hal* hal, qwc_stream stream, const float* logits, int64_t ld, int64_t rows, int64_t n,
                               int32_t* tokens) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (n <= 0 || n >= (int64_t(1) << 31) || ld < n) return qwc_fail(QWC_ERR_BAD_SHAPE, "bad vocabulary extent n=%lld ld=%lld", (long long)n, (long long)ld);
    if (rows < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "rows is negative");
    if (rows == 0) return QWC_OK;
    if (!logits || !tokens) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kArgmaxCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    for (int64_t r0 = 0; r0 < rows; r0 += 32768) {   // grid.y carries the rows
        const int64_t r = rows - r0 < 32768 ? rows - r0 : 32768;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kArgmaxCluster, static_cast<unsigned>(r), 1);
        cfg.blockDim = dim3(1024, 1, 1);
        cfg.stream = static_cast<cudaStream_t>(stream);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_head_argmax_kernel, logits + r0 * ld, ld, static_cast<int>(n), tokens + r0));
    }
    return QWC_OK;
}

extern "C" int qwc_rmsnorm_fwht(qwc_hal* hal, qwc_stream stream, const void* x_f16, const void* gamma_f16, void* y_f16,
                                void* residual_f16, int64_t rows, int64_t hidden, float eps, int32_t rotate) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    // the norm family's contract (EncodeKernels.swift:350-357): rows of 16-byte chunks rotating in groups of 32 halves
    if (hidden <= 0 || hidden % 256 != 0)
        return qwc_fail(QWC_ERR_BAD_GEOMETRY, "the norm family needs a hidden that is a multiple of 256, got %lld", (long long)hidden);
    if (hidden > 8 * kNormMaxChunks * 1024) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "hidden=%lld is above %d", (long long)hidden, 8 * kNormMaxChunks * 1024);
    if (rows < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "rows is negative");
    if (rows == 0) return QWC_OK;
    if (!x_f16 || !gamma_f16 || !y_f16) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    if ((reinterpret_cast<uintptr_t>(x_f16) | reinterpret_cast<uintptr_t>(gamma_f16) | reinterpret_cast<uintptr_t>(y_f16) |
         reinterpret_cast<uintptr_t>(residual_f16)) % 16 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "buffers must be 16-byte aligned");
    const int chunks = static_cast<int>(hidden / 8);
    int threads = (chunks + kNormMaxChunks - 1) / kNormMaxChunks;
    threads = ((threads + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    // more threads than strictly needed (up to one chunk per thread) shorten a row's latency at decode
    while (threads * 2 <= chunks && threads * 2 <= 1024) threads *= 2;
    qwc_rmsnorm_fwht_kernel<<<static_cast<unsigned>(rows), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x_f16), static_cast<const __half*>(gamma_f16), static_cast<__half*>(y_f16),
        static_cast<__half*>(residual_f16), static_cast<int>(hidden), eps, rotate);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}
