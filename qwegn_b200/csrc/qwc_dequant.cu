// Block decode (bit-exact with the reference's host decode) and the activation-side FWHT-32.
//
// Decode arithmetic follows Scripts/quantize/hq4.py:131-153 and hq_blocks.py:521-541 of the reference:
// HQ4_G32_M5 is (q + 1024) * scale, then + bias (the product is exact in f32, so two roundings equal the
// reference's separate multiply and add); rotatedHQ is q * scale + bias.  __fmul_rn/__fadd_rn forbid contraction.
#include "qwc_common.cuh"

namespace {

// One warp decodes one 32-element unit; lane = element index inside the unit.
template <int FMT>
__device__ __forceinline__ float decode_element(const uint8_t* __restrict__ row, int64_t unit, int lane) {
    using T = FmtTraits<FMT>;
    const uint8_t* blk = row + (unit / T::kUnitsPerBlock) * T::kBlockBytes;
    const uint32_t hdr = *reinterpret_cast<const uint32_t*>(blk);
    const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr & 0xFFFFu)));
    const float b = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr >> 16)));
    if (FMT == FMT_HQ4_G32_M5) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(blk + 4 + 4 * (lane >> 3));
        const int j = lane & 7;
        const uint32_t q = (w >> (4 * (j >> 1) + 16 * (j & 1))) & 0xFu;
        return __fadd_rn(__fmul_rn(static_cast<float>(q) + 1024.0f, s), b);
    } else if (FMT == FMT_HQ8_G32) {
        const uint32_t q = blk[4 + lane];
        return __fadd_rn(__fmul_rn(static_cast<float>(q), s), b);
    } else {
        const int e = static_cast<int>(unit % T::kUnitsPerBlock) * 32 + lane;
        const uint32_t q = (blk[4 + (e >> 1)] >> (4 * (e & 1))) & 0xFu;
        return __fadd_rn(__fmul_rn(static_cast<float>(q), s), b);
    }
}

template <int FMT, typename OutT>
__global__ void __launch_bounds__(256) qwc_dequant_kernel(const uint8_t* __restrict__ blocks, int64_t n, int64_t k,
                                                          OutT* __restrict__ out, int standard_domain) {
    using T = FmtTraits<FMT>;
    const int lane = threadIdx.x & 31;
    const int64_t units_per_row = k / 32;
    const int64_t row_bytes = (k / T::kGroup) * T::kBlockBytes;
    const int64_t total = n * units_per_row;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t u = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); u < total; u += warps) {
        const int64_t r = u / units_per_row, unit = u % units_per_row;
        float v = decode_element<FMT>(blocks + r * row_bytes, unit, lane);
        if (standard_domain) {
#pragma unroll
            for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
            v = __fmul_rn(v, qwc_inv_sqrt32());
        }
        if (sizeof(OutT) == 4) reinterpret_cast<float*>(out)[r * k + unit * 32 + lane] = v;
        else reinterpret_cast<__half*>(out)[r * k + unit * 32 + lane] = __float2half_rn(v);
    }
}

// In-place f16 FWHT-32: f32 butterflies, one rounding back to f16
// (reference kernel qwg_fwht32_f16, Sources/QWMetal/gemm/qwgemm.metal:27-32).
__global__ void __launch_bounds__(256) qwc_fwht32_f16_kernel(__half* __restrict__ x, int64_t count) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); b < count / 32; b += warps) {
        float v = __half2float(x[b * 32 + lane]);
#pragma unroll
        for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
        x[b * 32 + lane] = __float2half_rn(__fmul_rn(v, qwc_inv_sqrt32()));
    }
}

// ---- load-time quantizer -----------------------------------------------------------------------------------
// Device twin of the reference's packers (Scripts/quantize/hq4.py:54-123, hq_blocks.py:436-517; Metal twin
// Sources/QWMetal/quant/qw_online_quant.metal:17-55): same f32 operations in the same order, so the bytes equal
// the Python packer's.  One warp per group; a 64-wide group is two FWHT-32 units held as two values per lane.
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float rotate32(float v, int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
    return __fmul_rn(v, qwc_inv_sqrt32());
}

template <int FMT>
__global__ void __launch_bounds__(256) qwc_quantize_kernel(const float* __restrict__ w, int64_t n, int64_t k,
                                                           uint8_t* __restrict__ blocks, int32_t* status) {
    using T = FmtTraits<FMT>;
    const int lane = threadIdx.x & 31;
    const int64_t groups_per_row = k / T::kGroup;
    const int64_t total = n * groups_per_row;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); g < total; g += warps) {
        const float* src = w + g * T::kGroup;  // groups are contiguous in a row-major [n, k] tensor
        uint8_t* blk = blocks + g * T::kBlockBytes;
        float v[T::kUnitsPerBlock];
        bool finite = true;
#pragma unroll
        for (int u = 0; u < T::kUnitsPerBlock; ++u) {
            const float raw = src[32 * u + lane];
            finite = finite && isfinite(raw);
            v[u] = rotate32(raw, lane);
        }
        if (!__all_sync(0xFFFFFFFFu, finite) && lane == 0) atomicCAS(status, 0, QWC_DEV_NONFINITE_WEIGHT);
        if (FMT == FMT_HQ4_G32_M5) {
            const float amax = warp_max(fabsf(v[0]));
            float sc = __fdiv_rn(amax, 7.5f);
            if (!(sc < 63.46875f)) sc = 63.46875f;
            const __half sh = __float2half_rn(sc);
            const float es = __half2float(sh);
            const __half bh = __float2half_rn(__fmul_rn(-1032.0f, es));
            const float eb = __half2float(bh);
            const float safe = es > 0.0f ? es : 1.0f;
            float qf = floorf(__fsub_rn(__fdiv_rn(__fsub_rn(v[0], eb), safe), 1023.5f));
            qf = fminf(fmaxf(qf, 0.0f), 15.0f);
            const uint32_t q = es > 0.0f ? static_cast<uint32_t>(qf) : 8u;
            const int j = lane & 7;
            uint32_t word = q << (4 * (j >> 1) + 16 * (j & 1));
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 1);
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 4);
            if (j == 0) *reinterpret_cast<uint32_t*>(blk + 4 + 4 * (lane >> 3)) = word;
            if (lane == 0)
                *reinterpret_cast<uint32_t*>(blk) = static_cast<uint32_t>(__half_as_ushort(sh)) |
                                                    (static_cast<uint32_t>(__half_as_ushort(bh)) << 16);
        } else {
            float mn = v[0], mx = v[0];
#pragma unroll
            for (int u = 1; u < T::kUnitsPerBlock; ++u) { mn = fminf(mn, v[u]); mx = fmaxf(mx, v[u]); }
            mn = warp_min(mn);
            mx = warp_max(mx);
            const float qmax = FMT == FMT_HQ8_G32 ? 255.0f : 15.0f;
            const __half sh = __float2half_rn(__fdiv_rn(__fsub_rn(mx, mn), qmax));
            const __half bh = __float2half_rn(mn);
            const float es = __half2float(sh), eb = __half2float(bh);
            const float safe = es > 0.0f ? es : 1.0f;
            uint32_t q[T::kUnitsPerBlock];
#pragma unroll
            for (int u = 0; u < T::kUnitsPerBlock; ++u) {
                float qf = rintf(__fdiv_rn(__fsub_rn(v[u], eb), safe));
                qf = fminf(fmaxf(qf, 0.0f), qmax);
                q[u] = es > 0.0f ? static_cast<uint32_t>(qf) : 0u;
            }
            if (FMT == FMT_HQ8_G32) {
                blk[4 + lane] = static_cast<uint8_t>(q[0]);
            } else {
#pragma unroll
                for (int u = 0; u < T::kUnitsPerBlock; ++u) {
                    uint32_t nib = q[u] << (4 * (lane & 1));
                    nib |= __shfl_xor_sync(0xFFFFFFFFu, nib, 1);
                    if ((lane & 1) == 0) blk[4 + 16 * u + (lane >> 1)] = static_cast<uint8_t>(nib);
                }
            }
            if (lane == 0)
                *reinterpret_cast<uint32_t*>(blk) = static_cast<uint32_t>(__half_as_ushort(sh)) |
                                                    (static_cast<uint32_t>(__half_as_ushort(bh)) << 16);
        }
    }
}

template <int FMT>
int launch_quantize(const qwc_hal* hal, cudaStream_t st, const float* w, int64_t n, int64_t k, void* blocks) {
    const int64_t total = n * (k / FmtTraits<FMT>::kGroup);
    if (total == 0) return QWC_OK;
    int64_t grid = (total + 7) / 8;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    if (grid > cap) grid = cap;
    qwc_quantize_kernel<FMT><<<static_cast<unsigned>(grid), 256, 0, st>>>(w, n, k, static_cast<uint8_t*>(blocks), hal->status);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

template <int FMT>
int launch_dequant(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, void* out, int out_dtype, int std_dom) {
    const int64_t total = w->n * (w->k / 32);
    if (total == 0) return QWC_OK;
    int64_t blocks = (total + 7) / 8;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    const uint8_t* p = static_cast<const uint8_t*>(w->blocks);
    if (out_dtype == QWC_F32)
        qwc_dequant_kernel<FMT, float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p, w->n, w->k, static_cast<float*>(out), std_dom);
    else
        qwc_dequant_kernel<FMT, __half><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p, w->n, w->k, static_cast<__half*>(out), std_dom);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

}  // namespace

int qwc_launch_dequant(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, void* out, int out_dtype,
                       int standard_domain) {
    switch (qwc_fmt_of(*w)) {
        case FMT_HQ4_G32_M5: return launch_dequant<FMT_HQ4_G32_M5>(hal, st, w, out, out_dtype, standard_domain);
        case FMT_HQ8_G32: return launch_dequant<FMT_HQ8_G32>(hal, st, w, out, out_dtype, standard_domain);
        case FMT_HQ4_G64: return launch_dequant<FMT_HQ4_G64>(hal, st, w, out, out_dtype, standard_domain);
        default: return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unsupported container (kind %d bits %d group %d)", w->kind, w->bits, w->group);
    }
}

int qwc_launch_fwht32_f16(const qwc_hal* hal, cudaStream_t st, void* x, int64_t count) {
    if (count == 0) return QWC_OK;
    int64_t blocks = (count / 32 + 7) / 8;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    qwc_fwht32_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<__half*>(x), count);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

int qwc_launch_quantize(const qwc_hal* hal, cudaStream_t st, const float* w, int64_t n, int64_t k, int fmt, void* blocks) {
    switch (fmt) {
        case FMT_HQ4_G32_M5: return launch_quantize<FMT_HQ4_G32_M5>(hal, st, w, n, k, blocks);
        case FMT_HQ8_G32: return launch_quantize<FMT_HQ8_G32>(hal, st, w, n, k, blocks);
        case FMT_HQ4_G64: return launch_quantize<FMT_HQ4_G64>(hal, st, w, n, k, blocks);
        default: return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unsupported container");
    }
}
