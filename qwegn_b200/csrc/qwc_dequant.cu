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
