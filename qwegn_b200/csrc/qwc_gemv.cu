// Decode GEMV (M = 1) and small-M verify GEMM (M <= 16) over packed HQ blocks: the CUDA twin of the reference's
// qwg_gemv_q4g_* / qwg_gemv_aq* / qwg_skinny_m* / qwm_mlp_*_m* kernel families
// (Sources/QWMetal/gemm/qwgemm.metal, qwgemm_aq.metal, qwg_skinny.metal, Sources/QWMetal/mtp/qwmtp_mlp.metal).
//
// The path is bound by HBM: every weight byte is read exactly once.  Design:
//  * one persistent CTA per SM owns a contiguous range of output rows; the packed rows are streamed, unchanged,
//    into a 4-stage shared-memory ring with 1-D bulk async copies (cp.async.bulk + mbarrier tx counts), 16 rows x
//    one K-chunk per stage, each row padded by 16 B so the per-lane word reads are bank-conflict free; the duty of
//    refilling a stage rotates over the warps so no warp is set aside (512 threads keep 128 registers each);
//  * the 16 warps split K: warp w owns the 32-element units w, w+16, ... of the chunk and keeps the matching
//    activation fragments in registers for every row tile of the CTA (x is read once per CTA, rotated in
//    registers by FWHT-32 with two xor-shuffle stages when the caller passes standard-basis activations);
//  * nibbles/bytes are expanded in registers straight into m16n8k16 A fragments by the magic-bias form
//    (0x6400 | q as f16 = 1024 + q, then one f16 FMA with scale and bias -- the reference's decode class,
//    Sources/QWMetal/include/qw_dequant.metalh:53-61) and the dot products run on mma.sync with f32 accumulate.
//    A SIMT FMA dot needs >3 issue slots per weight and cannot keep up with the bulk-copy stream; the k order
//    inside a unit is permuted per format so that each lane's A words and B activations line up without shuffles;
//  * the split-K partial sums of the 16 warps are combined through shared memory in a fixed order (deterministic).
#include "qwc_common.cuh"

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kTileRows = 16;

template <int FMT> struct StreamCfg;
template <> struct StreamCfg<FMT_HQ4_G32_M5> { static constexpr int kUnitBytes = 20, kMaxChunkUnits = 128; };
template <> struct StreamCfg<FMT_HQ8_G32> { static constexpr int kUnitBytes = 36, kMaxChunkUnits = 64; };
template <> struct StreamCfg<FMT_HQ4_G64> { static constexpr int kUnitBytes = 18, kMaxChunkUnits = 128; };

struct GemvParams {
    const uint8_t* blocks;
    int64_t row_bytes;
    const __half* x;
    int64_t ldx;
    void* y;
    int64_t ldy;
    int32_t* status;
    int n_out;        // output rows (n, or n/2 for the silu-pair epilogues)
    int m;            // tokens, <= 8 * NT
    int units;        // k / 32
    int nchunks;      // K chunks
    int chunk_units;  // units per chunk (multiple of 16; the last chunk may be shorter)
    int y_f16;
    int epilogue;
    int x_is_rotated;
    int row_quantum;  // CTA row ranges start on multiples of this (32 for the fused-FWHT epilogue)
};

template <int FMT, int NT>
struct Smem {
    using C = StreamCfg<FMT>;
    static constexpr int kStride = C::kMaxChunkUnits * C::kUnitBytes + 16;  // (kStride / 4) % 32 == 4
    static constexpr int kStageBytes = kTileRows * kStride;
    static constexpr int kRT = NT == 1 ? 8 : 4;  // weight-row tiles per pass
    static constexpr int kRedBytes = 8 * kRT * NT * 32 * 16;
    static constexpr int kHBufBytes = 8 * NT * (kRT * kTileRows / 2) * 4;
    static constexpr int kOffRed = kStages * kStageBytes;
    static constexpr int kOffHBuf = kOffRed + kRedBytes;
    static constexpr int kOffBars = kOffHBuf + kHBufBytes;
    static constexpr int kTotal = kOffBars + 2 * kStages * 8 + 16;
    static_assert((kStride / 4) % 32 == 4 && kStride % 16 == 0, "row padding must shift banks by 4 words");
};

__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Decode this lane's share of one unit of one row into four f16x2 A-fragment registers
// (a[0], a[1] feed the first k16 MMA, a[2], a[3] the second).  srow = the row's chunk in shared memory.
template <int FMT>
__device__ __forceinline__ void decode_unit(const uint8_t* srow, int u, int t, uint32_t a[4]) {
    if (FMT == FMT_HQ4_G32_M5) {
        const uint8_t* blk = srow + u * 20;
        const uint32_t hdr = lds32(blk);
        const uint32_t w = lds32(blk + 4 + 4 * t);
        const uint32_t s2 = __byte_perm(hdr, hdr, 0x1010), b2 = __byte_perm(hdr, hdr, 0x3232);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = hfma2_u32(((w >> (4 * i)) & 0x000F000Fu) | 0x64006400u, s2, b2);
    } else if (FMT == FMT_HQ8_G32) {
        const uint8_t* blk = srow + u * 36;
        const uint32_t hdr = lds32(blk);
        const uint32_t w0 = lds32(blk + 4 + 4 * t), w1 = lds32(blk + 20 + 4 * t);
        const uint32_t s2 = __byte_perm(hdr, hdr, 0x1010), b2 = __byte_perm(hdr, hdr, 0x3232);
        const uint32_t k1024 = 0x64006400u;
        a[0] = hfma2_u32(hsub2_u32(__byte_perm(w0, 0x64646464u, 0x4140), k1024), s2, b2);
        a[1] = hfma2_u32(hsub2_u32(__byte_perm(w0, 0x64646464u, 0x4342), k1024), s2, b2);
        a[2] = hfma2_u32(hsub2_u32(__byte_perm(w1, 0x64646464u, 0x4140), k1024), s2, b2);
        a[3] = hfma2_u32(hsub2_u32(__byte_perm(w1, 0x64646464u, 0x4342), k1024), s2, b2);
    } else {
        const uint8_t* blk = srow + (u >> 1) * 36;
        const uint32_t hdr = lds32(blk);
        const uint32_t w = lds32(blk + 4 + 16 * (u & 1) + 4 * t);
        const uint32_t s2 = __byte_perm(hdr, hdr, 0x1010), b2 = __byte_perm(hdr, hdr, 0x3232);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            a[i] = hfma2_u32(hsub2_u32(((w >> (4 * i)) & 0x000F000Fu) | 0x64006400u, 0x64006400u), s2, b2);
    }
}

__device__ __forceinline__ void mma_16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Activation fragment of one unit for one token: this lane's 8 k values, in the k order decode_unit<FMT> uses.
// Natural layout: lane t of a quad holds elements 8t .. 8t+7 of the unit.
template <int FMT>
__device__ __forceinline__ void load_x_frag(const __half* xrow /* token row + unit*32, or nullptr */, int t, bool rotate,
                                            uint32_t xb[4]) {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (xrow != nullptr) raw = *reinterpret_cast<const uint4*>(xrow + 8 * t);
    uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    if (rotate) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2*>(&r[i]);
            f[2 * i] = __low2float(h);
            f[2 * i + 1] = __high2float(h);
        }
#pragma unroll
        for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if ((i & h) == 0) {
                    const float u = f[i], v = f[i + h];
                    f[i] = __fadd_rn(u, v);
                    f[i + h] = __fsub_rn(u, v);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 1, (t & 1) != 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 2, (t & 2) != 0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(__fmul_rn(f[2 * i], qwc_inv_sqrt32()), __fmul_rn(f[2 * i + 1], qwc_inv_sqrt32()));
            r[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    if (FMT == FMT_HQ4_G32_M5) {
#pragma unroll
        for (int i = 0; i < 4; ++i) xb[i] = r[i];
    } else if (FMT == FMT_HQ4_G64) {
        // pair i of the word is (element 8t+i, element 8t+i+4)
        xb[0] = __byte_perm(r[0], r[2], 0x5410);
        xb[1] = __byte_perm(r[0], r[2], 0x7632);
        xb[2] = __byte_perm(r[1], r[3], 0x5410);
        xb[3] = __byte_perm(r[1], r[3], 0x7632);
    } else {
        // lane t needs elements 4t..4t+3 (held by lane t>>1, half t&1) and 16+4t..16+4t+3 (lane 2+(t>>1), half t&1)
        const int lane = threadIdx.x & 31;
        const int src_lo = (lane & ~3) | (t >> 1), src_hi = src_lo | 2;
        const uint32_t l0 = __shfl_sync(0xFFFFFFFFu, r[0], src_lo), l1 = __shfl_sync(0xFFFFFFFFu, r[1], src_lo);
        const uint32_t l2 = __shfl_sync(0xFFFFFFFFu, r[2], src_lo), l3 = __shfl_sync(0xFFFFFFFFu, r[3], src_lo);
        const uint32_t h0 = __shfl_sync(0xFFFFFFFFu, r[0], src_hi), h1 = __shfl_sync(0xFFFFFFFFu, r[1], src_hi);
        const uint32_t h2 = __shfl_sync(0xFFFFFFFFu, r[2], src_hi), h3 = __shfl_sync(0xFFFFFFFFu, r[3], src_hi);
        const bool odd = (t & 1) != 0;
        xb[0] = odd ? l2 : l0;
        xb[1] = odd ? l3 : l1;
        xb[2] = odd ? h2 : h0;
        xb[3] = odd ? h3 : h1;
    }
}

__device__ __forceinline__ void cta_bar_sync() { __syncthreads(); }

// Position of one stage fill in the CTA's fixed schedule: pass (group of row tiles) -> K chunk -> row tile.
struct FillIter {
    int pass, c, rt;
    int r0, rows, tiles_out, ntiles;
    bool done;
};

template <int FMT, int NT>
__global__ void __launch_bounds__(kThreads, 1) qwc_gemv_stream_kernel(const GemvParams p) {
    using S = Smem<FMT, NT>;
    using C = StreamCfg<FMT>;
    constexpr int kRT = S::kRT;
    constexpr int kXU = C::kMaxChunkUnits / kWarps;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kOffBars);
    uint64_t* empty = full + kStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // This CTA's output rows [rb, re).
    const int quanta = p.n_out / p.row_quantum;  // n_out % row_quantum == 0 is checked on the host
    const int rb = static_cast<int>((static_cast<int64_t>(quanta) * blockIdx.x) / gridDim.x) * p.row_quantum;
    const int re = static_cast<int>((static_cast<int64_t>(quanta) * (blockIdx.x + 1)) / gridDim.x) * p.row_quantum;
    const bool paired = p.epilogue != QWC_EPI_NONE;
    const int out_rows_per_pass = (paired ? kRT / 2 : kRT) * kTileRows;
    const int npasses = (re - rb + out_rows_per_pass - 1) / out_rows_per_pass;

    auto set_pass = [&](FillIter& it) {
        it.r0 = rb + it.pass * out_rows_per_pass;
        it.rows = min(re - it.r0, out_rows_per_pass);
        it.tiles_out = (it.rows + kTileRows - 1) / kTileRows;
        it.ntiles = paired ? 2 * it.tiles_out : it.tiles_out;
    };
    auto advance = [&](FillIter& it) {
        if (++it.rt < it.ntiles) return;
        it.rt = 0;
        if (++it.c < p.nchunks) return;
        it.c = 0;
        if (++it.pass < npasses) set_pass(it);
        else it.done = true;
    };
    bool ok = true;
    // Fill one stage: wait until its previous contents were consumed by all warps, then one bulk copy per row.
    // Executed by a whole warp; the duty rotates over the warps (fill number seq is issued by warp seq % 16).
    auto fill = [&](const FillIter& it, uint32_t seq) {
        const int stage = seq % kStages;
        if (seq >= kStages && ok && !*abort_flag) {
            ok = mbar_wait(&empty[stage], ((seq / kStages) - 1) & 1);
            if (!ok) {
                *abort_flag = 1;
                if (lane == 0) atomicCAS(p.status, 0, QWC_DEV_WAIT_EMPTY_TIMEOUT);
            }
        }
        if (!ok || *abort_flag) return;
        const int u0 = it.c * p.chunk_units;
        const uint32_t cbytes = static_cast<uint32_t>(min(p.chunk_units, p.units - u0)) * C::kUnitBytes;
        const bool up = paired && it.rt >= it.tiles_out;
        const int first = it.r0 + (up ? it.rt - it.tiles_out : it.rt) * kTileRows;  // first output row of the tile
        const int valid = min(kTileRows, it.r0 + it.rows - first);
        const int64_t wrow = static_cast<int64_t>(first) + (up ? p.n_out : 0);
        if (lane == 0) mbar_arrive_expect_tx(&full[stage], cbytes * valid);
        __syncwarp();
        if (lane < valid) {
            const uint8_t* src = p.blocks + (wrow + lane) * p.row_bytes + static_cast<int64_t>(u0) * C::kUnitBytes;
            bulk_g2s(smem + stage * S::kStageBytes + lane * S::kStride, src, cbytes, &full[stage]);
        }
    };

    FillIter pit{};  // the next fill to issue (runs kStages - 1 ahead of consumption)
    pit.done = npasses == 0;
    if (!pit.done) set_pass(pit);
    uint32_t fill_seq = 0;
    for (; fill_seq < kStages - 1 && !pit.done; ++fill_seq) {
        if (warp == static_cast<int>(fill_seq % kWarps)) fill(pit, fill_seq);
        advance(pit);
    }

    const int gid = lane >> 2, t = lane & 3;
    float* red = reinterpret_cast<float*>(smem + S::kOffRed);
    float* hbuf = reinterpret_cast<float*>(smem + S::kOffHBuf);
    uint32_t seq = 0;
    for (int pass = 0; pass < npasses; ++pass) {
        const int r0 = rb + pass * out_rows_per_pass;
        const int rows = min(re - r0, out_rows_per_pass);
        const int tiles_out = (rows + kTileRows - 1) / kTileRows;
        const int ntiles = paired ? 2 * tiles_out : tiles_out;
        float d[kRT][NT][4];
#pragma unroll
        for (int rt = 0; rt < kRT; ++rt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) d[rt][nt][i] = 0.0f;

        for (int c = 0; c < p.nchunks; ++c) {
            const int u0 = c * p.chunk_units;
            const int cu = min(p.chunk_units, p.units - u0);
            uint32_t xb[kXU][NT][4];
#pragma unroll
            for (int j = 0; j < kXU; ++j) {
                const int u = warp + kWarps * j;
                if (u < cu) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int tok = nt * 8 + gid;
                        const __half* xr = tok < p.m ? p.x + tok * p.ldx + static_cast<int64_t>(u0 + u) * 32 : nullptr;
                        load_x_frag<FMT>(xr, t, p.x_is_rotated == 0, xb[j][nt]);
                    }
                }
            }
#pragma unroll
            for (int rt = 0; rt < kRT; ++rt) {
                if (rt < ntiles) {
                    if (!pit.done) {
                        if (warp == static_cast<int>(fill_seq % kWarps)) fill(pit, fill_seq);
                        advance(pit);
                        ++fill_seq;
                    }
                    const int stage = seq % kStages;
                    if (ok && !*abort_flag) {
                        ok = mbar_wait(&full[stage], (seq / kStages) & 1);
                        if (!ok) {
                            *abort_flag = 1;
                            if (lane == 0) atomicCAS(p.status, 0, QWC_DEV_WAIT_FULL_TIMEOUT);
                        }
                    }
                    if (ok && !*abort_flag) {
                        const uint8_t* row_lo = smem + stage * S::kStageBytes + gid * S::kStride;
                        const uint8_t* row_hi = row_lo + 8 * S::kStride;
#pragma unroll
                        for (int j = 0; j < kXU; ++j) {
                            const int u = warp + kWarps * j;
                            if (u < cu) {
                                uint32_t alo[4], ahi[4];
                                decode_unit<FMT>(row_lo, u, t, alo);
                                decode_unit<FMT>(row_hi, u, t, ahi);
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    mma_16816(d[rt][nt], alo[0], ahi[0], alo[1], ahi[1], xb[j][nt][0], xb[j][nt][1]);
                                    mma_16816(d[rt][nt], alo[2], ahi[2], alo[3], ahi[3], xb[j][nt][2], xb[j][nt][3]);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[stage]);
                    ++seq;
                }
            }
        }

        // ---- split-K reduction over the 16 warps, fixed order: (w) + (w+8), then slots 0..7 in sequence ----
        float4* red4 = reinterpret_cast<float4*>(red);
        if (warp >= 8) {
#pragma unroll
            for (int rt = 0; rt < kRT; ++rt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    red4[(((warp - 8) * kRT + rt) * NT + nt) * 32 + lane] =
                        make_float4(d[rt][nt][0], d[rt][nt][1], d[rt][nt][2], d[rt][nt][3]);
        }
        cta_bar_sync();
        if (warp < 8) {
#pragma unroll
            for (int rt = 0; rt < kRT; ++rt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float4* slot = &red4[((warp * kRT + rt) * NT + nt) * 32 + lane];
                    const float4 o = *slot;
                    *slot = make_float4(d[rt][nt][0] + o.x, d[rt][nt][1] + o.y, d[rt][nt][2] + o.z, d[rt][nt][3] + o.w);
                }
        }
        cta_bar_sync();
        const int out_tiles = paired ? kRT / 2 : kRT;
        for (int item = threadIdx.x; item < out_tiles * NT * 32; item += kThreads) {
            const int l = item & 31, nt = (item >> 5) % NT, rt = item / (32 * NT);
            if (rt >= tiles_out) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), acc_up = acc;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const float4 v = red4[((s * kRT + rt) * NT + nt) * 32 + l];
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            if (paired) {
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    const float4 v = red4[((s * kRT + rt + tiles_out) * NT + nt) * 32 + l];
                    acc_up.x += v.x; acc_up.y += v.y; acc_up.z += v.z; acc_up.w += v.w;
                }
            }
            const int g = l >> 2, tt = l & 3;
            const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
            const float ups[4] = {acc_up.x, acc_up.y, acc_up.z, acc_up.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int lrow = rt * kTileRows + g + 8 * (i >> 1);  // row inside the pass
                const int tok = nt * 8 + 2 * tt + (i & 1);
                if (lrow >= rows || tok >= p.m) continue;
                float v = vals[i];
                if (paired) v = (v / (1.0f + expf(-v))) * ups[i];
                if (p.epilogue == QWC_EPI_SILU_PAIR_FWHT) {
                    hbuf[tok * (out_tiles * kTileRows) + lrow] = __half2float(__float2half_rn(v));
                } else {
                    const int64_t o = static_cast<int64_t>(tok) * p.ldy + r0 + lrow;
                    if (p.y_f16) static_cast<__half*>(p.y)[o] = __float2half_rn(v);
                    else static_cast<float*>(p.y)[o] = v;
                }
            }
        }
        if (p.epilogue == QWC_EPI_SILU_PAIR_FWHT) {
            cta_bar_sync();
            // rows is a multiple of 32 here; one warp rotates one (token, 32-row block).
            const int blocks32 = rows / 32;
            for (int item = warp; item < p.m * blocks32; item += kWarps) {
                const int tok = item / blocks32, b = item % blocks32;
                float v = hbuf[tok * (out_tiles * kTileRows) + b * 32 + lane];
#pragma unroll
                for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
                v = __fmul_rn(v, qwc_inv_sqrt32());
                const int64_t o = static_cast<int64_t>(tok) * p.ldy + r0 + b * 32 + lane;
                if (p.y_f16) static_cast<__half*>(p.y)[o] = __float2half_rn(v);
                else static_cast<float*>(p.y)[o] = __half2float(__float2half_rn(v));
            }
        }
        cta_bar_sync();  // red / hbuf are reused by the next pass
    }
    // After a failed wait some fills may never have been consumed: let this CTA's own copies land (bounded
    // wait on the last phase of every stage that was filled) before the CTA exits.
    if (*abort_flag && threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages && s < fill_seq; ++s) {
            const uint32_t last = ((fill_seq - 1 - s) / kStages) * kStages + s;  // last fill number that used stage s
            mbar_wait(&full[s], (last / kStages) & 1);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Row-wise fallback for banks the bulk-copy kernel cannot take (row bytes or base not 16-byte aligned, i.e.
// K % 128 != 0 for the 20/36-byte blocks): one warp per output row, lanes stride the units, plain loads, f32 FMA
// with the f16-rounded decode.  Correctness path for odd shapes; never the timed one.
template <int FMT>
__device__ __forceinline__ float decode_one_f16class(const uint8_t* blk, int e /* element inside the block */) {
    const uint32_t hdr = *reinterpret_cast<const uint32_t*>(blk);
    const __half s = __ushort_as_half(static_cast<unsigned short>(hdr & 0xFFFFu));
    const __half b = __ushort_as_half(static_cast<unsigned short>(hdr >> 16));
    if (FMT == FMT_HQ4_G32_M5) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(blk + 4 + 4 * (e >> 3));
        const int j = e & 7;
        const uint32_t q = (w >> (4 * (j >> 1) + 16 * (j & 1))) & 0xFu;
        return __half2float(__hfma(__ushort_as_half(static_cast<unsigned short>(0x6400u | q)), s, b));
    } else if (FMT == FMT_HQ8_G32) {
        return __half2float(__hfma(__ushort2half_rn(blk[4 + e]), s, b));
    } else {
        const uint32_t q = (blk[4 + (e >> 1)] >> (4 * (e & 1))) & 0xFu;
        return __half2float(__hfma(__ushort2half_rn(static_cast<unsigned short>(q)), s, b));
    }
}

template <int FMT>
__global__ void __launch_bounds__(256) qwc_gemv_rowwise_kernel(const GemvParams p, int m_total) {
    using T = FmtTraits<FMT>;
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    const bool paired = p.epilogue != QWC_EPI_NONE;
    const int64_t items = static_cast<int64_t>(p.n_out) * m_total;
    for (int64_t it = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += warps) {
        const int r = static_cast<int>(it % p.n_out), tok = static_cast<int>(it / p.n_out);
        float acc[2] = {0.f, 0.f};
        for (int half_i = 0; half_i < (paired ? 2 : 1); ++half_i) {
            const uint8_t* row = p.blocks + (static_cast<int64_t>(r) + (half_i ? p.n_out : 0)) * p.row_bytes;
            float a = 0.f;
            for (int u = 0; u < p.units; ++u) {
                float xv = __half2float(p.x[tok * p.ldx + u * 32 + lane]);
                if (!p.x_is_rotated) {
#pragma unroll
                    for (int h = 1; h < 32; h <<= 1) xv = fwht_xor_stage(xv, h, (lane & h) != 0);
                    xv = __half2float(__float2half_rn(__fmul_rn(xv, qwc_inv_sqrt32())));
                }
                const uint8_t* blk = row + (u / T::kUnitsPerBlock) * T::kBlockBytes;
                a = fmaf(decode_one_f16class<FMT>(blk, (u % T::kUnitsPerBlock) * 32 + lane), xv, a);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
            acc[half_i] = a;
        }
        float v = acc[0];
        if (paired) v = (v / (1.0f + expf(-v))) * acc[1];
        if (lane == 0) {
            const int64_t o = static_cast<int64_t>(tok) * p.ldy + r;
            if (p.y_f16) static_cast<__half*>(p.y)[o] = __float2half_rn(v);
            else static_cast<float*>(p.y)[o] = v;
        }
    }
}

template <int FMT, int NT>
int launch_stream(const qwc_hal* hal, cudaStream_t st, GemvParams p) {
    using S = Smem<FMT, NT>;
    using C = StreamCfg<FMT>;
    static bool configured[64] = {};
    if (!configured[hal->device & 63]) {
        QWC_CUDA_TRY(cudaFuncSetAttribute(qwc_gemv_stream_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured[hal->device & 63] = true;
    }
    p.nchunks = (p.units + C::kMaxChunkUnits - 1) / C::kMaxChunkUnits;
    const int per = (p.units + p.nchunks - 1) / p.nchunks;
    p.chunk_units = ((per + 15) / 16) * 16;
    p.nchunks = (p.units + p.chunk_units - 1) / p.chunk_units;
    const int quanta = p.n_out / p.row_quantum;
    int grid = hal->sm_count;
    if (grid > quanta) grid = quanta;
    if (grid < 1) grid = 1;
    qwc_gemv_stream_kernel<FMT, NT><<<grid, kThreads, S::kTotal, st>>>(p);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

template <int FMT>
int launch_fmt(const qwc_hal* hal, cudaStream_t st, GemvParams p, int64_t m, bool stream_ok) {
    const char* xb = reinterpret_cast<const char*>(p.x);
    char* yb = static_cast<char*>(p.y);
    const int64_t ysz = p.y_f16 ? 2 : 4;
    if (!stream_ok) {
        if (p.epilogue == QWC_EPI_SILU_PAIR_FWHT)
            return qwc_fail(QWC_ERR_BAD_GEOMETRY, "fused FWHT epilogue needs 16-byte aligned rows (K %% 128 == 0)");
        p.m = static_cast<int>(m);
        const int64_t items = static_cast<int64_t>(p.n_out) * m;
        int64_t grid = (items + 7) / 8;
        if (grid > hal->sm_count * 8) grid = hal->sm_count * 8;
        if (grid < 1) grid = 1;
        qwc_gemv_rowwise_kernel<FMT><<<static_cast<unsigned>(grid), 256, 0, st>>>(p, static_cast<int>(m));
        QWC_CUDA_TRY(cudaGetLastError());
        return QWC_OK;
    }
    // M > 16 is served in slabs of 16 tokens (each slab re-reads the weights); the tensor-core GEMM takes over there.
    for (int64_t m0 = 0; m0 < m; m0 += 16) {
        GemvParams q = p;
        q.m = static_cast<int>(m - m0 < 16 ? m - m0 : 16);
        q.x = reinterpret_cast<const __half*>(xb + m0 * p.ldx * 2);
        q.y = yb + m0 * p.ldy * ysz;
        const int rc = q.m <= 8 ? launch_stream<FMT, 1>(hal, st, q) : launch_stream<FMT, 2>(hal, st, q);
        if (rc) return rc;
    }
    return QWC_OK;
}

}  // namespace

// Host entry used by qwc_gemm.  All arguments were validated by the caller.
int qwc_launch_gemv(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx,
                    void* y, int y_dtype, int64_t ldy, int epilogue, int x_is_rotated, bool allow_stream) {
    GemvParams p{};
    const int fmt = qwc_fmt_of(*w);
    const int64_t bb = qwc_block_bytes(w->kind, w->bits, w->group);
    const int group = fmt == FMT_HQ4_G64 ? 64 : 32;
    p.blocks = static_cast<const uint8_t*>(w->blocks);
    p.row_bytes = (w->k / group) * bb;
    p.x = static_cast<const __half*>(x);
    p.ldx = ldx;
    p.y = y;
    p.ldy = ldy;
    p.status = hal->status;
    p.n_out = static_cast<int>(epilogue == QWC_EPI_NONE ? w->n : w->n / 2);
    p.units = static_cast<int>(w->k / 32);
    p.y_f16 = y_dtype == QWC_F16;
    p.epilogue = epilogue;
    p.x_is_rotated = x_is_rotated;
    p.row_quantum = epilogue == QWC_EPI_SILU_PAIR_FWHT ? 32 : 1;
    const bool stream_ok = allow_stream && (p.row_bytes % 16 == 0) && (reinterpret_cast<uintptr_t>(w->blocks) % 16 == 0) &&
                           (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (ldx % 8 == 0);
    switch (fmt) {
        case FMT_HQ4_G32_M5: return launch_fmt<FMT_HQ4_G32_M5>(hal, st, p, m, stream_ok);
        case FMT_HQ8_G32: return launch_fmt<FMT_HQ8_G32>(hal, st, p, m, stream_ok);
        case FMT_HQ4_G64: return launch_fmt<FMT_HQ4_G64>(hal, st, p, m, stream_ok);
        default: return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unsupported container");
    }
}
