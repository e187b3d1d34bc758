// Prefill GEMM and grouped expert GEMM over packed HQ blocks on the 5th-generation tensor cores: the CUDA twin of the
// reference's qwg_gemm_q4g_h16 / qwg_gemm_q4g_nax_f32 / qwg_gemm_aq*_h16 kernels
// (Sources/QWMetal/gemm/qwgemm_batched.metal:24-36, 266-277; qwgemm_aq_batched.metal:8-60; tile loop
// Sources/QWMetal/include/qw_gemm_nax.metalh:153-423).
//
//   Y[m, n] = sum_k Xrot[m, k] * Wrot[n, k],   f16 operands, f32 accumulate in tensor memory.
//
// One persistent CTA per SM walks (weight tile, token tile) pairs.  Roles: warp 0 activation TMA, warp 1 MMA issue
// (+ TMEM allocation), warp 2 packed-weight TMA, 16 converter warps, 4 epilogue warps.
//   * Per raw step a TMA copy brings 128 packed weight rows, unchanged, into a shared-memory ring (2-D tensor copy;
//     one raw step = 128 k for the 20- and 36-byte blocks of 32, 256 k for the 36-byte blocks of 64, so that a row of a
//     step is a multiple of 16 bytes); per 64-wide K tile another TMA copy brings the rotated activations (128-byte
//     swizzle).
//   * A converter thread owns one weight row = one TMEM lane: it reads its row's 64 k of the raw step, decodes them in
//     registers (magic-bias form and one f16 FMA with scale and bias: the reference's in-register decode,
//     qw_gemm_nax.metalh:114-127) and only then waits for the operand stage to be free and writes 32 TMEM columns
//     with tcgen05.st, so the decode of stage j + S overlaps the MMAs of stage j.  Converter warp c serves lane
//     quarter c % 4 and the operand stages j with j % 4 == c / 4.
//   * The MMAs take A from tensor memory and B (the activations) from shared memory: tcgen05.mma, M = 128 weight rows,
//     N = tokens, K = 16, into a TMEM accumulator; tcgen05.commit releases the stage and, after the last K tile, hands
//     the accumulator to the epilogue warps (tcgen05.ld, lane = weight row; plain store or the fused SwiGLU (+ FWHT)
//     epilogue); two accumulators alternate so the epilogue of one tile overlaps the main loop of the next.
//   * TMEM budget (512 columns), four operand stages: tiles of up to 192 tokens use two 192-column accumulators and stages
//     of one 64-wide K tile (32 columns of A each); tiles of up to 128 tokens (expert tiles, verify-sized calls) use two
//     128-column accumulators and stages of two K tiles (64 columns of A, two activation sub-tiles), because the MMA
//     warp's issue loop costs a fixed ~400 cycles per stage (barrier wait, fence, election, commit: measured with every
//     other role idle) and with few tokens the MMAs of one K tile are shorter than that.
// Weights are the M operand so that all tokens of a tile share every decoded weight.  The grouped (mixture-of-experts)
// door runs the same kernel over a device-side tile list.  The kernel is launched with programmatic stream
// serialization and waits for the grid before it (griddepcontrol.wait) after its own set-up, before any global access.
// Every wait is bounded in time; a wait that gives up sets the device status word, raises the CTA's abort flag (which
// the other roles poll) and the CTA winds down and frees its tensor memory.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "qwc_common.cuh"

namespace {

constexpr int kBM = 128;        // weight rows per tile (UMMA M)
constexpr int kBK = 64;         // k per operand stage (one 128-byte swizzle atom of f16)
constexpr int kConvWarps = 16;
constexpr int kEpiWarps = 4;
constexpr int kMaxStages = 8;   // operand stages (one decoded weight tile in TMEM + one activation tile in shared memory each)
constexpr int kTsFirstConvWarp = 4;   // warps 0..2 as above, warp 3 idle so that converter warp c serves quarter c % 4
constexpr int kTsWarps = kTsFirstConvWarp + kConvWarps + kEpiWarps;
constexpr int kTsThreads = kTsWarps * 32;
constexpr int kTsMaxRaw = 8;    // raw (packed weight) stages
constexpr int kTsBN = 192;      // most tokens per tile (UMMA N)

// Packed geometry of one 64-wide K tile of one row, and K tiles per raw step.
template <int FMT> struct TcFmt;
template <> struct TcFmt<FMT_HQ4_G32_M5> { static constexpr int kTileBytes = 40, kTilesPerRaw = 2; };
template <> struct TcFmt<FMT_HQ8_G32> { static constexpr int kTileBytes = 72, kTilesPerRaw = 2; };
template <> struct TcFmt<FMT_HQ4_G64> { static constexpr int kTileBytes = 36, kTilesPerRaw = 4; };

struct TcParams {
    void* y;
    int64_t ldy;
    int32_t* status;
    int m, n, k;
    int y_f16;
    int raw_stages;
    int stages;          // operand stages; a power of two
    int stage_shift;     // log2(stages): slot of stage j = j & (stages - 1), its use count = j >> stage_shift
    int kt_per_stage;    // 64-wide K tiles per operand stage: 1 or 2 (a divisor of the K tiles of a raw step)
    int acc_stride;      // TMEM columns per accumulator: 192 or 128; the operand stages start at column 2 * acc_stride
    int x_tile_rows;     // activation rows per tile: 192, 128 or 64
    int x_slot_bytes;    // bytes of one activation stage: kt_per_stage x x_tile_rows x 128 B
    int raw_row_bytes;   // packed bytes of one raw step of one row: 80 (HQ4_G32_M5) or 144 (HQ8_G32, HQ4_G64)
    int m_tiles, n_tiles;
    int epilogue;        // QWC_EPI_NONE, or a SwiGLU epilogue: a tile is then 64 gate rows + the 64 matching up rows
    int up_delta;        // dense SwiGLU mode: row distance gate -> up (= n / 2)
    int xch_bytes;       // shared memory of the gate/up exchange buffer (SwiGLU epilogues)
    // grouped mode (MoE expert GEMMs): tiles come from a device-side list built by the pair sort
    const qwc_moe_tile* tiles;   // null in dense mode
    const int32_t* tile_count;   // device: number of valid entries of `tiles`
};

// One unit of work of the kernel: 128 weight rows x up to 192 activation rows.
struct TileInfo {
    int w_row0;     // first weight row (row coordinate of the weight tensor map)
    int w_row1;     // SwiGLU epilogues: first up row (rows 64..127 of the tile); unused otherwise
    int w_rows;     // valid weight rows in the tile (<= 128)
    int x_row0;     // first activation row (row coordinate of the activation tensor map)
    int x_rows;     // valid activation rows
    int y_col0;     // output column of weight row 0 of the tile
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// K-major, 128-byte-swizzled operand descriptor: start address, LBO = 1 (unused for swizzled K-major),
// SBO = 1024 B (one 8-row atom), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// One lane of the (converged) warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ uint64_t pack_desc(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, M = 128 weight rows, N = tokens of the
// tile rounded up to a multiple of 16 (16..256).
__device__ __forceinline__ uint32_t make_idesc(int n_tokens) {
    return (1u << 4) | (static_cast<uint32_t>(n_tokens >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t nib2_f16x2(uint32_t v) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(0x000F000Fu), "r"(0x64006400u));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, __half2 s2, __half2 b2) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), s2, b2);
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hsub2_1024(uint32_t a) {
    const uint32_t k = 0x64006400u;
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&k));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Latency-critical wait of the MMA-issuing thread: a plain spin on try_wait (no suspend hint, no sleep); bounded.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 1023u) == 1023u) {   // the clock is read rarely: the loop stays a plain poll
            const uint64_t now = qwc_globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (*abort_flag || now - t0 > QWC_WAIT_LIMIT_NS) return false;
        }
    }
}

// Tile number `tile` of the launch: from the device-side list (grouped mode) or the dense (weight tile, token tile) grid.
__device__ __forceinline__ TileInfo tc_get_tile(const TcParams& p, int tile) {
    TileInfo t;
    if (p.tiles != nullptr) {
        const qwc_moe_tile g = p.tiles[tile];
        t.w_row0 = g.w_row0;
        t.w_row1 = g.pad0;
        t.w_rows = g.w_rows;
        t.x_row0 = g.x_row0;
        t.x_rows = g.x_rows;
        t.y_col0 = g.y_col0;
    } else {
        const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;   // token tiles fastest: CTAs share weight rows in L2
        if (p.epilogue == QWC_EPI_NONE) {
            t.w_row0 = nt * kBM;
            t.w_row1 = 0;
            t.w_rows = min(kBM, p.n - t.w_row0);
        } else {
            t.w_row0 = nt * (kBM / 2);
            t.w_row1 = t.w_row0 + p.up_delta;
            t.w_rows = kBM;
        }
        t.x_row0 = mt * p.x_tile_rows;
        t.x_rows = min(p.x_tile_rows, p.m - t.x_row0);
        t.y_col0 = t.w_row0;
    }
    return t;
}

// One chunk of TOK (16 or 32) tokens of a SwiGLU epilogue for one epilogue warp.  rr = the warp's TOK accumulator columns
// (lane = weight row).  The warp parks the TOK / 2 tokens its partner finishes in the exchange buffer (f16, as the reference's
// threadgroup tile), meets the other three warps, takes its partner's values for the TOK / 2 tokens it finishes itself:
// h = f16(silu(g) * u), FWHT-32 across the 32 rows the warp holds, store.  All TOK / 2 tokens go through each step side by
// side: the five butterfly stages of one token are a chain of dependent shuffles (~30 cycles each), and token after token
// those chains alone took ~1200 cycles per 16 tokens.
template <int TOK>
__device__ __forceinline__ void tc_swiglu_chunk(const TcParams& p, const TileInfo& ti, const uint32_t* rr, uint8_t* xch, bool is_up,
                                                int hrow, int lane, int tok_base) {
    constexpr int HALF = TOK / 2;
    constexpr int ROWB = TOK;   // bytes per row of one side of the exchange buffer: HALF f16
    uint8_t* park = xch + (is_up ? 0 : 64 * ROWB) + hrow * ROWB;          // what this warp gives
    const uint8_t* take = xch + (is_up ? 64 * ROWB : 0) + hrow * ROWB;    // what it gets
    {
        // the gate warps give the upper half of the chunk's tokens, the up warps the lower (selects between constant
        // register indices: a computed index would put the columns in local memory)
#pragma unroll
        for (int v = 0; v < HALF / 8; ++v) {
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = 8 * v + 2 * i;
                const float a = __uint_as_float(is_up ? rr[j] : rr[HALF + j]), b = __uint_as_float(is_up ? rr[j + 1] : rr[HALF + j + 1]);
                const __half2 h2 = __floats2half2_rn(a, b);
                pk[i] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            reinterpret_cast<uint4*>(park)[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    uint32_t other[HALF / 2];
#pragma unroll
    for (int v = 0; v < HALF / 8; ++v) {
        const uint4 got = reinterpret_cast<const uint4*>(take)[v];
        other[4 * v] = got.x; other[4 * v + 1] = got.y; other[4 * v + 2] = got.z; other[4 * v + 3] = got.w;
    }
    const int m0 = is_up ? HALF : 0;       // the tokens this warp finishes
    const int tok0 = tok_base + m0;
    float h[HALF];
#pragma unroll
    for (int jj = 0; jj < HALF; ++jj) {
        const __half2 o2 = *reinterpret_cast<const __half2*>(&other[jj >> 1]);
        const float o = (jj & 1) ? __high2float(o2) : __low2float(o2);
        const float mine = __half2float(__float2half_rn(__uint_as_float(is_up ? rr[HALF + jj] : rr[jj])));
        const float g = is_up ? o : mine, u = is_up ? mine : o;
        h[jj] = __half2float(__float2half_rn(__fdividef(g, 1.0f + __expf(-g)) * u));
    }
    if (p.epilogue == QWC_EPI_SILU_PAIR_FWHT) {
#pragma unroll
        for (int st = 0; st < 5; ++st) {
            const float sg = (lane >> st) & 1 ? -1.0f : 1.0f;
            float oh[HALF];
#pragma unroll
            for (int jj = 0; jj < HALF; ++jj) oh[jj] = __shfl_xor_sync(0xFFFFFFFFu, h[jj], 1 << st);
#pragma unroll
            for (int jj = 0; jj < HALF; ++jj) h[jj] = fmaf(h[jj], sg, oh[jj]);
        }
#pragma unroll
        for (int jj = 0; jj < HALF; ++jj) h[jj] = __fmul_rn(h[jj], qwc_inv_sqrt32());
    }
    const int esz = p.y_f16 ? 2 : 4;
    uint8_t* yrow = static_cast<uint8_t*>(p.y) + (static_cast<int64_t>(ti.x_row0 + tok0) * p.ldy + ti.y_col0 + hrow) * esz;
    const int64_t ystep = p.ldy * esz;
#pragma unroll
    for (int jj = 0; jj < HALF; ++jj) {
        if (tok0 + jj < ti.x_rows) {
            if (p.y_f16) *reinterpret_cast<__half*>(yrow) = __float2half_rn(h[jj]);
            else *reinterpret_cast<float*>(yrow) = __half2float(__float2half_rn(h[jj]));
        }
        yrow += ystep;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the exchange buffer is reused by the next chunk
}

// Epilogue of one tile for one of the four epilogue warps: taddr = TMEM address of the accumulator's first column in
// this warp's lane quarter; xch = 4 KB of shared memory (SwiGLU epilogues only).
__device__ __forceinline__ void tc_epilogue_tile(const TcParams& p, const TileInfo& ti, uint32_t taddr, uint8_t* xch, int quarter,
                                                 int lane) {
    const int wr = quarter * 32 + lane;          // weight row inside the tile
    if (p.epilogue != QWC_EPI_NONE) {
        // SwiGLU epilogues (the reference's qwg_gemm_q4g_h16_swiglu, include/qw_gemm_nax_swiglu.metalh:8-154): TMEM
        // lanes 0..63 hold gate rows, lanes 64..127 the matching up rows, so the two halves of a pair sit in
        // different warps.  Per chunk of tokens each warp parks the half its partner will finish in shared memory: the
        // gate warps finish the lower half with the partner's up values, the up warps the upper half with the partner's
        // gate values, so all four warps share the SwiGLU, the FWHT-32 across the 32 rows a warp holds, and the stores.
        const bool is_up = quarter >= 2;
        const int hrow = (quarter & 1) * 32 + lane;   // row of h inside the tile
        // chunks of 32 tokens while more than 16 are left (half as many meetings of the four warps), one of 16 at the end
        int c0 = 0;
#pragma unroll 1
        for (; ti.x_rows - c0 > 16; c0 += 32) {
            uint32_t rr[32];
            tmem_ld32(taddr + c0, rr);
            tmem_ld_wait();
            tc_swiglu_chunk<32>(p, ti, rr, xch, is_up, hrow, lane, c0);
        }
        if (c0 < ti.x_rows) {
            uint32_t rr[16];
            tmem_ld16(taddr + c0, rr);
            tmem_ld_wait();
            tc_swiglu_chunk<16>(p, ti, rr, xch, is_up, hrow, lane, c0);
        }
    } else {
    // plain epilogue: lane = weight row, 32 token columns per TMEM load; a lane's stores walk down one output column
    const int chunks = (ti.x_rows + 31) / 32;    // only the token columns the MMA wrote
    const int esz = p.y_f16 ? 2 : 4;
    const int64_t ystep = p.ldy * esz;
    uint8_t* ycolp = static_cast<uint8_t*>(p.y) + (static_cast<int64_t>(ti.x_row0) * p.ldy + ti.y_col0 + wr) * esz;
    const bool row_ok = wr < ti.w_rows;
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
        uint32_t rr[32];
        tmem_ld32(taddr + c * 32, rr);
        tmem_ld_wait();
        const int left = ti.x_rows - c * 32;   // valid tokens in this chunk (>= 1)
        if (row_ok) {
            uint8_t* yp = ycolp;
            if (left >= 32) {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) {
                    if (p.y_f16) *reinterpret_cast<__half*>(yp) = __float2half_rn(__uint_as_float(rr[jj]));
                    else *reinterpret_cast<float*>(yp) = __uint_as_float(rr[jj]);
                    yp += ystep;
                }
            } else {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) {
                    if (jj < left) {
                        if (p.y_f16) *reinterpret_cast<__half*>(yp) = __float2half_rn(__uint_as_float(rr[jj]));
                        else *reinterpret_cast<float*>(yp) = __uint_as_float(rr[jj]);
                    }
                    yp += ystep;
                }
            }
        }
        ycolp += 32 * ystep;
    }
    }
}


__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t r[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem desc]: M = 128, K = 16, A = 128 lanes x 8 columns of f16 pairs.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Decode the 64 k of one K tile of one row, held in registers as packed words, into 32 f16 pairs in natural k order:
// out[c] = elements (2c, 2c + 1).
//   HQ4_G32_M5: two blocks of (header, 4 words of interleaved nibbles); HQ8_G32: two blocks of (header, 8 words of code
//   bytes); HQ4_G64: one block of (header, 8 words of linear nibbles: byte c holds elements 2c (low nibble), 2c + 1).
template <int FMT>
__device__ __forceinline__ void decode_tile_natural(const uint32_t* w, uint32_t* out) {
    if (FMT == FMT_HQ4_G64) {
        const uint32_t hdr = w[0];
        const __half2 h = *reinterpret_cast<const __half2*>(&hdr);
        const __half2 s2 = __half2half2(__low2half(h)), b2 = __half2half2(__high2half(h));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t v = w[1 + i];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // byte b -> (low nibble, high nibble) in the two halves: x * 0x1001 = x | x << 12 puts the high nibble
                // at bits 16..19 (x < 256, so the two copies do not overlap); the multiply runs on the FMA pipe
                const uint32_t x = __byte_perm(v, 0u, 0x4440u + b);
                out[4 * i + b] = hfma2_u32(hsub2_1024(nib2_f16x2(x * 0x1001u)), s2, b2);
            }
        }
        return;
    }
    constexpr int kWordsPerUnit = FMT == FMT_HQ4_G32_M5 ? 5 : 9;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t hdr = w[u * kWordsPerUnit];
        const __half2 h = *reinterpret_cast<const __half2*>(&hdr);
        const __half2 s2 = __half2half2(__low2half(h)), b2 = __half2half2(__high2half(h));
        if (FMT == FMT_HQ4_G32_M5) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t v = w[u * 5 + 1 + i];
                out[16 * u + 4 * i + 0] = hfma2_u32(nib2_f16x2(v), s2, b2);
                out[16 * u + 4 * i + 1] = hfma2_u32(nib2_f16x2(v >> 4), s2, b2);
                out[16 * u + 4 * i + 2] = hfma2_u32(nib2_f16x2(v >> 8), s2, b2);
                out[16 * u + 4 * i + 3] = hfma2_u32(nib2_f16x2(v >> 12), s2, b2);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t v = w[u * 9 + 1 + i];
                out[16 * u + 2 * i + 0] = hfma2_u32(hsub2_1024(__byte_perm(v, 0x64646464u, 0x4140)), s2, b2);
                out[16 * u + 2 * i + 1] = hfma2_u32(hsub2_1024(__byte_perm(v, 0x64646464u, 0x4342)), s2, b2);
            }
        }
    }
}

// The packed words of K tile `sub` of a raw step of one row (src = the row's bytes of the raw step in shared memory).
// Rows of a raw step are 80 or 144 bytes apart, so a quarter warp's 16-byte loads fall in 8 distinct bank groups.
template <int FMT>
__device__ __forceinline__ void load_tile_words(const uint8_t* src, int sub, uint32_t* w) {
    if (FMT == FMT_HQ4_G32_M5) {
        // 40 bytes at offset 0 (16-byte aligned) or 40 (8-byte aligned)
        if (sub == 0) {
            const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 16);
            const uint2 d = *reinterpret_cast<const uint2*>(src + 32);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w; w[8] = d.x; w[9] = d.y;
        } else {
            const uint2 d = *reinterpret_cast<const uint2*>(src + 40);
            const uint4 a = *reinterpret_cast<const uint4*>(src + 48), b = *reinterpret_cast<const uint4*>(src + 64);
            w[0] = d.x; w[1] = d.y; w[2] = a.x; w[3] = a.y; w[4] = a.z; w[5] = a.w; w[6] = b.x; w[7] = b.y; w[8] = b.z; w[9] = b.w;
        }
    } else if (FMT == FMT_HQ8_G32) {
        // 72 bytes at offset 0 (16-byte aligned) or 72 (8-byte aligned)
        if (sub == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 a = *reinterpret_cast<const uint4*>(src + 16 * i);
                w[4 * i] = a.x; w[4 * i + 1] = a.y; w[4 * i + 2] = a.z; w[4 * i + 3] = a.w;
            }
            const uint2 d = *reinterpret_cast<const uint2*>(src + 64);
            w[16] = d.x; w[17] = d.y;
        } else {
            const uint2 d = *reinterpret_cast<const uint2*>(src + 72);
            w[0] = d.x; w[1] = d.y;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 a = *reinterpret_cast<const uint4*>(src + 80 + 16 * i);
                w[2 + 4 * i] = a.x; w[3 + 4 * i] = a.y; w[4 + 4 * i] = a.z; w[5 + 4 * i] = a.w;
            }
        }
    } else {
        // 36 bytes at offset 36 * sub (4-byte aligned)
        const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src + 36 * sub);
#pragma unroll
        for (int i = 0; i < 9; ++i) w[i] = s32[i];
    }
}

// KS = 64-wide K tiles per operand stage: compile-time, because the loops that use it pace the kernel and every instruction
// in them counts.
template <int FMT, int KS>
__global__ void __launch_bounds__(kTsThreads, 1)
qwc_gemm_ts_kernel(const TcParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   const __grid_constant__ CUtensorMap xmap128, const __grid_constant__ CUtensorMap xmap64,
                   const __grid_constant__ CUtensorMap wmap64) {
    using F = TcFmt<FMT>;
    constexpr int KPR = F::kTilesPerRaw;
    constexpr int kTileWords = F::kTileBytes / 4;
    // Let the next kernel of the stream be scheduled as early as its resources allow (it waits for this grid itself).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // layout (1024-byte aligned base): [X tiles][raw stages][barriers][SwiGLU exchange]
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* xt = smem;
    uint8_t* raw = xt + p.stages * p.x_slot_bytes;
    const int raw_stage_bytes = ((kBM * p.raw_row_bytes + 127) / 128) * 128;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + p.raw_stages * raw_stage_bytes);
    uint64_t* full = bars;                         // [kMaxStages]  activations landed (tx) + the four quarter warps stored A
    uint64_t* empty = bars + kMaxStages;           // [kMaxStages]  tcgen05.commit: the MMAs have read both operands of the stage
    uint64_t* raw_full = bars + 2 * kMaxStages;    // [kTsMaxRaw]
    uint64_t* raw_empty = raw_full + kTsMaxRaw;    // [kTsMaxRaw]
    uint64_t* acc_full = raw_empty + kTsMaxRaw;    // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(tmem_slot + 4);   // [2][4] the epilogue warps' verdicts on a tile
    uint8_t* xch = reinterpret_cast<uint8_t*>(bars) + 512;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1 + 4);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < p.raw_stages; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], 4 * KPR / KS);   // every operand stage of the step: four quarter warps
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], kEpiWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        // 512 columns.  One CTA per SM, so the allocation cannot contend.
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above needed no global data.  From here on the kernel reads what earlier kernels of the stream wrote
    // (tile list, activations, possibly the weights) and writes y: wait for the grid before this one.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int total_tiles = p.tiles != nullptr ? *p.tile_count : p.m_tiles * p.n_tiles;
    const int ktiles = p.k / kBK;
    const int raw_steps = ktiles / KPR;
    const int kstages = ktiles / KS;                       // operand stages per tile
    const uint32_t x_sub_bytes = static_cast<uint32_t>(p.x_slot_bytes / KS);   // one 64-wide K tile of the activations inside a stage
    const uint32_t a_col0 = static_cast<uint32_t>(2 * p.acc_stride);
    const uint32_t smask = static_cast<uint32_t>(p.stages - 1);
    auto fail = [&](int code) {
        if (!*abort_flag) atomicCAS(p.status, 0, code);
        *abort_flag = 1;
    };

    // Operand stage number j of the kernel (all tiles) holds KS consecutive K tiles, uses slot j % stages in phase
    // (j / stages) & 1 and reads raw step j * KS / KPR, which uses raw slot r % raw_stages in phase (r / raw_stages) & 1.
    if (warp == 0) {
        // ---------------- TMA producer: rotated activations (one tile per K tile) ----------------
        if (lane == 0) {
            uint32_t j = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const TileInfo ti = tc_get_tile(p, tile);
                const CUtensorMap* xm = ti.x_rows <= 64 ? &xmap64 : (ti.x_rows <= 128 ? &xmap128 : &xmap);
                const uint32_t xbytes = (ti.x_rows <= 64 ? 64u : (ti.x_rows <= 128 ? 128u : static_cast<uint32_t>(p.x_tile_rows))) * kBK * 2u;
                for (int ks = 0; ks < kstages; ++ks, ++j) {
                    const uint32_t s = j & smask;
                    const bool got_x = j < static_cast<uint32_t>(p.stages) || mbar_wait_relaxed(&empty[s], ((j >> p.stage_shift) - 1) & 1u, abort_flag);
                    if (!got_x) {
                        fail(QWC_DEV_WAIT_EMPTY_TIMEOUT);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], xbytes * static_cast<uint32_t>(KS));
#pragma unroll
                    for (int q = 0; q < KS; ++q)
                        tma_load_2d(xt + s * p.x_slot_bytes + q * x_sub_bytes, xm, (ks * KS + q) * kBK, ti.x_row0, &full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------- TMA producer: packed weight rows (one raw step = KPR K tiles) ----------------
        uint32_t r = 0;
        int ok = 1;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            if (lane == 0) {
                const TileInfo ti = tc_get_tile(p, tile);
                for (int rs = 0; rs < raw_steps; ++rs, ++r) {
                    const uint32_t s = r % p.raw_stages;
                    const bool got_w = r < static_cast<uint32_t>(p.raw_stages) || mbar_wait_relaxed(&raw_empty[s], ((r / p.raw_stages) - 1) & 1u, abort_flag);
                    if (!got_w) {
                        fail(QWC_DEV_WAIT_EMPTY_TIMEOUT);
                        ok = 0;
                        break;
                    }
                    mbar_arrive_expect_tx(&raw_full[s], static_cast<uint32_t>(kBM * p.raw_row_bytes));
                    if (p.epilogue == QWC_EPI_NONE) {
                        tma_load_2d(raw + s * raw_stage_bytes, &wmap, rs * (p.raw_row_bytes / 8), ti.w_row0, &raw_full[s]);
                    } else {   // 64 gate rows, then the 64 up rows that pair with them
                        tma_load_2d(raw + s * raw_stage_bytes, &wmap64, rs * (p.raw_row_bytes / 8), ti.w_row0, &raw_full[s]);
                        tma_load_2d(raw + s * raw_stage_bytes + (kBM / 2) * p.raw_row_bytes, &wmap64, rs * (p.raw_row_bytes / 8),
                                    ti.w_row1, &raw_full[s]);
                    }
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer (whole warp in lockstep, one elected lane issues) ----------------
        uint32_t j = 0, tiles_done = 0;
        bool ok = true;
        const uint64_t b_d0 = umma_desc_sw128(smem_u32(xt));
        const uint32_t b_lo0 = static_cast<uint32_t>(b_d0), b_hi = static_cast<uint32_t>(b_d0 >> 32);
        const uint32_t b_step = static_cast<uint32_t>(p.x_slot_bytes) >> 4;
        int next_rows = total_tiles > 0 ? tc_get_tile(p, min(static_cast<int>(blockIdx.x), total_tiles - 1)).x_rows : 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tiles_done) {
            const int as = tiles_done & 1;
            if (tiles_done >= 2 && !mbar_wait_spin(&acc_empty[as], ((tiles_done >> 1) - 1) & 1, abort_flag)) {
                if (lane == 0) fail(QWC_DEV_WAIT_TMEM_TIMEOUT);
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(as * p.acc_stride);
            const uint32_t idesc = make_idesc(min(p.acc_stride, (next_rows + 15) & ~15));
            {   // the entry of the tile after this one is fetched now: a list entry is a global-memory round trip
                const int tn = tile + static_cast<int>(gridDim.x);
                next_rows = tc_get_tile(p, tn < total_tiles ? tn : tile).x_rows;
            }
            for (int ks = 0; ks < kstages; ++ks, ++j) {
                const uint32_t s = j & smask;
                const bool got_full = mbar_wait_spin(&full[s], (j >> p.stage_shift) & 1u, abort_flag);   // all lanes poll: measured faster than one polling lane
                if (!got_full) {
                    if (lane == 0) fail(QWC_DEV_WAIT_FULL_TIMEOUT);
                    ok = false;
                    break;
                }
                tc_fence_after();   // the converters' tcgen05.st happen-before these MMAs
                const uint32_t b_lo = b_lo0 + s * b_step;
                const uint32_t a_tmem = tmem_base + a_col0 + s * 32 * KS;
                if (elect_one()) {
#pragma unroll
                    for (int h = 0; h < KS; ++h) {
                        const uint32_t bh = b_lo + h * (x_sub_bytes >> 4);
#pragma unroll
                        for (int q = 0; q < kBK / 16; ++q)
                            umma_f16_ts(d_tmem, a_tmem + (h * 4 + q) * 8, pack_desc(bh + 2 * q, b_hi), idesc, (ks > 0 || h > 0 || q > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit(&acc_full[as]);
            __syncwarp();
        }
        __syncwarp();
    } else if (warp >= kTsFirstConvWarp && warp < kTsFirstConvWarp + kConvWarps) {
        // ------------------------------- converters -------------------------------
        // Converter warp c: TMEM lane quarter c & 3, operand stages j with j % 4 == c >> 2.  A thread owns one weight row.
        const int c = warp - kTsFirstConvWarp;
        const int qd = c & 3, cl = c >> 2;
        const uint32_t row_ofs = static_cast<uint32_t>(qd * 32 + lane) * p.raw_row_bytes;
        const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) + a_col0;
        bool ok = true;
        uint32_t jbase = 0;   // operand stages of the tiles already done
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, jbase += kstages) {
            // first stage of this tile that belongs to this warp's class
            for (uint32_t j = jbase + ((cl + 4u - (jbase & 3u)) & 3u); j < jbase + kstages; j += 4) {
                const uint32_t kt0 = j * KS;          // first K tile of the stage (KS divides KPR: one raw step per stage)
                const uint32_t r = kt0 / KPR;
                const int sub0 = static_cast<int>(kt0 % KPR);
                const uint32_t rslot = r % p.raw_stages, rpar = (r / p.raw_stages) & 1u;
                const uint32_t s = j & smask, use = j >> p.stage_shift;
                // The parity wait is exact: raw_stages is a power of two, so this warp (every fourth stage) meets every phase
                // of the raw slots it uses, and it has seen phase k - 1 of a slot complete before it waits for phase k.
                const bool got_raw = mbar_wait(&raw_full[rslot], rpar, abort_flag);
                if (!got_raw) {
                    if (lane == 0) fail(QWC_DEV_WAIT_FULL_TIMEOUT);
                    ok = false;
                    break;
                }
                const uint8_t* src = raw + rslot * raw_stage_bytes + row_ofs;
                uint32_t w[kTileWords];
                uint32_t a32[32];
                uint32_t w1[KS == 2 ? kTileWords : 1];
                load_tile_words<FMT>(src, sub0, w);
                if (KS == 2) load_tile_words<FMT>(src, sub0 + 1, w1);
                decode_tile_natural<FMT>(w, a32);
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rslot]);   // the packed words of the stage are in registers
                // only now wait for the operand stage: the decode above overlapped the MMAs that were reading it
                const bool got_empty = use == 0 || mbar_wait(&empty[s], (use - 1) & 1u, abort_flag);
                if (!got_empty) {
                    if (lane == 0) fail(QWC_DEV_WAIT_EMPTY_TIMEOUT);
                    ok = false;
                    break;
                }
                tc_fence_after();   // the MMAs that read this A stage are complete (tcgen05.commit -> empty[s])
                tmem_st32(lane_taddr + s * 32 * KS, a32);
                if (KS == 2) {
                    tmem_st_wait();   // the first store has read its registers
                    decode_tile_natural<FMT>(w1, a32);
                    tmem_st32(lane_taddr + s * 64 + 32, a32);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
    } else if (warp >= kTsFirstConvWarp + kConvWarps) {
        // ------------------------------- epilogue -------------------------------
        const int quarter = warp & 3;
        uint32_t tiles_done = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tiles_done) {
            const TileInfo ti = tc_get_tile(p, tile);
            const int as = tiles_done & 1;
            const bool got = mbar_wait_relaxed(&acc_full[as], (tiles_done >> 1) & 1, abort_flag);
            // The four warps decide together whether to go on: the SwiGLU epilogue meets at a named barrier per 16
            // tokens, so a warp that gave up alone would leave the others waiting there for ever.
            volatile int* verdict = epi_ok + (tiles_done & 1u) * 4;
            if (lane == 0) verdict[quarter] = got ? 1 : 0;
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (!(verdict[0] && verdict[1] && verdict[2] && verdict[3])) {
                if (lane == 0) fail(QWC_DEV_WAIT_MMA_TIMEOUT);
                break;
            }
            tc_fence_after();
            tc_epilogue_tile(p, ti, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(as * p.acc_stride), xch,
                             quarter, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

// Staging pre-pass of the tensor path: rows of ldx -> rows of ldo, rotated (FWHT-32 per unit) or copied.
__global__ void __launch_bounds__(256) qwc_rotate_rows_kernel(const __half* __restrict__ x, int64_t ldx, __half* __restrict__ out,
                                                              int64_t ldo, int64_t m, int64_t k, int rotate) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t units = k / 32, total = m * units;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t it = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); it < total; it += warps) {
        const int64_t r = it / units, u = it % units;
        const __half xin = x[r * ldx + u * 32 + lane];
        if (!rotate) {
            out[r * ldo + u * 32 + lane] = xin;
            continue;
        }
        float v = __half2float(xin);
#pragma unroll
        for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
        out[r * ldo + u * 32 + lane] = __float2half_rn(__fmul_rn(v, qwc_inv_sqrt32()));
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int FMT, int KS>
int launch_ts_inst(const qwc_hal* hal, cudaStream_t st, const TcParams& p, const CUtensorMap& wmap, const CUtensorMap& wmap64,
                   const CUtensorMap* xmaps, int smem, int grid) {
    // once per device and instantiation; racing first calls both set the same value, which is harmless
    static std::atomic<bool> configured[64];
    if (!configured[hal->device & 63].load(std::memory_order_acquire)) {
        QWC_CUDA_TRY(cudaFuncSetAttribute(qwc_gemm_ts_kernel<FMT, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured[hal->device & 63].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_gemm_ts_kernel<FMT, KS>, p, wmap, xmaps[0], xmaps[1], xmaps[2], wmap64));
    return QWC_OK;
}

template <int FMT>
int launch_ts(const qwc_hal* hal, cudaStream_t st, const TcParams& p, const CUtensorMap& wmap, const CUtensorMap& wmap64,
              const CUtensorMap* xmaps, int smem, int grid) {
    if (p.kt_per_stage == 2) return launch_ts_inst<FMT, 2>(hal, st, p, wmap, wmap64, xmaps, smem, grid);
    return launch_ts_inst<FMT, 1>(hal, st, p, wmap, wmap64, xmaps, smem, grid);
}

}  // namespace

// Can the tensor-core path take this call?  (K a multiple of one raw step, 16-byte aligned rows.)
bool qwc_gemm_tc_supported(const qwc_hal* hal, const qwc_weight_view* w, int64_t m, int epilogue) {
    const int fmt = qwc_fmt_of(*w);
    if (hal->encode_tiled == nullptr) return false;
    if (fmt == FMT_UNSUPPORTED) return false;
    // SwiGLU epilogues pair 64 gate rows with 64 up rows per tile
    if (epilogue != QWC_EPI_NONE && (w->n % 2 != 0 || (w->n / 2) % (kBM / 2) != 0)) return false;
    // 9 tokens and more (8 for HQ8_G32): below that the streaming kernel (register fragments, no decoded operand in memory)
    // wins (N = 17408, K = 5120, us per call, stream / tensor: HQ4_G32 8 tokens 19.0 / 19.1, 9 tokens 22.5 / 18.1; HQ8_G32
    // 4 tokens 25.3 / 33.5 (with so few activation rows the activation reads of all CTAs land on the same few lines, whatever
    // the row stride), 8 tokens 27.8 / 23.2; HQ4_G64 8 tokens 21.7 / 22.7, 9 tokens 23.7 / 22.7)
    if (w->k % (fmt == FMT_HQ4_G64 ? 256 : 128) != 0 || m < tune_env("QWC_TC_MIN_M", qwc_tc_min_tokens(fmt))) return false;
    if (reinterpret_cast<uintptr_t>(w->blocks) % 16 != 0) return false;
    return tune_env("QWC_NO_TCGEN05", 0) == 0;
}

// The activations are staged (rotated, or copied when they come rotated) into the caller's workspace when the caller passes
// standard-basis x, and always below 16 tokens.  Row stride of the staged copy: all CTAs read the same few activation rows
// at the same time, and measured on B200 those reads crawl when the rows span less than 128 KiB of addresses (N = 17408,
// K = 5120, rotated x: 25-28 us per call for 1..12 tokens, 15.9 us for 13 tokens and more, and 15.9 us for 8 tokens once the
// rows lie 20 KB apart), so short staged copies get a row stride that spreads them over 136 KiB.
static int64_t tc_stage_ld(int64_t k, int64_t m) {
    const int64_t span = 136 * 1024;
    if (m * k * 2 >= span) return k;
    const int64_t ld = (span / (2 * m) + 63) / 64 * 64;
    return ld > k ? ld : k;
}
static bool tc_stages_x(int64_t m, int x_is_rotated) { return !x_is_rotated || m < 16; }
size_t qwc_gemm_tc_workspace_bytes(const qwc_weight_view* w, int64_t m, int x_is_rotated) {
    return tc_stages_x(m, x_is_rotated) ? static_cast<size_t>(m) * static_cast<size_t>(tc_stage_ld(w->k, m)) * 2 : 0;
}

// Shared by the dense door and the grouped (MoE) door: tensor maps, shared-memory budget, launch.
static int tc_run(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const __half* xr, int64_t ldxr, int64_t m,
                  void* y, int y_dtype, int64_t ldy, const qwc_moe_tile* tiles, const int32_t* tile_count, int64_t max_tiles,
                  int x_tile_rows, int epilogue) {
    const int fmt = qwc_fmt_of(*w);
    TcParams p{};
    p.tiles = tiles;
    p.tile_count = tile_count;
    p.y = y;
    p.ldy = ldy;
    p.status = hal->status;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(w->n);
    p.k = static_cast<int>(w->k);
    p.y_f16 = y_dtype == QWC_F16;
    p.raw_row_bytes = fmt == FMT_HQ4_G32_M5 ? 80 : 144;
    if (tiles == nullptr) x_tile_rows = m <= 64 ? 64 : (m <= 128 ? 128 : kTsBN);   // dense: the narrowest tile that holds all tokens
    if (x_tile_rows > kTsBN) x_tile_rows = kTsBN;
    p.x_tile_rows = x_tile_rows;
    // Four operand stages.  The issue loop of the MMA warp costs a fixed ~0.2 us per stage (barrier wait, fence, commit), so a
    // stage of one 64-wide K tile paces the kernel whenever its MMAs are shorter than that: tiles of up to 128 tokens (expert
    // tiles, verify-sized calls) take 128 k per stage and narrower accumulators to make room in tensor memory.
    p.kt_per_stage = x_tile_rows <= 128 ? 2 : 1;
    if (const int ks_env = tune_env("QWC_TC_KS", 0); ks_env == 1 || (ks_env == 2 && x_tile_rows <= 128)) p.kt_per_stage = ks_env;
    p.stages = 4;
    if (p.kt_per_stage == 1 && x_tile_rows <= 128 && tune_env("QWC_TC_STAGES", 8) == 8) p.stages = kMaxStages;
    p.acc_stride = x_tile_rows <= 128 ? 128 : kTsBN;
    p.stage_shift = p.stages == kMaxStages ? 3 : 2;
    p.m_tiles = static_cast<int>((m + x_tile_rows - 1) / x_tile_rows);
    p.epilogue = epilogue;
    p.up_delta = static_cast<int>(w->n / 2);
    p.xch_bytes = epilogue == QWC_EPI_NONE ? 0 : (kBM / 2) * 32 * 2;   // 64 rows x 16 parked tokens (f16) per side
    p.n_tiles = epilogue == QWC_EPI_NONE ? static_cast<int>((w->n + kBM - 1) / kBM) : static_cast<int>(w->n / kBM);
    const int raw_stage_bytes = ((kBM * p.raw_row_bytes + 127) / 128) * 128;
    p.x_slot_bytes = p.kt_per_stage * x_tile_rows * kBK * 2;
    p.raw_stages = kTsMaxRaw;
    auto smem_need = [&](int rs) { return 1024 + p.stages * p.x_slot_bytes + rs * raw_stage_bytes + 512 + p.xch_bytes; };
    while (smem_need(p.raw_stages) > 227 * 1024 && p.raw_stages > 2) p.raw_stages >>= 1;   // a power of two (see the converters' raw wait)
    if (smem_need(p.raw_stages) > 227 * 1024) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "shared-memory budget exceeded");
    const int smem = smem_need(p.raw_stages);

    const EncodeFn enc = reinterpret_cast<EncodeFn>(hal->encode_tiled);
    alignas(64) CUtensorMap wmaps[2];   // packed-weight boxes of 128 rows and (SwiGLU epilogues) 64 rows
    alignas(64) CUtensorMap xmaps[3];   // activation boxes of x_tile_rows, 128 and 64 rows
    const int64_t row_bytes = (w->k / w->group) * qwc_block_bytes(w->kind, w->bits, w->group);
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(row_bytes / 8), static_cast<cuuint64_t>(w->n)};
        const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(row_bytes)};
        cuuint32_t box[2] = {static_cast<cuuint32_t>(p.raw_row_bytes / 8), static_cast<cuuint32_t>(i == 0 ? kBM : kBM / 2)};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = enc(&wmaps[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(w->blocks), gdim, gstride, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return qwc_fail(QWC_ERR_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", static_cast<int>(cr));
    }
    for (int i = 0; i < 3; ++i) {
        const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(w->k), static_cast<cuuint64_t>(m)};
        const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ldxr * 2)};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(i == 0 ? x_tile_rows : (i == 1 ? 128 : 64))};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = enc(&xmaps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xr), gdim, gstride, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return qwc_fail(QWC_ERR_CUDA, "cuTensorMapEncodeTiled(activations) failed with %d", static_cast<int>(cr));
    }
    const int64_t ntiles = tiles != nullptr ? max_tiles : static_cast<int64_t>(p.m_tiles) * p.n_tiles;
    const int grid = static_cast<int>(ntiles < hal->sm_count ? (ntiles < 1 ? 1 : ntiles) : hal->sm_count);
    if (fmt == FMT_HQ4_G32_M5) return launch_ts<FMT_HQ4_G32_M5>(hal, st, p, wmaps[0], wmaps[1], xmaps, smem, grid);
    if (fmt == FMT_HQ8_G32) return launch_ts<FMT_HQ8_G32>(hal, st, p, wmaps[0], wmaps[1], xmaps, smem, grid);
    return launch_ts<FMT_HQ4_G64>(hal, st, p, wmaps[0], wmaps[1], xmaps, smem, grid);
}

// Validation shared with the callers that must refuse before their first launch.
int qwc_gemm_tc_check(const qwc_weight_view* w, const void* x, int64_t ldx, int64_t m, int x_is_rotated, const void* workspace,
                      size_t workspace_bytes) {
    if (tc_stages_x(m, x_is_rotated)) {
        const size_t need = qwc_gemm_tc_workspace_bytes(w, m, x_is_rotated);
        if (workspace == nullptr || workspace_bytes < need)
            return qwc_fail(QWC_ERR_BAD_SHAPE, "workspace of %zu bytes needed (qwc_gemm_workspace_bytes), got %zu", need, workspace_bytes);
        if (reinterpret_cast<uintptr_t>(workspace) % 16 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "workspace must be 16-byte aligned");
    } else if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || ldx % 8 != 0) {
        return qwc_fail(QWC_ERR_BAD_SHAPE, "rotated activations must be 16-byte aligned with ldx %% 8 == 0 for the tensor-core path");
    }
    return QWC_OK;
}

int qwc_launch_gemm_tc(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx,
                       void* y, int y_dtype, int64_t ldy, int epilogue, int x_is_rotated, void* workspace, size_t workspace_bytes) {
    if (int rc = qwc_gemm_tc_check(w, x, ldx, m, x_is_rotated, workspace, workspace_bytes)) return rc;
    const __half* xr = static_cast<const __half*>(x);
    int64_t ldxr = ldx;
    if (tc_stages_x(m, x_is_rotated)) {
        int64_t blocks = (m * (w->k / 32) + 7) / 8;
        if (blocks > hal->sm_count * 16) blocks = hal->sm_count * 16;
        ldxr = tc_stage_ld(w->k, m);
        qwc_rotate_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(xr, ldx, static_cast<__half*>(workspace), ldxr, m, w->k,
                                                                             x_is_rotated ? 0 : 1);
        QWC_CUDA_TRY(cudaGetLastError());
        xr = static_cast<const __half*>(workspace);
    }
    return tc_run(hal, st, w, xr, ldxr, m, y, y_dtype, ldy, nullptr, nullptr, 0, kTsBN, epilogue);
}

// Grouped expert GEMM: the same kernel over a device-side tile list (see qwc_moe_group_pairs).
int qwc_launch_gemm_tc_grouped(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* bank, const void* xs, int64_t pairs,
                               const qwc_moe_tile* tiles, const int32_t* tile_count, int64_t max_tiles, void* y, int y_dtype,
                               int64_t ldy, int x_tile_rows, int epilogue) {
    return tc_run(hal, st, bank, static_cast<const __half*>(xs), bank->k, pairs, y, y_dtype, ldy, tiles, tile_count, max_tiles,
                  x_tile_rows, epilogue);
}
