// Decode GEMV (M = 1) and small-M verify GEMM (M <= 16) over packed HQ blocks: the CUDA twin of the reference's
// qwg_gemv_q4g_* / qwg_gemv_aq* / qwg_skinny_m* / qwm_mlp_*_m* kernel families
// (Sources/QWMetal/gemm/qwgemm.metal, qwgemm_aq.metal, qwg_skinny.metal, Sources/QWMetal/mtp/qwmtp_mlp.metal).
//
// The path is bound by HBM: every weight byte is read exactly once.  Design:
//  * one persistent CTA per SM owns a contiguous range of output rows.  A producer warp streams the packed rows,
//    unchanged, into a ring of shared-memory stages: 16 rows x one K chunk per stage, one 2-D tensor copy (TMA) per
//    stage with an mbarrier transaction count (per-row 1-D bulk copies for ragged tail tiles); rows are padded by 16 B
//    and chunks are multiples of 8 units so per-lane word reads hit 32 distinct banks.  A slot of the ring is shared
//    by the teams, so a fill counter published by the producer guards the parity waits (see the consumer loop);
//  * the activations are rotated (FWHT-32, f32 butterflies, one rounding to f16) once per CTA into shared memory,
//    stored in the k order and 16-byte-chunk swizzle the fragment loads want;
//  * the 16 consumer warps form T teams of W warps.  A team owns one 16-row tile at a time (all K chunks), so the
//    accumulators stay in registers for the whole tile; teams work on different tiles concurrently.  Inside a team
//    the 4-unit groups of a chunk are dealt round-robin to the warps; the W partial tiles are summed in a fixed
//    order through shared memory (deterministic);
//  * each lane decodes one whole block per row (5 or 9 word loads, one header) straight into m16n8k16 A fragments
//    by the magic-bias form (0x6400 | q as f16 = 1024 + q, then one f16 FMA with scale and bias: the reference's
//    decode class, Sources/QWMetal/include/qw_dequant.metalh:53-61); the dot products run on mma.sync with f32
//    accumulate.  A SIMT FMA dot needs > 3 issue slots per weight and cannot keep up with the copy stream.  The k
//    slots of an MMA are permuted (4 k from each of the 4 units a quad holds), which A and B share, so no shuffle
//    is needed between the packed layout and the fragment layout.
// Three optional forms of the same kernel: static-weights mode (programmatic dependent launch: the producer streams
// weights while the previous kernel of the stream finishes), segment mode (CTA b serves entry b of a device-side list
// of (expert bank rows, tokens) — the decode-time mixture of experts), and the fused all-reduce epilogue (row-parallel
// shards of a tensor-parallel group: peer stores into every rank's inbox, flags, rank-ordered sum).
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "qwc_common.cuh"

namespace {

#ifndef QWC_GEMV_CONSUMER_WARPS
#define QWC_GEMV_CONSUMER_WARPS 16
#endif
#ifndef QWC_GEMV_SMEM_KB
#define QWC_GEMV_SMEM_KB 227
#endif
constexpr int kConsumerWarps = QWC_GEMV_CONSUMER_WARPS;
constexpr int kCtasPerSm = QWC_GEMV_SMEM_KB <= 113 ? 2 : 1;   // half the shared memory: a second CTA (the next call's) fits beside this one
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + one producer warp
constexpr int kTileRows = 16;
constexpr int kMaxStages = 24;
constexpr int kRowPad = 16;  // smem row stride = chunk bytes + 16: (stride / 4) % 32 == 4 -> conflict-free word reads
constexpr int kSmemBudget = QWC_GEMV_SMEM_KB * 1024;
constexpr int kBarrierBytes = 512;  // 2 x kMaxStages mbarriers + the abort flag, padded to keep the stages 128-byte aligned

template <int FMT> struct StreamCfg;
template <> struct StreamCfg<FMT_HQ4_G32_M5> { static constexpr int kUnitBytes = 20, kGroupUnits = 4; };
template <> struct StreamCfg<FMT_HQ8_G32> { static constexpr int kUnitBytes = 36, kGroupUnits = 4; };
template <> struct StreamCfg<FMT_HQ4_G64> { static constexpr int kUnitBytes = 18, kGroupUnits = 4; };

// One unit of work of the segment mode: output columns [col0, col0 + cols) of one expert (weight rows w_row0 + col,
// plus n_out for the up half of a paired bank), for the m expert-sorted rows starting at x_row0 (same rows of y).
struct qwc_gemv_seg {
    int32_t w_row0, col0, cols, x_row0, m, pad0, pad1, pad2;
};

struct GemvParams {
    const uint8_t* blocks;
    int64_t row_bytes;
    const __half* x;
    int64_t ldx;
    void* y;
    int64_t ldy;
    float* partial;   // [m, n] f32 raw dot products carried between the K slices of one call (may be null)
    int32_t* status;
    int n;            // weight rows
    int n_out;        // output rows (n, or n/2 for the silu-pair epilogues)
    int m;            // tokens, <= 8 * NT
    int unit0;        // first 32-element unit of this launch's K slice
    int units;        // units in this launch's K slice
    int nchunks;      // K chunks per tile
    int chunk_units;  // units per chunk (the last chunk may be shorter)
    int stages;       // ring depth
    int stride;       // smem row stride in bytes
    int team_warps;   // W
    int y_f16;
    int epilogue;
    int x_is_rotated;
    int acc_in;       // add `partial` before the epilogue
    int acc_out;      // store raw sums to `partial` instead of y
    int row_quantum;  // CTA row ranges start on multiples of this (32 for the fused-FWHT epilogue)
    int q_lo, q_rem;  // (n_out / row_quantum) / grid and % grid: how the row quanta are dealt to the CTAs
    int x_bytes;      // smem bytes of the activation region
    int red_bytes;    // smem bytes of the team reduction region
    int pdl;          // launched with programmatic stream serialization: weights prefetch before the dependency wait
    int use_tmap;     // full 16-row tiles arrive by one 2-D tensor copy instead of 16 row copies
    int l2_evict_first;  // the weight stream is read once: mark its lines evict-first so that what a prefetch kernel
                         // brought in for the next call outlives them in L2
    // segment mode (see the kernel): null in the ordinary one-bank form
    const qwc_gemv_seg* segs;
    const int32_t* seg_count;
    int seg_grid, seg_cols;   // host side: capacity of the list (= grid) and output columns per entry
    // fused one-shot all-reduce over peer memory (row-parallel shards of a tensor-parallel group; ar_world > 1):
    int ar_world, ar_rank;
    uint32_t ar_epoch;        // call number: the tag that marks a slot as holding this call's value (never 0)
    uint64_t ar_wait_ns;      // limit of the peer wait (0: the library's default)
    uint32_t* ar_state;       // device-side call counter (see qwc_allreduce_ctx::epoch_state); null: ar_epoch comes from the host
    int64_t ar_inbox_stride;  // distance between the two inbox buffers (floats) when the kernel picks the buffer
    float* ar_inbox[8];       // rank r's inbox for this call: [world][m][n] slots of (f32 value, u32 call number); [s] is written by rank s
};

// Shared-memory loads by 32-bit shared-window address (no 64-bit pointer arithmetic in the inner loop).
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, __half2 s2, __half2 b2) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), s2, b2);
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hfma2_k(uint32_t a, uint32_t mul, uint32_t add) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&mul),
                              *reinterpret_cast<const __half2*>(&add));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hsub2_1024(uint32_t a) {
    const uint32_t k = 0x64006400u;
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&k));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// (v & mask) | 0x64006400 as one three-input logic op.  With mask 0x000F000F the two nibbles become the f16 pair
// (1024 + q, 1024 + q'); with mask 0x00F000F0 the nibbles four bits up become (1024 + 16 q, 1024 + 16 q').
template <uint32_t MASK> __device__ __forceinline__ uint32_t nib2_f16x2(uint32_t v) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(MASK), "r"(0x64006400u));
    return d;
}
constexpr uint32_t kH2Sixteenth = 0x2C002C00u;   // f16x2 (1/16, 1/16)
constexpr uint32_t kH2_960 = 0x63806380u;        // f16x2 (960, 960)
constexpr uint32_t kH2_m64 = 0xD400D400u;        // f16x2 (-64, -64)

// Decode one whole unit (32 k of one row) into 16 f16x2 registers a[P], P = pair index.  The k each pair holds
// is fixed per format (natural order for HQ4_G32_M5 / HQ8_G32; (8w+p, 8w+p+4) for the linear-nibble HQ4_G64) and
// the activation staging writes x in the same order.  ublk = shared address of the unit's header word; wofs =
// byte offset of the unit's first payload word from the header.
//
// The integer/logic pipe is the scarce resource of this kernel (it runs at half the rate of the FMA pipe), so only
// one shift per word is spent there: the nibbles at bits 4..7 of a byte are taken in place as 1024 + 16 q and brought
// to 1024 + q by an exact f16 FMA (x / 16 + 960), which leaves every decoded weight bit-identical to the one-FMA
// form (1024 + q) * scale + bias of the reference (Sources/QWMetal/include/qw_dequant.metalh:53-61).
template <int FMT>
__device__ __forceinline__ void decode_unit(uint32_t ublk, int wofs, uint32_t a[16]) {
    const uint32_t hdr = lds32(ublk);
    const __half2 h = *reinterpret_cast<const __half2*>(&hdr);
    const __half2 s2 = __half2half2(__low2half(h)), b2 = __half2half2(__high2half(h));
    const uint32_t pay = ublk + wofs;
    if (FMT == FMT_HQ4_G32_M5) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t v = lds32(pay + 4 * w), v8 = v >> 8;
            a[4 * w] = hfma2_u32(nib2_f16x2<0x000F000Fu>(v), s2, b2);
            a[4 * w + 1] = hfma2_u32(hfma2_k(nib2_f16x2<0x00F000F0u>(v), kH2Sixteenth, kH2_960), s2, b2);
            a[4 * w + 2] = hfma2_u32(nib2_f16x2<0x000F000Fu>(v8), s2, b2);
            a[4 * w + 3] = hfma2_u32(hfma2_k(nib2_f16x2<0x00F000F0u>(v8), kH2Sixteenth, kH2_960), s2, b2);
        }
    } else if (FMT == FMT_HQ8_G32) {
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const uint32_t v = lds32(pay + 4 * w);
            a[2 * w] = hfma2_u32(hsub2_1024(__byte_perm(v, 0x64646464u, 0x4140)), s2, b2);
            a[2 * w + 1] = hfma2_u32(hsub2_1024(__byte_perm(v, 0x64646464u, 0x4342)), s2, b2);
        }
    } else {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t v = lds32(pay + 4 * w), v8 = v >> 8;
            a[4 * w] = hfma2_u32(hsub2_1024(nib2_f16x2<0x000F000Fu>(v)), s2, b2);
            a[4 * w + 1] = hfma2_u32(hfma2_k(nib2_f16x2<0x00F000F0u>(v), kH2Sixteenth, kH2_m64), s2, b2);
            a[4 * w + 2] = hfma2_u32(hsub2_1024(nib2_f16x2<0x000F000Fu>(v8)), s2, b2);
            a[4 * w + 3] = hfma2_u32(hfma2_k(nib2_f16x2<0x00F000F0u>(v8), kH2Sixteenth, kH2_m64), s2, b2);
        }
    }
}

__device__ __forceinline__ void mma_16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2-D tiled tensor copy global -> shared, completion counted on an mbarrier.  x is in elements of the map's data
// type (8-byte here, so x must be even: the copy starts on a 16-byte boundary); y is the row.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Release store of a shared-memory word (CTA scope).
__device__ __forceinline__ void st_release_cta(uint32_t* p, uint32_t v) {
    asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Byte offset of (token, unit, 16-byte chunk c) in the staged activations: chunks are xor-swizzled so that the
// four lanes of a quad (units u..u+3, or u, u+2, u+4, u+6) and two adjacent tokens hit 8 distinct 16-byte bank groups.
template <int FMT> __device__ __forceinline__ int x_offset(int tok, int unit, int c, int units) {
    const int usel = FMT == FMT_HQ4_G64 ? (unit >> 1) : unit;
    return (tok * units + unit) * 64 + ((c ^ (usel & 3) ^ (tok & 1)) << 4);
}

template <int FMT, int NT, int SUB>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
qwc_gemv_stream_kernel(const GemvParams p, const __grid_constant__ CUtensorMap tmap) {
    using C = StreamCfg<FMT>;
    if (p.segs != nullptr) {
        // The segment list is the work of a kernel earlier in the stream: a programmatic launch must wait for it
        // before the first read (nothing can be prefetched without the list anyway).
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (static_cast<int>(blockIdx.x) >= *p.seg_count) return;   // whole CTA: nothing is set up yet
    }
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: [x region][reduction region][barriers][stages...]
    uint8_t* xs = smem;
    float4* red = reinterpret_cast<float4*>(smem + p.x_bytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.x_bytes + p.red_bytes);
    uint64_t* empty = full + kMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
    uint32_t* issued = reinterpret_cast<uint32_t*>(empty + kMaxStages) + 1;   // fills the producer has started
    uint8_t* stage0 = smem + p.x_bytes + p.red_bytes + kBarrierBytes;  // 128-byte aligned
    const int stage_bytes = kTileRows * p.stride;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = p.team_warps, T = kConsumerWarps / W;
    // The producer warp initialises the barriers and goes straight on to fill the ring; the consumers meet it at
    // named barrier 10 only after they have staged the activations, so nobody waits for anybody at kernel start.
    if (warp == kConsumerWarps) {
        if (lane < p.stages) {
            mbar_init(&full[lane], 1);
            mbar_init(&empty[lane], W);
        }
        if (lane == 0) {
            *abort_flag = 0;
            *issued = 0;
            if (p.use_tmap) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap)) : "memory");
        }
        fence_barrier_init();
        __syncwarp();
        asm volatile("bar.arrive 10, %0;" ::"r"(kThreads) : "memory");
    }

    // This CTA's output rows [rb, re) and its jobs: one job = 16 output rows (32 for the fused-FWHT epilogue) =
    // SUB weight sub-tiles of 16 rows.  Job i goes to team i % T in round i / T.  The row quanta are dealt evenly,
    // the first q_rem CTAs taking one more.
    const int bq = static_cast<int>(blockIdx.x);
    int rb = (p.q_lo * bq + min(bq, p.q_rem)) * p.row_quantum;
    int re = rb + (p.q_lo + (bq < p.q_rem ? 1 : 0)) * p.row_quantum;
    // Segment mode (decode-time mixture of experts): CTA b serves entry b of a device-side list, each entry one expert's
    // weight rows [w_row0 + col0, ...) of a stacked bank, that expert's few tokens, and its own rows of x and y.
    int M_ = p.m;
    const __half* X_ = p.x;
    void* Y_ = p.y;
    int64_t wbase = 0;   // weight row of output column 0
    if (p.segs != nullptr) {
        const qwc_gemv_seg sg = p.segs[bq];   // the host launches exactly *seg_count CTAs' worth or more; extra CTAs left above
        rb = sg.col0;
        re = sg.col0 + sg.cols;
        M_ = sg.m;
        X_ = p.x + static_cast<int64_t>(sg.x_row0) * p.ldx;
        Y_ = static_cast<char*>(p.y) + static_cast<int64_t>(sg.x_row0) * p.ldy * (p.y_f16 ? 2 : 4);
        wbase = sg.w_row0;
    }
    constexpr int kJobRows = SUB == 4 ? 32 : 16;
    const int njobs = (re - rb + kJobRows - 1) / kJobRows;
    const int E = SUB * p.nchunks;  // stage fills per job
    const int rounds = (njobs + T - 1) / T;

    // Weight row of (job, sub-tile): SUB 1: rows; SUB 2: gate, up; SUB 4: gate lo, gate hi, up lo, up hi.
    auto first_weight_row = [&](int job, int sub, int& valid) {
        const int out0 = rb + job * kJobRows + (SUB == 4 ? (sub & 1) * 16 : 0);
        valid = min(kTileRows, re - out0);
        const bool up = SUB == 2 ? sub == 1 : (SUB == 4 ? sub >= 2 : false);
        return wbase + static_cast<int64_t>(out0) + (up ? p.n_out : 0);
    };

    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------
        uint32_t q = 0;
        int pslot = 0;
        uint32_t pparity = 0;  // phase parity of fill q in its slot
        bool ok = true;
        uint64_t policy = 0;
        if (p.l2_evict_first) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        for (int r = 0; r < rounds && ok; ++r) {
            const int tl = min(T, njobs - r * T);
            for (int e = 0, sub = 0, c = 0; e < E && ok; ++e, ++c) {
                if (c == p.nchunks) {
                    c = 0;
                    ++sub;
                }
                const int u0 = c * p.chunk_units;
                const uint32_t cbytes = static_cast<uint32_t>(min(p.chunk_units, p.units - u0)) * C::kUnitBytes;
                for (int tau = 0; tau < tl; ++tau, ++q) {
                    const int slot = pslot;
                    const uint32_t wait_parity = pparity ^ 1u;  // phase of the previous use of this slot
                    if (++pslot == p.stages) {
                        pslot = 0;
                        pparity ^= 1u;
                    }
                    if (q >= static_cast<uint32_t>(p.stages)) {
                        if (*abort_flag || !mbar_wait(&empty[slot], wait_parity, abort_flag)) {
                            if (!*abort_flag && lane == 0) atomicCAS(p.status, 0, QWC_DEV_WAIT_EMPTY_TIMEOUT);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    int valid;
                    const int64_t wrow = first_weight_row(r * T + tau, sub, valid);
                    if (valid <= 0) {
                        // sub-tile past the CTA's rows (second half of a short FWHT job): nothing to copy
                        if (lane == 0) {
                            mbar_arrive(&full[slot]);
                            st_release_cta(issued, q + 1);
                        }
                        continue;
                    }
                    if (p.use_tmap && valid == kTileRows) {
                        // one 2-D tensor copy per stage: 16 rows x (chunk + 16 pad bytes), rows land `stride` apart
                        if (lane == 0) {
                            mbar_arrive_expect_tx(&full[slot], static_cast<uint32_t>(stage_bytes));
                            st_release_cta(issued, q + 1);
                            const int tx = static_cast<int>((static_cast<int64_t>(p.unit0 + u0) * C::kUnitBytes) >> 3);
                            if (p.l2_evict_first)
                                tma_load_2d_hint(stage0 + slot * stage_bytes, &tmap, tx, static_cast<int>(wrow), &full[slot], policy);
                            else
                                tma_load_2d(stage0 + slot * stage_bytes, &tmap, tx, static_cast<int>(wrow), &full[slot]);
                        }
                        continue;
                    }
                    if (lane == 0) {
                        mbar_arrive_expect_tx(&full[slot], cbytes * valid);
                        st_release_cta(issued, q + 1);
                    }
                    __syncwarp();
                    if (lane < valid) {
                        const uint8_t* src = p.blocks + (wrow + lane) * p.row_bytes +
                                             static_cast<int64_t>(p.unit0 + u0) * C::kUnitBytes;
                        bulk_g2s(stage0 + slot * stage_bytes + lane * p.stride, src, cbytes, &full[slot]);
                    }
                }
            }
        }
        // After a failed wait the consumers stop draining: let this CTA's own copies land (bounded) before exit.
        if (!ok && lane == 0) {
            for (uint32_t s = 0; s < static_cast<uint32_t>(p.stages) && s < q; ++s) {
                const uint32_t last = ((q - 1 - s) / p.stages) * p.stages + s;
                mbar_wait(&full[s], (last / p.stages) & 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // Everything that needs no global data is set up first: under programmatic dependent launch it runs while the
    // previous grid of the stream is still finishing.
    const int gid = lane >> 2, t = lane & 3;
    const int team = warp / W, wj = warp % W;
    const int team_threads = W * 32;
    const uint32_t xs_a = smem_u32(xs), stage0_a = smem_u32(stage0);
    // Per-lane constants of the activation fragment loads: the chunk swizzle depends only on (t, token parity)
    // because chunk starts and group starts are multiples of 4 units (8 for HQ4_G64).
    uint32_t xtok[NT];
    int xsw[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int tok = min(nt * 8 + gid, M_ - 1);
        xtok[nt] = xs_a + static_cast<uint32_t>(tok) * p.units * 64;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) xsw[nt][cc] = (cc ^ t ^ (tok & 1)) << 4;
    }
    // this lane's unit inside a chunk for group wj (advances by W groups), as byte offsets into the row / x
    int hofs0, wofs, xofs0;
    if (FMT == FMT_HQ4_G64) {
        const int ul = 8 * (wj >> 1) + (wj & 1) + 2 * t;  // even units, then odd units, of an 8-unit span
        hofs0 = (ul >> 1) * 36;
        wofs = 4 + 16 * (ul & 1);
        xofs0 = ul * 64;
    } else {
        const int ul = 4 * wj + t;
        hofs0 = ul * C::kUnitBytes;
        wofs = 4;
        xofs0 = ul * 64;
    }
    // HQ4_G64 with odd W would alternate the unit parity between steps; the host only picks W = 1 there when
    // forced, and the general form in the loop handles it by recomputing the offsets per group.
    const bool g64_recompute = FMT == FMT_HQ4_G64 && (W & 1);
    const int hstep = FMT == FMT_HQ4_G64 ? (W >> 1) * 4 * 36 : W * 4 * C::kUnitBytes;  // W groups further along the row
    const int xstep = W * 4 * 64;
    const int row_ofs = gid * p.stride + hofs0, hi_ofs = 8 * p.stride;

    // Staging of the rotated activations, once per CTA.  A quad handles one (token, unit): lane t holds elements
    // 8t..8t+7, rotates them with three in-lane butterfly stages and two xor-shuffle stages (the reference's
    // h = 1, 2, 4, 8, 16 order), and writes one 16-byte chunk.  Items are taken two at a time so that both global
    // loads are in flight together.
    const int t4 = lane & 3, sub8 = lane >> 2;
    const int items = M_ * p.units;  // (token, unit) pairs
    const bool vec_ok = (reinterpret_cast<uintptr_t>(X_) % 16 == 0) && (p.ldx % 8 == 0);
    struct StageItem {
        const __half* src;
        int tok, unit;
        bool live;
    };
    auto make_item = [&](int it) {
        StageItem si;
        si.live = it < items;
        si.tok = si.live ? it / p.units : 0;
        si.unit = si.live ? it - si.tok * p.units : 0;
        si.src = X_ + si.tok * p.ldx + static_cast<int64_t>(p.unit0 + si.unit) * 32 + 8 * t4;
        return si;
    };
    auto load_item = [&](const StageItem& si) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (si.live) {
            if (vec_ok) raw = *reinterpret_cast<const uint4*>(si.src);
            else {
                __half tmp[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) tmp[i] = si.src[i];
                raw = *reinterpret_cast<const uint4*>(tmp);
            }
        }
        return raw;
    };
    auto finish_item = [&](const StageItem& si, uint4 raw) {
        __half2 hv[4] = {*reinterpret_cast<__half2*>(&raw.x), *reinterpret_cast<__half2*>(&raw.y),
                         *reinterpret_cast<__half2*>(&raw.z), *reinterpret_cast<__half2*>(&raw.w)};
        if (!p.x_is_rotated) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(hv[i]); f[2 * i + 1] = __high2float(hv[i]); }
#pragma unroll
            for (int h = 1; h < 8; h <<= 1)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if ((i & h) == 0) {
                        const float u = f[i], v = f[i + h];
                        f[i] = __fadd_rn(u, v);
                        f[i + h] = __fsub_rn(u, v);
                    }
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 1, (t4 & 1) != 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 2, (t4 & 2) != 0);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                hv[i] = __floats2half2_rn(__fmul_rn(f[2 * i], qwc_inv_sqrt32()), __fmul_rn(f[2 * i + 1], qwc_inv_sqrt32()));
        }
        if (si.live) {
            uint4 outv;
            if (FMT == FMT_HQ4_G64) {
                // slot order inside a chunk: e0 e4 e1 e5 e2 e6 e3 e7
                outv.x = __byte_perm(*reinterpret_cast<uint32_t*>(&hv[0]), *reinterpret_cast<uint32_t*>(&hv[2]), 0x5410);
                outv.y = __byte_perm(*reinterpret_cast<uint32_t*>(&hv[0]), *reinterpret_cast<uint32_t*>(&hv[2]), 0x7632);
                outv.z = __byte_perm(*reinterpret_cast<uint32_t*>(&hv[1]), *reinterpret_cast<uint32_t*>(&hv[3]), 0x5410);
                outv.w = __byte_perm(*reinterpret_cast<uint32_t*>(&hv[1]), *reinterpret_cast<uint32_t*>(&hv[3]), 0x7632);
            } else {
                outv = make_uint4(*reinterpret_cast<uint32_t*>(&hv[0]), *reinterpret_cast<uint32_t*>(&hv[1]),
                                  *reinterpret_cast<uint32_t*>(&hv[2]), *reinterpret_cast<uint32_t*>(&hv[3]));
            }
            *reinterpret_cast<uint4*>(xs + x_offset<FMT>(si.tok, si.unit, t4, p.units)) = outv;
        }
    };
    constexpr int kItemStride = kConsumerWarps * 8;
    StageItem ia = make_item(warp * 8 + sub8), ib = make_item(warp * 8 + sub8 + kItemStride);

    // Under programmatic dependent launch this grid may have started before the previous grid of the stream finished:
    // everything the previous grid may have produced (activations, outputs, the K-slice scratch) is touched only after
    // this point.  The producer warp above does not wait: packed weights are load-time data.
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    // Fused all-reduce with a device-side call counter: the call number is read here (the previous call of the stream
    // has completed), and its parity picks one of the two inbox / flag buffers.
    uint32_t ar_epoch = p.ar_epoch;
    int64_t ar_inbox_ofs = 0;
    if (SUB == 1 && p.ar_world > 1 && p.ar_state != nullptr) {
        ar_epoch = *reinterpret_cast<volatile uint32_t*>(p.ar_state) + 1u;
        ar_inbox_ofs = (ar_epoch & 1u) ? p.ar_inbox_stride : 0;
    }
    for (int base = warp * 8; base < items; base += 2 * kItemStride) {
        const uint4 ra = load_item(ia), rb4 = load_item(ib);
        const StageItem na = make_item(base + 2 * kItemStride + sub8), nb = make_item(base + 3 * kItemStride + sub8);
        finish_item(ia, ra);
        finish_item(ib, rb4);
        ia = na;
        ib = nb;
    }
    named_bar_sync(9, kConsumerWarps * 32);
    named_bar_sync(10, kThreads);   // the producer arrived here after initialising the barriers

    bool ok = true;
    const int ET = E * T;
    for (int r = 0; r < rounds; ++r) {
        const int job = r * T + team;
        const int tl = min(T, njobs - r * T);
        if (job >= njobs) break;  // uniform inside a team
        float d[SUB][NT][2][4];
#pragma unroll
        for (int s = 0; s < SUB; ++s)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) d[s][nt][h][i] = 0.0f;

        // Ring position of this team's first fill of the job; it advances by tl (the teams active in this round)
        // per fill, so slot and phase parity are kept incrementally (no division in the loop).
        uint32_t qn = static_cast<uint32_t>(r) * ET + team;   // index of this team's next fill in the producer's order
        int slot = team;
        uint32_t parity = 0;
        if (r > 0) {
            slot = qn % p.stages;
            parity = (qn / p.stages) & 1;
        }
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
            for (int c = 0; c < p.nchunks; ++c) {
                if (ok) {
                    // A slot is shared by teams: successive phases of full[slot] belong to different teams, and a parity
                    // wait cannot tell phase k from phase k - 2.  So first wait until the producer has started fill qn
                    // (it does that only after phase k - 1 of the slot was consumed); from then on the barrier is in
                    // phase k or past it and the parity wait is exact.
                    ok = wait_counter_above(issued, qn, abort_flag) && mbar_wait(&full[slot], parity, abort_flag);
                    if (!ok) {
                        *abort_flag = 1;
                        if (lane == 0) atomicCAS(p.status, 0, QWC_DEV_WAIT_FULL_TIMEOUT);
                    }
                }
                const int u0 = c * p.chunk_units;
                const int cu = min(p.chunk_units, p.units - u0);
                if (ok) {
                    uint32_t row_lo = stage0_a + slot * stage_bytes + row_ofs;
                    uint32_t xu[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) xu[nt] = xtok[nt] + u0 * 64 + xofs0;
                    const int ngroups = cu / C::kGroupUnits;
                    for (int g = wj; g < ngroups; g += W) {
                        int wo = wofs;
                        if (g64_recompute) {
                            const int ul = 8 * (g >> 1) + (g & 1) + 2 * t;
                            row_lo = stage0_a + slot * stage_bytes + gid * p.stride + (ul >> 1) * 36;
                            wo = 4 + 16 * (ul & 1);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) xu[nt] = xtok[nt] + (u0 + ul) * 64;
                        }
                        uint32_t alo[16], ahi[16];
                        decode_unit<FMT>(row_lo, wo, alo);
                        decode_unit<FMT>(row_lo + hi_ofs, wo, ahi);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            uint4 xv[4];
#pragma unroll
                            for (int cc = 0; cc < 4; ++cc) xv[cc] = lds128(xu[nt] + xsw[nt][cc]);
                            const uint32_t* xp = reinterpret_cast<const uint32_t*>(xv);
#pragma unroll
                            for (int s = 0; s < 8; ++s)
                                mma_16816(d[sub][nt][s & 1], alo[2 * s], ahi[2 * s], alo[2 * s + 1], ahi[2 * s + 1],
                                          xp[2 * s], xp[2 * s + 1]);
                            xu[nt] += xstep;
                        }
                        row_lo += hstep;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
                qn += tl;
                slot += tl;
                if (slot >= p.stages) {
                    slot -= p.stages;
                    parity ^= 1u;
                }
            }
        }

        // ---- team reduction (fixed order) and epilogue ----
        // red layout per team: [warp_in_team][sub][nt][lane] float4
        float4* tred = red + static_cast<size_t>(team) * W * SUB * NT * 32;
#pragma unroll
        for (int s = 0; s < SUB; ++s)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                tred[((wj * SUB + s) * NT + nt) * 32 + lane] =
                    make_float4(d[s][nt][0][0] + d[s][nt][1][0], d[s][nt][0][1] + d[s][nt][1][1],
                                d[s][nt][0][2] + d[s][nt][1][2], d[s][nt][0][3] + d[s][nt][1][3]);
        if (W > 1) named_bar_sync(1 + team, team_threads); else __syncwarp();

        const int out0 = rb + job * kJobRows;
        constexpr int kOutTiles = SUB == 4 ? 2 : 1;  // 16-row output tiles per job
        float* hbuf = reinterpret_cast<float*>(tred);  // reused after the sums are in registers (FWHT epilogue)
        float hval[kOutTiles][NT][4];
        bool mine[kOutTiles][NT];
#pragma unroll
        for (int ot = 0; ot < kOutTiles; ++ot)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mine[ot][nt] = (ot * NT + nt) % W == wj;  // spread the (ot, nt) tiles over the team's warps
#pragma unroll
                for (int i = 0; i < 4; ++i) hval[ot][nt][i] = 0.0f;
                if (!mine[ot][nt]) continue;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), accu = acc;
                const int sg = SUB == 4 ? ot : 0, su = SUB == 4 ? 2 + ot : 1;
                for (int w = 0; w < W; ++w) {
                    const float4 v = tred[((w * SUB + sg) * NT + nt) * 32 + lane];
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    if (SUB > 1) {
                        const float4 u = tred[((w * SUB + su) * NT + nt) * 32 + lane];
                        accu.x += u.x; accu.y += u.y; accu.z += u.z; accu.w += u.w;
                    }
                }
                float g4[4] = {acc.x, acc.y, acc.z, acc.w}, u4[4] = {accu.x, accu.y, accu.z, accu.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = out0 + ot * 16 + gid + 8 * (i >> 1);
                    const int tok = nt * 8 + 2 * t + (i & 1);
                    const bool live = row < re && tok < M_;
                    float v = g4[i], u = u4[i];
                    if (live && p.acc_in) {
                        v += p.partial[static_cast<int64_t>(tok) * p.n + row];
                        if (SUB > 1) u += p.partial[static_cast<int64_t>(tok) * p.n + p.n_out + row];
                    }
                    if (live && p.acc_out) {
                        p.partial[static_cast<int64_t>(tok) * p.n + row] = v;
                        if (SUB > 1) p.partial[static_cast<int64_t>(tok) * p.n + p.n_out + row] = u;
                    } else if (live) {
                        if (SUB > 1) v = (v / (1.0f + expf(-v))) * u;
                        if (SUB == 4) {
                            hval[ot][nt][i] = __half2float(__float2half_rn(v));
                        } else if (SUB == 1 && p.ar_world > 1) {
                            // the partial sum goes straight into every rank's inbox (peer stores over NVLink), its own too,
                            // as ONE 8-byte store of (value, call number): the receiver polls the slot itself, so neither
                            // side needs a fence or a flag
                            const int64_t o = ar_inbox_ofs + 2 * ((static_cast<int64_t>(p.ar_rank) * M_ + tok) * p.n + row);
                            for (int r = 0; r < p.ar_world; ++r)
                                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.ar_inbox[r] + o), "r"(__float_as_uint(v)),
                                             "r"(ar_epoch) : "memory");
                        } else {
                            const int64_t o = static_cast<int64_t>(tok) * p.ldy + row;
                            if (p.y_f16) static_cast<__half*>(Y_)[o] = __float2half_rn(v);
                            else static_cast<float*>(Y_)[o] = v;
                        }
                    }
                }
            }
        if (SUB == 4 && !p.acc_out) {
            // fused FWHT-32 over the job's 32 output rows: h (already rounded to f16) -> smem -> one warp per token
            if (W > 1) named_bar_sync(1 + team, team_threads); else __syncwarp();
#pragma unroll
            for (int ot = 0; ot < kOutTiles; ++ot)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (!mine[ot][nt]) continue;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int lrow = ot * 16 + gid + 8 * (i >> 1), tok = nt * 8 + 2 * t + (i & 1);
                        if (tok < M_) hbuf[tok * 32 + lrow] = hval[ot][nt][i];
                    }
                }
            if (W > 1) named_bar_sync(1 + team, team_threads); else __syncwarp();
            for (int tok = wj; tok < M_; tok += W) {
                float v = hbuf[tok * 32 + lane];
#pragma unroll
                for (int h = 1; h < 32; h <<= 1) v = fwht_xor_stage(v, h, (lane & h) != 0);
                v = __fmul_rn(v, qwc_inv_sqrt32());
                const int64_t o = static_cast<int64_t>(tok) * p.ldy + out0 + lane;
                if (p.y_f16) static_cast<__half*>(Y_)[o] = __float2half_rn(v);
                else static_cast<float*>(Y_)[o] = __half2float(__float2half_rn(v));
            }
        }
        if (W > 1) named_bar_sync(1 + team, team_threads); else __syncwarp();  // red is reused by the next job
    }

    if (SUB == 1 && p.ar_world > 1) {
        // ---- fused one-shot all-reduce: CTA c of every rank owns the same output rows, so a thread only has to wait for
        // the slots of its own (token, row) from every rank: each slot is an 8-byte (value, call number) pair stored whole
        // by its producer, so a slot that carries this call's number holds this call's value -- no fences, no flags (a
        // system-scope fence or release / acquire access costs microseconds here; this form costs one NVLink latency).
        // The world slots are summed in rank order (same bits on every rank).  The wait is bounded in time.
        {
            const int rows_cta = re - rb;
            const float* inbox = p.ar_inbox[p.ar_rank] + ar_inbox_ofs;
            const uint64_t limit = p.ar_wait_ns != 0 ? p.ar_wait_ns : static_cast<uint64_t>(QWC_WAIT_LIMIT_NS);
            uint64_t t0 = 0;
            bool gave_up = false;
            for (int i = threadIdx.x; i < rows_cta * M_; i += kConsumerWarps * 32) {
                const int tok = i / rows_cta, row = rb + (i - tok * rows_cta);
                float sum = 0.0f;
                for (int r = 0; r < p.ar_world; ++r) {
                    const float* slot = inbox + 2 * ((static_cast<int64_t>(r) * M_ + tok) * p.n + row);
                    uint32_t val = 0, tag = 0;
                    for (uint32_t spin = 0; !gave_up; ++spin) {
                        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(val), "=r"(tag) : "l"(slot) : "memory");
                        if (tag == ar_epoch) break;
                        // a peer that never stores (it failed, or it never made the call) costs this rank the limit once;
                        // then the status word says so and the kernel finishes with whatever the inbox holds
                        if ((spin & 31u) == 31u) {
                            const uint64_t now = qwc_globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > limit) gave_up = true;
                        }
                        if (spin > 16) __nanosleep(spin < 256 ? 40 : 250);
                    }
                    sum += __uint_as_float(val);
                }
                const int64_t o = static_cast<int64_t>(tok) * p.ldy + row;
                if (p.y_f16) static_cast<__half*>(Y_)[o] = __float2half_rn(sum);
                else static_cast<float*>(Y_)[o] = sum;
            }
            if (gave_up) atomicCAS(p.status, 0, QWC_DEV_WAIT_PEER_TIMEOUT);
        }
        const int grid = static_cast<int>(gridDim.x);
        if (p.ar_state != nullptr) {
            // the last CTA to finish publishes the call number: every CTA read the old one before it got here
            named_bar_sync(11, kConsumerWarps * 32);
            if (threadIdx.x == 0) {
                __threadfence();
                if (atomicAdd(p.ar_state + 1, 1u) == static_cast<uint32_t>(grid) - 1u) {
                    p.ar_state[1] = 0u;
                    __threadfence();
                    *reinterpret_cast<volatile uint32_t*>(p.ar_state) = ar_epoch;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Companion of the stream kernel in static-weights mode: brings the head of every CTA's row range of the NEXT call's
// bank into L2 while the previous kernel of the stream is still running.  The stream kernel keeps one CTA of ~220 KB
// of shared memory per SM, so the next call's CTAs cannot become resident (and start their own copies) before the
// previous call's CTAs have left; between the two, HBM would idle for the launch gap, the barrier set-up and one DRAM
// latency.  This kernel needs no shared memory and one warp per SM, so it runs beside the previous call's CTAs: it
// issues bulk L2 prefetches and then waits for the previous grid (so that the stream kernel launched after it, which
// waits for THIS grid, still runs after everything before it).  Weights are load-time data under the static-weights
// promise, so reading them early is safe.  CTA b covers the rows CTA b of the stream kernel will read.
__global__ void __launch_bounds__(32) qwc_gemv_prefetch_kernel(const uint8_t* __restrict__ blocks, int64_t row_bytes,
                                                               int row_quantum, int q_lo, int q_rem, int sub_stride_rows,
                                                               int subs, int64_t cap_bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int bq = static_cast<int>(blockIdx.x);
    const int64_t rb = static_cast<int64_t>(q_lo * bq + min(bq, q_rem)) * row_quantum;
    const int64_t re = rb + static_cast<int64_t>(q_lo + (bq < q_rem ? 1 : 0)) * row_quantum;
    constexpr int kPiece = 4096;
    for (int s = 0; s < subs; ++s) {   // a paired gate||up bank has two row ranges per CTA
        const uint8_t* base = blocks + (rb + static_cast<int64_t>(s) * sub_stride_rows) * row_bytes;
        int64_t bytes = (re - rb) * row_bytes;
        if (bytes > cap_bytes / subs) bytes = cap_bytes / subs;
        bytes &= ~static_cast<int64_t>(15);
        for (int64_t o = static_cast<int64_t>(threadIdx.x) * kPiece; o < bytes; o += 32 * kPiece) {
            const uint32_t sz = static_cast<uint32_t>(bytes - o < kPiece ? bytes - o : kPiece);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + o), "r"(sz) : "memory");
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
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

// ---------------------------------------------------------------------------------------------------------------
// Host side: geometry of one launch (chunking, team shape, ring depth) and K slicing when the activations of all
// tokens do not fit in shared memory next to the ring.

struct StreamGeom {
    int chunk_units, nchunks, team_warps, stages, stride, x_bytes, red_bytes, smem_bytes;
};

constexpr int kXCapBytes = (QWC_GEMV_SMEM_KB / 2 - 1) * 1024;  // at most this much shared memory for the staged activations of a K slice

// units: 32-element units of this launch's K slice; jobs: 16-row (32 for FWHT) jobs per CTA.  The team count T
// follows the jobs a CTA has (teams work on different jobs concurrently); K is cut into the fewest equal chunks that
// leave the ring T + 2 stages deep (measured: wide chunks beat a deep ring, equal chunks beat a short last one).
// Chunks are multiples of 8 units: with the 16-byte row pad the smem row stride in words is then 4 mod 8, which
// makes the per-lane word reads of 8 rows x 4 units hit 32 distinct banks (a multiple of 4 only gives 8-way
// conflicts).  Returns false when no geometry fits.
template <int FMT>
bool plan_geometry(int units, int m, int nt, int sub, int jobs, int budget, StreamGeom* g) {
    using C = StreamCfg<FMT>;
    // units per chunk must be a multiple of this (HQ4_G64: 36-byte blocks of two units; 16 units keep the row stride in
    // words at 4 mod 8 there, 8 units would give 0 mod 8 every other size)
    const int quantum = FMT == FMT_HQ4_G64 ? 16 : 8;
    // chunk bytes + 16 pad <= 2048: the box of the 2-D tensor copy is at most 256 8-byte elements wide
    const int max_chunk = FMT == FMT_HQ4_G32_M5 ? 96 : (FMT == FMT_HQ8_G32 ? 56 : 112);
    g->x_bytes = ((m * units * 64 + 127) / 128) * 128;
    g->red_bytes = kConsumerWarps * sub * nt * 32 * 16;
    const int fixed = g->x_bytes + g->red_bytes + kBarrierBytes;
    int teams = 1;
    // at most 8 teams: 16 single-warp teams need 18 stages, which forces 32-unit chunks, and narrow chunks cost far more
    // than wide teams (N = 248320: 198 us with 16 x 1 warps and 32-unit chunks, 139 us with 8 x 2 warps and 56-unit chunks)
    while (teams < jobs && teams < 8 && teams < kConsumerWarps) teams <<= 1;
    // short rows (K <= 1024): a job is a handful of groups, so a warp takes a whole job alone and there is no team reduction
    if (units <= 32 && jobs >= 16) teams = kConsumerWarps;
    const int env_w = tune_env("QWC_GEMV_W", 0), env_chunk = tune_env("QWC_GEMV_CHUNK", 0);
    if ((env_w == 1 || env_w == 2 || env_w == 4 || env_w == 8 || env_w == 16) && env_w <= kConsumerWarps) teams = kConsumerWarps / env_w;
    for (; teams >= 1; teams >>= 1) {
        const int w = kConsumerWarps / teams;
        const int want = teams + 2;
        int best_per = 0, best_stages = 0;
        for (int nch = 1; nch <= (units + quantum - 1) / quantum; ++nch) {
            int per = (units + nch - 1) / nch;
            per = ((per + quantum - 1) / quantum) * quantum;
            if (env_chunk > 0) per = ((env_chunk + quantum - 1) / quantum) * quantum;
            if (per > max_chunk) continue;
            const int stage_bytes = kTileRows * (per * C::kUnitBytes + kRowPad);
            int stages = (budget - fixed) / stage_bytes;
            if (stages > kMaxStages) stages = kMaxStages;
            if (stages >= want || (env_chunk > 0 && stages >= teams + 1)) { best_per = per; best_stages = stages; break; }
            if (env_chunk > 0) break;
        }
        if (best_per == 0) continue;
        if (best_per / C::kGroupUnits < w && teams > 1 && env_w == 0) continue;  // fewer groups than warps: idle warps
        // narrow chunks cost more than wide teams: if half as many teams allow a chunk of 48 units or more, take them
        if (best_per < 48 && teams >= 4 && env_w == 0 && env_chunk == 0 && units >= 48) {
            const int want2 = teams / 2 + 2;
            for (int nch = 1; nch <= (units + quantum - 1) / quantum; ++nch) {
                int per = (units + nch - 1) / nch;
                per = ((per + quantum - 1) / quantum) * quantum;
                if (per > max_chunk) continue;
                if (per < 48) break;
                const int stage_bytes = kTileRows * (per * C::kUnitBytes + kRowPad);
                int stages = (budget - fixed) / stage_bytes;
                if (stages > kMaxStages) stages = kMaxStages;
                if (stages >= want2) {
                    best_per = per;
                    best_stages = stages;
                    break;
                }
            }
            if (best_per >= 48) {
                g->chunk_units = best_per;
                g->nchunks = (units + best_per - 1) / best_per;
                g->stride = best_per * C::kUnitBytes + kRowPad;
                g->team_warps = kConsumerWarps / (teams / 2);
                g->stages = best_stages;
                g->smem_bytes = fixed + best_stages * kTileRows * g->stride;
                return true;
            }
        }
        g->chunk_units = best_per;
        g->nchunks = (units + best_per - 1) / best_per;
        g->stride = best_per * C::kUnitBytes + kRowPad;
        g->team_warps = w;
        g->stages = best_stages;
        g->smem_bytes = fixed + best_stages * kTileRows * g->stride;
        return true;
    }
    return false;
}

template <int FMT, int NT, int SUB>
int launch_stream_inst(const qwc_hal* hal, cudaStream_t st, const GemvParams& p, const CUtensorMap& tmap, int smem_bytes,
                       int grid) {
    // once per device and instantiation; racing first calls both set the same value, which is harmless
    static std::atomic<bool> configured[64];
    if (!configured[hal->device & 63].load(std::memory_order_acquire)) {
        QWC_CUDA_TRY(cudaFuncSetAttribute(qwc_gemv_stream_kernel<FMT, NT, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemBudget));
        configured[hal->device & 63].store(true, std::memory_order_release);
    }
    if (p.pdl) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_gemv_stream_kernel<FMT, NT, SUB>, p, tmap));
        return QWC_OK;
    }
    qwc_gemv_stream_kernel<FMT, NT, SUB><<<grid, kThreads, smem_bytes, st>>>(p, tmap);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

constexpr int kMaxSlices = 64;

// dry != 0: plan only (every refusal this function can make), launch nothing.
template <int FMT, int NT>
int launch_stream(const qwc_hal* hal, cudaStream_t st, GemvParams p, int total_units, float* workspace, bool dry = false) {
    const int sub = p.epilogue == QWC_EPI_NONE ? 1 : (p.epilogue == QWC_EPI_SILU_PAIR ? 2 : 4);
    // K slices: as few as keep the staged activations within their share of shared memory.
    const int quantum = FMT == FMT_HQ4_G64 ? 8 : 4;
    const int x_cap_units = kXCapBytes / (p.m * 64);
    int slices = 1;
    if (total_units > x_cap_units) slices = (total_units + x_cap_units - 1) / x_cap_units;
    int per_slice = (total_units + slices - 1) / slices;
    per_slice = ((per_slice + quantum - 1) / quantum) * quantum;
    slices = (total_units + per_slice - 1) / per_slice;
    if (slices > 1 && workspace == nullptr)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "this call needs a workspace of qwc_gemm_workspace_bytes() bytes");
    const int quanta = p.n_out / p.row_quantum;
    int grid = hal->sm_count;
    if (grid > quanta) grid = quanta;
    if (grid < 1) grid = 1;
    if (p.segs != nullptr) {   // segment mode: one CTA per list entry, the list's capacity is the grid
        if (slices > 1) return qwc_fail(QWC_ERR_BLOCKED, "segment mode takes one K slice (tokens x K x 2 B <= 112 KB)");
        grid = p.seg_grid;
    }
    // The geometry of every K slice is planned before the first launch, so that a refusal leaves the stream untouched.
    if (slices > kMaxSlices) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "k needs %d slices, at most %d are planned", slices, kMaxSlices);
    StreamGeom geoms[kMaxSlices];
    {
        const int rows_per_cta = p.segs != nullptr ? p.seg_cols : (p.n_out + grid - 1) / grid;
        const int job_rows = sub == 4 ? 32 : 16;
        const int jobs = (rows_per_cta + job_rows - 1) / job_rows;
        for (int s = 0; s < slices; ++s) {
            const int u0 = s * per_slice;
            const int units = total_units - u0 < per_slice ? total_units - u0 : per_slice;
            if (!plan_geometry<FMT>(units, p.m, NT, sub, jobs, kSmemBudget, &geoms[s]))
                return qwc_fail(QWC_ERR_BAD_GEOMETRY, "no shared-memory geometry fits this k slice");
        }
    }
    if (dry) return QWC_OK;
    // Static-weights mode: a shared-memory-free companion kernel brings the head of every CTA's row range into L2 while
    // the previous kernel of the stream still holds the SMs' shared memory (see qwc_gemv_prefetch_kernel).  A bank that
    // fits in L2 beside the one being streamed (<= 48 MB of the 126 MB) is prefetched whole; of a larger one only the
    // first 128 KB per CTA (19 MB: what the gap between two calls can absorb), and the stream kernel then marks its
    // own reads evict-first so that they do not push the prefetched lines out (measured, N x K = 12288 x 4096 /
    // 17408 x 5120 HQ4_G32 / 17408 x 5120 HQ8_G32: 9.8 -> 8.6, 14.2 -> 14.0, 19.6 -> 18.7 us per call; prefetching
    // the larger banks whole, or without the evict-first mark, lost up to 18 %).
    const bool small_bank = static_cast<int64_t>(p.n) * p.row_bytes <= (48ll << 20);
    const int64_t pf_cap = static_cast<int64_t>(tune_env("QWC_GEMV_PF_KB", small_bank ? 512 : 128)) * 1024;
    if (p.pdl && p.segs == nullptr && pf_cap > 0 && p.row_bytes % 16 == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(32);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        QWC_CUDA_TRY(cudaLaunchKernelEx(&cfg, qwc_gemv_prefetch_kernel, p.blocks, p.row_bytes, p.row_quantum, quanta / grid,
                                        quanta % grid, p.n_out, sub == 1 ? 1 : 2, pf_cap));
    }
    for (int s = 0; s < slices; ++s) {
        GemvParams q = p;
        q.q_lo = quanta / grid;
        q.q_rem = quanta % grid;
        q.l2_evict_first = p.pdl && tune_env("QWC_GEMV_EVICT_FIRST", small_bank ? 0 : 1) != 0;
        q.unit0 = s * per_slice;
        q.units = total_units - q.unit0 < per_slice ? total_units - q.unit0 : per_slice;
        q.partial = workspace;
        q.acc_in = s > 0;
        q.acc_out = s + 1 < slices;
        const StreamGeom& g = geoms[s];
        if (tune_env("QWC_GEMV_TRACE", 0))   // tuning aid: print the chosen geometry
            fprintf(stderr, "qwc_gemv: fmt %d m %d units %d -> chunk %d x %d, teams %d x %d warps, %d stages, stride %d, smem %d\n",
                    FMT, q.m, q.units, g.chunk_units, g.nchunks, kConsumerWarps / g.team_warps, g.team_warps, g.stages,
                    g.stride, g.smem_bytes);
        q.chunk_units = g.chunk_units;
        q.nchunks = g.nchunks;
        q.team_warps = g.team_warps;
        q.stages = g.stages;
        q.stride = g.stride;
        q.x_bytes = g.x_bytes;
        q.red_bytes = g.red_bytes;
        // Tensor map over the bank as [n rows][row_bytes / 8] 8-byte elements; box = 16 rows x stride bytes.
        alignas(64) CUtensorMap tmap;
        memset(&tmap, 0, sizeof(tmap));
        q.use_tmap = 0;
        if (hal->encode_tiled != nullptr && g.stride / 8 <= 256) {
            using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                          const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
            const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(p.row_bytes / 8), static_cast<cuuint64_t>(p.n)};
            const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(p.row_bytes)};
            const cuuint32_t box[2] = {static_cast<cuuint32_t>(g.stride / 8), static_cast<cuuint32_t>(kTileRows)};
            const cuuint32_t estr[2] = {1, 1};
            const CUresult cr = reinterpret_cast<EncodeFn>(hal->encode_tiled)(
                &tmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(p.blocks), gdim, gstride, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            q.use_tmap = cr == CUDA_SUCCESS;
        }
        int rc;
        if (sub == 1) rc = launch_stream_inst<FMT, NT, 1>(hal, st, q, tmap, g.smem_bytes, grid);
        else if (sub == 2) rc = launch_stream_inst<FMT, NT, 2>(hal, st, q, tmap, g.smem_bytes, grid);
        else rc = launch_stream_inst<FMT, NT, 4>(hal, st, q, tmap, g.smem_bytes, grid);
        if (rc) return rc;
    }
    return QWC_OK;
}

template <int FMT>
int launch_fmt(const qwc_hal* hal, cudaStream_t st, GemvParams p, int64_t m, bool stream_ok, int total_units,
               float* workspace, bool dry) {
    const char* xb = reinterpret_cast<const char*>(p.x);
    char* yb = static_cast<char*>(p.y);
    const int64_t ysz = p.y_f16 ? 2 : 4;
    if (!stream_ok) {
        if (p.epilogue == QWC_EPI_SILU_PAIR_FWHT)
            return qwc_fail(QWC_ERR_BAD_GEOMETRY, "fused FWHT epilogue needs 16-byte aligned rows (K %% 128 == 0)");
        if (dry) return QWC_OK;
        p.m = static_cast<int>(m);
        p.units = total_units;
        const int64_t items = static_cast<int64_t>(p.n_out) * m;
        int64_t grid = (items + 7) / 8;
        if (grid > hal->sm_count * 8) grid = hal->sm_count * 8;
        if (grid < 1) grid = 1;
        qwc_gemv_rowwise_kernel<FMT><<<static_cast<unsigned>(grid), 256, 0, st>>>(p, static_cast<int>(m));
        QWC_CUDA_TRY(cudaGetLastError());
        return QWC_OK;
    }
    // M > 16 is served in slabs of 16 tokens (each slab re-reads the weights); the tensor-core GEMM takes over there.
    // With several slabs a planning pass comes first, so that no slab can refuse after an earlier one ran (a single slab
    // plans all its K slices before its first launch anyway).
    for (int pass = (dry || m <= 16) ? 1 : 0; pass < 2; ++pass)
    for (int64_t m0 = 0; m0 < m; m0 += 16) {
        const bool plan_only = pass == 0 || dry;
        if (pass == 0 && m0 != 0 && m0 + 16 < m) continue;   // full slabs plan alike: the first and the last are enough
        GemvParams q = p;
        q.m = static_cast<int>(m - m0 < 16 ? m - m0 : 16);
        q.x = reinterpret_cast<const __half*>(xb + m0 * p.ldx * 2);
        q.y = yb + m0 * p.ldy * ysz;
        const int rc = q.m <= 8 ? launch_stream<FMT, 1>(hal, st, q, total_units, workspace, plan_only)
                                : launch_stream<FMT, 2>(hal, st, q, total_units, workspace, plan_only);
        if (rc) return rc;
    }
    return QWC_OK;
}

}  // namespace

// Bytes of f32 scratch a call needs: non-zero only when the staged activations of up to 16 tokens exceed their
// shared-memory share, so that K is processed in slices whose raw sums are carried in the workspace.
size_t qwc_gemv_workspace_bytes(const qwc_weight_view* w, int64_t m) {
    const int64_t mm = m < 16 ? m : 16;
    if (mm <= 0) return 0;
    const int64_t row_bytes = (w->k / w->group) * qwc_block_bytes(w->kind, w->bits, w->group);
    if (row_bytes % 16 != 0) return 0;  // row-wise kernel: no scratch
    const int64_t x_cap_units = kXCapBytes / (mm * 64);
    return (w->k / 32) > x_cap_units ? static_cast<size_t>(mm) * static_cast<size_t>(w->n) * 4 : 0;
}

// Host entry used by qwc_gemm.  All arguments were validated by the caller.
int qwc_launch_gemv_ar(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx,
                       void* y, int y_dtype, int64_t ldy, int epilogue, int x_is_rotated, void* workspace,
                       size_t workspace_bytes, const qwc_allreduce_ctx* ar, bool dry = false);

// Every refusal the streaming path can make for these arguments, without a launch.
int qwc_gemv_check(const qwc_hal* hal, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx, void* y, int y_dtype,
                   int64_t ldy, int epilogue, int x_is_rotated, void* workspace, size_t workspace_bytes) {
    return qwc_launch_gemv_ar(hal, nullptr, w, x, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, workspace, workspace_bytes, nullptr, true);
}

int qwc_launch_gemv(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx,
                    void* y, int y_dtype, int64_t ldy, int epilogue, int x_is_rotated, void* workspace,
                    size_t workspace_bytes) {
    return qwc_launch_gemv_ar(hal, st, w, x, m, ldx, y, y_dtype, ldy, epilogue, x_is_rotated, workspace, workspace_bytes, nullptr);
}

// ar != null: the fused all-reduce form (validated by the caller: one K slice, <= 8 tokens, no epilogue, 16-byte rows).
int qwc_launch_gemv_ar(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* w, const void* x, int64_t m, int64_t ldx,
                       void* y, int y_dtype, int64_t ldy, int epilogue, int x_is_rotated, void* workspace,
                       size_t workspace_bytes, const qwc_allreduce_ctx* ar, bool dry) {
    GemvParams p{};
    if (ar != nullptr) {
        p.ar_world = ar->world;
        p.ar_rank = ar->rank;
        p.ar_epoch = ar->epoch;
        p.ar_wait_ns = ar->reserved > 0 ? static_cast<uint64_t>(ar->reserved) * 1000ull : 0ull;
        p.ar_state = static_cast<uint32_t*>(ar->epoch_state);
        p.ar_inbox_stride = ar->inbox_floats;
        for (int r = 0; r < ar->world && r < 8; ++r) {
            p.ar_inbox[r] = static_cast<float*>(ar->inbox[r]);
        }
    }
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
    p.n = static_cast<int>(w->n);
    p.n_out = static_cast<int>(epilogue == QWC_EPI_NONE ? w->n : w->n / 2);
    p.y_f16 = y_dtype == QWC_F16;
    p.epilogue = epilogue;
    p.x_is_rotated = x_is_rotated;
    p.row_quantum = epilogue == QWC_EPI_SILU_PAIR_FWHT ? 32 : 1;
    if (const int rq = tune_env("QWC_GEMV_RQ", 0); rq > 0 && p.n_out % rq == 0 && rq % p.row_quantum == 0) p.row_quantum = rq;
    p.pdl = hal->static_weights;
    const int total_units = static_cast<int>(w->k / 32);
    const bool stream_ok = (p.row_bytes % 16 == 0) && (reinterpret_cast<uintptr_t>(w->blocks) % 16 == 0);
    const size_t need = stream_ok ? qwc_gemv_workspace_bytes(w, m) : 0;
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
        return qwc_fail(QWC_ERR_BAD_SHAPE, "workspace of %zu bytes needed (qwc_gemm_workspace_bytes), got %zu", need, workspace_bytes);
    if (need > 0 && reinterpret_cast<uintptr_t>(workspace) % 4 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "workspace must be 4-byte aligned");
    float* ws = need > 0 ? static_cast<float*>(workspace) : nullptr;
    switch (fmt) {
        case FMT_HQ4_G32_M5: return launch_fmt<FMT_HQ4_G32_M5>(hal, st, p, m, stream_ok, total_units, ws, dry);
        case FMT_HQ8_G32: return launch_fmt<FMT_HQ8_G32>(hal, st, p, m, stream_ok, total_units, ws, dry);
        case FMT_HQ4_G64: return launch_fmt<FMT_HQ4_G64>(hal, st, p, m, stream_ok, total_units, ws, dry);
        default: return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unsupported container");
    }
}

// Segment mode of the stream kernel (decode-time mixture of experts): `bank` is the stacked expert bank, xs the
// expert-sorted (rotated) activation rows, y the expert-sorted outputs [pairs, n_out]; entry i of the device-side list
// `segs` (at most max_segs entries, *seg_count valid) names one expert's column range and its <= 8 rows.
int qwc_launch_gemv_segments(const qwc_hal* hal, cudaStream_t st, const qwc_weight_view* bank, const void* xs, int64_t ldx,
                             void* y, int y_dtype, int64_t ldy, int epilogue, int64_t n_out, int seg_cols, const void* segs,
                             const int32_t* seg_count, int64_t max_segs) {
    GemvParams p{};
    const int fmt = qwc_fmt_of(*bank);
    const int64_t bb = qwc_block_bytes(bank->kind, bank->bits, bank->group);
    const int group = fmt == FMT_HQ4_G64 ? 64 : 32;
    p.blocks = static_cast<const uint8_t*>(bank->blocks);
    p.row_bytes = (bank->k / group) * bb;
    p.x = static_cast<const __half*>(xs);
    p.ldx = ldx;
    p.y = y;
    p.ldy = ldy;
    p.status = hal->status;
    p.n = static_cast<int>(bank->n);
    p.n_out = static_cast<int>(n_out);
    p.m = 8;   // sizes the activation region; a CTA stages only its entry's rows
    p.y_f16 = y_dtype == QWC_F16;
    p.epilogue = epilogue;
    p.x_is_rotated = 1;
    p.row_quantum = epilogue == QWC_EPI_SILU_PAIR_FWHT ? 32 : 1;
    p.pdl = hal->static_weights;
    p.segs = static_cast<const qwc_gemv_seg*>(segs);
    p.seg_count = seg_count;
    p.seg_grid = static_cast<int>(max_segs);
    p.seg_cols = seg_cols;
    if (p.row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(bank->blocks) % 16 != 0)
        return qwc_fail(QWC_ERR_BLOCKED, "segment mode needs 16-byte aligned bank rows");
    const int total_units = static_cast<int>(bank->k / 32);
    switch (fmt) {
        case FMT_HQ4_G32_M5: return launch_stream<FMT_HQ4_G32_M5, 1>(hal, st, p, total_units, nullptr);
        case FMT_HQ8_G32: return launch_stream<FMT_HQ8_G32, 1>(hal, st, p, total_units, nullptr);
        case FMT_HQ4_G64: return launch_stream<FMT_HQ4_G64, 1>(hal, st, p, total_units, nullptr);
        default: return qwc_fail(QWC_ERR_BAD_WEIGHTS, "unsupported container");
    }
}
