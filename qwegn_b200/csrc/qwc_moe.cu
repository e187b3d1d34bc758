// Mixture-of-experts operator chain: the CUDA twins of the reference's router, pair sort, SwiGLU and combine
// kernels and the host orchestration of QWMoEOperator.encodeResident
// (Sources/Operators/QWGEMM/QWMoEOperator.swift:206-442, grouped path, T > 8).
//   qwg_moe_route                      Sources/QWMetal/subsystems/qwrouter.metal:84-168
//   qwg_moe_group_pairs_f32            Sources/QWMetal/gemm/qwgemm_moe_group_f32.metal:10-148
//   qwg_silu_mul_split_f16             Sources/QWMetal/gemm/qwgemm_batched.metal:55-97
//   qwg_moe_down_reduce_combine_f32    Sources/QWMetal/gemm/qwgemm_moe_nax_f16.metal:7-126
// The grouped expert GEMMs run on the tensor-core kernel of qwc_gemm_tc.cu over the tile list built here.
#include <cstdlib>

#include "qwc_common.cuh"

int qwc_launch_gemm_tc_grouped(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, const qwc_moe_tile*,
                               const int32_t*, int64_t, void*, int, int64_t, int, int);
bool qwc_gemm_tc_supported(const qwc_hal*, const qwc_weight_view*, int64_t, int);
int qwc_launch_gemv_segments(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, void*, int, int64_t, int,
                             int64_t, int, const void*, const int32_t*, int64_t);

namespace {

constexpr int kTileW = 128;  // weight rows per grouped-GEMM tile
// Activation rows per grouped-GEMM tile.  Every tile decodes its 128 weight rows once whatever its token count, so an
// expert should fit in one tile; 192 rows is the tallest tile the tensor-memory budget allows.  The kernel fetches only
// a 64- or 128-row activation box when the tile is that small.
inline int moe_tile_rows(int64_t pairs, int64_t e) {
    const int env_rows = tune_env("QWC_MOE_TILE_ROWS", 0);
    if (env_rows == 64 || env_rows == 128 || env_rows == 192) return env_rows;
    // Up to ~85 rows per expert on average, hardly any expert exceeds 128 rows: tiles of 128 rows then let the kernel run
    // with eight operand stages (see qwc_gemm_tc.cu); above that, 192-row tiles keep an expert in one tile more often.
    return (e > 0 && pairs * 3 <= e * 256) ? 128 : 192;
}

__device__ __forceinline__ bool finite_bits(float v) { return (__float_as_uint(v) & 0x7F800000u) != 0x7F800000u; }

// One warp routes one token.  Lane l holds experts l, l + 32, ... (e <= 512 -> at most 16 per lane).
__global__ void __launch_bounds__(128) qwc_moe_route_kernel(const float* __restrict__ logits, int t_rows, int e, int k,
                                                            int norm_topk, float routed_scale, int32_t* __restrict__ idx,
                                                            float* __restrict__ wts) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= t_rows) return;
    constexpr int kMaxPer = 16;
    float pv[kMaxPer];
    bool valid[kMaxPer];
    const int per = (e + 31) / 32;
    float mx = -3.4e38f;
    bool any = false;
#pragma unroll
    for (int j = 0; j < kMaxPer; ++j) {
        const int id = lane + 32 * j;
        pv[j] = (j < per && id < e) ? logits[static_cast<int64_t>(t) * e + id] : 0.0f;
        valid[j] = j < per && id < e && finite_bits(pv[j]);
        if (valid[j]) {
            mx = any ? fmaxf(mx, pv[j]) : pv[j];
            any = true;
        }
    }
    const bool any_finite = __any_sync(0xFFFFFFFFu, any);
    float wmx = any ? mx : -3.4e38f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmx = fmaxf(wmx, __shfl_xor_sync(0xFFFFFFFFu, wmx, o));
    const float max_logit = any_finite ? wmx : 0.0f;
    // total = sum over experts in index order groups (lane-major partial sums, then a warp sum): f32, like the
    // reference's simd_sum per 32-wide slice accumulated over slices
    float total = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPer; ++j) {
        if (j >= per) break;   // warp-uniform: slices beyond the expert count hold nothing
        float ex = valid[j] ? expf(pv[j] - max_logit) : 0.0f;
        pv[j] = ex;
        float s = ex;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        total += s;
    }
#pragma unroll
    for (int j = 0; j < kMaxPer; ++j) {
        valid[j] = valid[j] && total > 0.0f;
        pv[j] = valid[j] ? pv[j] / total : -1e30f;
    }
    float sel_w = 0.0f;   // lane r keeps the weight of the r-th choice
    int sel_i = -1;
    float acc = 0.0f;
    for (int r = 0; r < k; ++r) {
        float bv = -3.4e38f;
        int bi = 0x7FFFFFFF;
#pragma unroll
        for (int j = 0; j < kMaxPer; ++j) {
            if (j >= per) break;
            const int id = lane + 32 * j;
            if (valid[j] && (pv[j] > bv || (pv[j] == bv && id < bi))) {
                bv = pv[j];
                bi = id;
            }
        }
        // warp argmax with ties to the lower id.  Valid weights are softmax outputs (finite, >= 0), so their bit patterns
        // order like the values: one integer max over the warp, then the lowest id among the lanes that hold it.
        const uint32_t key = bi != 0x7FFFFFFF ? __float_as_uint(bv) + 1u : 0u;   // 0: this lane has no candidate
        const uint32_t kmax = __reduce_max_sync(0xFFFFFFFFu, key);
        const uint32_t cand = (kmax != 0u && key == kmax) ? static_cast<uint32_t>(bi) : 0x7FFFFFFFu;
        bi = static_cast<int>(__reduce_min_sync(0xFFFFFFFFu, cand));
        bv = kmax != 0u ? __uint_as_float(kmax - 1u) : -3.4e38f;
        const bool found = bi != 0x7FFFFFFF;
        if (found && (bi & 31) == lane) {
#pragma unroll
            for (int j = 0; j < kMaxPer; ++j)
                if (j == (bi >> 5)) valid[j] = false;
        }
        if (lane == r) {
            sel_w = found ? bv : 0.0f;
            sel_i = found ? bi : -1;
        }
        acc += found ? bv : 0.0f;   // same order on every lane: sum of the chosen weights in rank order
    }
    if (lane < k) {
        const float rs = routed_scale > 0.0f ? routed_scale : 1.0f;
        const float nw = norm_topk ? (acc > 0.0f ? sel_w / acc : 0.0f) : sel_w;
        idx[static_cast<int64_t>(t) * k + lane] = sel_i;
        wts[static_cast<int64_t>(t) * k + lane] = nw * rs;
    }
}

// Router logits: y[t, e] = x[t, :] . W[e, :], f32 accumulate (the reference's qwg_router_gemm,
// Sources/QWMetal/subsystems/qwrouter.metal:460-520; host door QWGemmMoERouter.swift:78-125).  The router weight is a
// raw, un-rotated plane (bf16, f16 or f32), the activations are the plain (un-rotated) hidden states (f16 or f32).
// A CTA computes 64 tokens x 64 experts; K goes through shared memory 32 columns at a time; a thread owns a 4 x 4
// block (tokens 4 ty .. 4 ty + 3, experts tx, tx + 16, tx + 32, tx + 48).
__device__ __forceinline__ float router_cvt(float v) { return v; }
__device__ __forceinline__ float router_cvt(__half v) { return __half2float(v); }
__device__ __forceinline__ float router_cvt(unsigned short v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }   // bf16 bits

template <typename XT, typename WT>
__global__ void __launch_bounds__(256) qwc_moe_router_gemm_kernel(const XT* __restrict__ x, int64_t ldx, const WT* __restrict__ w,
                                                                  int t_rows, int e, int h, float* __restrict__ y) {
    pdl_enter();
    __shared__ float xs[64][33];
    __shared__ float ws[64][33];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int t0 = blockIdx.y * 64, e0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < h; k0 += 32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = (tid >> 5) + 8 * i, c = tid & 31;
            xs[r][c] = t0 + r < t_rows ? router_cvt(x[static_cast<int64_t>(t0 + r) * ldx + k0 + c]) : 0.0f;
            ws[r][c] = e0 + r < e ? router_cvt(w[static_cast<int64_t>(e0 + r) * h + k0 + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xv[i] = xs[4 * ty + i][kk];
                wv[i] = ws[tx + 16 * i][kk];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = t0 + 4 * ty + i, ex = e0 + tx + 16 * j;
            if (t < t_rows && ex < e) y[static_cast<int64_t>(t) * e + ex] = acc[i][j];
        }
}

// Tile j of expert ex for a bank with `rows` rows per expert.  paired != 0 (gate||up bank feeding a SwiGLU epilogue):
// the tile is 64 gate rows followed by the 64 up rows that pair with them, and its output columns are the 64 rows of h.
__device__ __forceinline__ qwc_moe_tile moe_make_tile(int ex, int rows, int j, int paired, int x_row0, int x_rows) {
    qwc_moe_tile tl;
    if (paired) {
        tl.w_row0 = ex * rows + j * (kTileW / 2);
        tl.pad0 = tl.w_row0 + rows / 2;
        tl.w_rows = kTileW;
        tl.y_col0 = j * (kTileW / 2);
        tl.pad1 = 1;
    } else {
        tl.w_row0 = ex * rows + j * kTileW;
        tl.pad0 = 0;
        tl.w_rows = min(kTileW, rows - j * kTileW);
        tl.y_col0 = j * kTileW;
        tl.pad1 = 0;
    }
    tl.x_row0 = x_row0;
    tl.x_rows = x_rows;
    tl.expert = ex;
    return tl;
}

// Pass 1 of the pair sort: one warp per expert counts its pairs; warp `e` (one past the last expert) marks the
// dropped pairs (idx < 0 or >= e) in inv_perm.  The CTA stages the pair list through shared memory in chunks so the
// per-warp scans run at shared-memory latency instead of one L2 round trip per 32 pairs.
constexpr int kSortChunk = 8192;

__global__ void __launch_bounds__(512) qwc_moe_count_kernel(const int32_t* __restrict__ idx, int pairs, int e,
                                                            int32_t* __restrict__ counts, int32_t* __restrict__ inv_perm) {
    pdl_enter();
    __shared__ int s_idx[kSortChunk];
    const int lane = threadIdx.x & 31;
    const int ex = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int c = 0;
    for (int base = 0; base < pairs; base += kSortChunk) {
        const int n = min(kSortChunk, pairs - base);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_idx[i] = idx[base + i];
        __syncthreads();
        if (ex > e) continue;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const int v = i < n ? s_idx[i] : 0;
            if (ex == e) {
                if (i < n && (v < 0 || v >= e)) inv_perm[base + i] = -1;
            } else {
                c += __popc(__ballot_sync(0xFFFFFFFFu, i < n && v == ex));
            }
        }
    }
    if (ex < e && lane == 0) counts[ex] = c;
}

// Pass 2: exclusive prefix over the experts and the two tile lists (one CTA).
__global__ void __launch_bounds__(512) qwc_moe_plan_kernel(const int32_t* counts, int e, int kTileX, int32_t* expert_off,
                                                           int gu_rows, int dn_rows, int gu_paired, qwc_moe_tile* __restrict__ tiles_gu,
                                                           qwc_moe_tile* __restrict__ tiles_dn, int32_t* __restrict__ tile_counts) {
    __shared__ int s_off[513];
    __shared__ int s_tx[513];   // activation-tile prefix
    pdl_enter();
    if (threadIdx.x == 0) {
        int run = 0, tx = 0;
        for (int i = 0; i < e; ++i) {
            s_off[i] = run;
            s_tx[i] = tx;
            run += counts[i];
            tx += (counts[i] + kTileX - 1) / kTileX;
        }
        s_off[e] = run;
        s_tx[e] = tx;
        tile_counts[0] = tx * ((gu_rows + kTileW - 1) / kTileW);
        tile_counts[1] = tx * ((dn_rows + kTileW - 1) / kTileW);
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= e; i += blockDim.x) expert_off[i] = s_off[i];
    for (int ex = threadIdx.x; ex < e; ex += blockDim.x) {
        const int cnt = s_off[ex + 1] - s_off[ex];
        const int ntx = s_tx[ex + 1] - s_tx[ex];
        for (int which = 0; which < 2; ++which) {
            const int rows = which == 0 ? gu_rows : dn_rows;
            qwc_moe_tile* tiles = which == 0 ? tiles_gu : tiles_dn;
            if (tiles == nullptr) continue;
            const int ntw = (rows + kTileW - 1) / kTileW;
            // weight tiles fastest inside an activation tile: consecutive tiles re-read the same activations
            for (int mt = 0; mt < ntx; ++mt)
                for (int j = 0; j < ntw; ++j)
                    tiles[(s_tx[ex] + mt) * ntw + j] = moe_make_tile(ex, rows, j, which == 0 && gu_paired, s_off[ex] + mt * kTileX,
                                                                     min(kTileX, cnt - mt * kTileX));
        }
    }
}

// Pass 3: one warp per expert places its pairs in ascending pair order (same staging as pass 1).
__global__ void __launch_bounds__(512) qwc_moe_place_kernel(const int32_t* __restrict__ idx, int pairs, int e, int k,
                                                            const int32_t* __restrict__ expert_off, int32_t* __restrict__ sorted_pair,
                                                            int32_t* __restrict__ sorted_tok, int32_t* __restrict__ inv_perm) {
    pdl_enter();
    __shared__ int s_idx[kSortChunk];
    const int lane = threadIdx.x & 31;
    const int ex = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int at = ex < e ? expert_off[ex] : 0;
    for (int base = 0; base < pairs; base += kSortChunk) {
        const int n = min(kSortChunk, pairs - base);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_idx[i] = idx[base + i];
        __syncthreads();
        if (ex >= e) continue;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < n && s_idx[i] == ex;
            const unsigned m = __ballot_sync(0xFFFFFFFFu, hit);
            if (hit) {
                const int pos = at + __popc(m & ((1u << lane) - 1u));
                sorted_pair[pos] = base + i;
                sorted_tok[pos] = (base + i) / k;
                inv_perm[base + i] = pos;
            }
            at += __popc(m);
        }
    }
}

// xs[p, :] = rot(x[sorted_tok[p], :]).  A quad handles one (sorted row, 32-element unit): lane t holds elements
// 8t..8t+7 (one 16-byte load), rotates with three in-lane butterfly stages and two xor-shuffle stages (the
// reference's h = 1, 2, 4, 8, 16 order) and writes one 16-byte chunk.  vec != 0 needs 16-byte aligned rows.
// IdxT = uint32_t while pairs * units fits (the item index is divided per item: 32-bit division is several times cheaper).
// sorted_tok == nullptr: rows in place (row p of the output is row p of x): the rotate-once pre-pass of the row-copy gather.
// Block `block` of `nblocks` blocks of 256 threads.
template <typename IdxT>
__device__ __forceinline__ void moe_gather_items(const __half* __restrict__ x, int64_t ldx, int h, const int32_t* __restrict__ sorted_tok,
                                                 IdxT rows, int rotate, int vec, __half* __restrict__ xs, int block, int nblocks) {
    const int lane = threadIdx.x & 31, t4 = lane & 3, q8 = lane >> 2;
    const int units = h / 32;
    const IdxT total = rows * static_cast<IdxT>(units);
    const IdxT step = static_cast<IdxT>(nblocks) * (blockDim.x >> 5) * 8;
    for (IdxT base = (static_cast<IdxT>(block) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 8; base < total; base += step) {
        const IdxT it = base + q8;
        const bool live = it < total;
        const IdxT prq = live ? it / static_cast<IdxT>(units) : 0;
        const int u = live ? static_cast<int>(it - prq * static_cast<IdxT>(units)) : 0;
        const int64_t pr = static_cast<int64_t>(prq);
        const __half* src = x + static_cast<int64_t>(live ? (sorted_tok != nullptr ? sorted_tok[pr] : static_cast<int32_t>(pr)) : 0) * ldx + u * 32 + 8 * t4;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (live) {
            if (vec) raw = *reinterpret_cast<const uint4*>(src);
            else {
                __half tmp[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) tmp[i] = src[i];
                raw = *reinterpret_cast<const uint4*>(tmp);
            }
        }
        if (rotate) {
            __half2 hv[4] = {*reinterpret_cast<__half2*>(&raw.x), *reinterpret_cast<__half2*>(&raw.y),
                             *reinterpret_cast<__half2*>(&raw.z), *reinterpret_cast<__half2*>(&raw.w)};
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(hv[i]); f[2 * i + 1] = __high2float(hv[i]); }
#pragma unroll
            for (int s = 1; s < 8; s <<= 1)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if ((i & s) == 0) {
                        const float a = f[i], b = f[i + s];
                        f[i] = __fadd_rn(a, b);
                        f[i + s] = __fsub_rn(a, b);
                    }
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 1, (t4 & 1) != 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = fwht_xor_stage(f[i], 2, (t4 & 2) != 0);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                hv[i] = __floats2half2_rn(__fmul_rn(f[2 * i], qwc_inv_sqrt32()), __fmul_rn(f[2 * i + 1], qwc_inv_sqrt32()));
            raw = make_uint4(*reinterpret_cast<uint32_t*>(&hv[0]), *reinterpret_cast<uint32_t*>(&hv[1]),
                             *reinterpret_cast<uint32_t*>(&hv[2]), *reinterpret_cast<uint32_t*>(&hv[3]));
        }
        if (live) *reinterpret_cast<uint4*>(xs + pr * h + u * 32 + 8 * t4) = raw;
    }
}

template <typename IdxT>
__global__ void __launch_bounds__(256) qwc_moe_gather_kernel(const __half* __restrict__ x, int64_t ldx, int h,
                                                             const int32_t* __restrict__ sorted_tok,
                                                             const int32_t* __restrict__ expert_off, int e, int rotate, int vec,
                                                             __half* __restrict__ xs) {
    pdl_enter();
    moe_gather_items<IdxT>(x, ldx, h, sorted_tok, static_cast<IdxT>(sorted_tok != nullptr ? expert_off[e] : e), rotate, vec, xs,
                           static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

// The whole pair sort in one launch, for pair counts where reading the pair list once per CTA is cheap (the list is
// 64 KB at 2048 tokens x top-8 and sits in L2).  CTA c owns pairs [256 c, 256 c + 256).  Every CTA histograms ALL
// pairs in shared memory (one shared atomic per pair), snapshotting the histogram when it reaches its own range: that
// snapshot is the number of earlier pairs per expert.  An exclusive scan of the totals gives expert_off; the rank of a
// pair inside its CTA comes from __match_any_sync (rank inside the warp) plus a per-warp, per-expert table (rank of the
// warp inside the CTA).  The result is the stable counting sort of the reference (pairs of one expert in ascending pair
// order).  CTA 0 publishes expert_off and the tile counts; the tile lists are written by all CTAs, experts dealt round
// robin.  No scratch, no inter-CTA communication.
constexpr int kSortCta = 256;

__global__ void __launch_bounds__(kSortCta) qwc_moe_sort_kernel(const int32_t* __restrict__ idx, int pairs, int e, int k, int kTileX,
                                                                int gu_rows, int dn_rows, int gu_paired, int32_t* __restrict__ expert_off,
                                                                int32_t* __restrict__ sorted_pair, int32_t* __restrict__ sorted_tok,
                                                                int32_t* __restrict__ inv_perm, qwc_moe_tile* __restrict__ tiles_gu,
                                                                qwc_moe_tile* __restrict__ tiles_dn, int32_t* __restrict__ tile_counts,
                                                                int sort_blocks, const __half* __restrict__ rot_x, int64_t rot_ldx, int rot_h,
                                                                int rot_rows, int rot_vec, __half* __restrict__ rot_out) {
    __shared__ int s_cnt[512];
    __shared__ int s_prev[512];
    __shared__ int s_off[513];
    __shared__ int s_tx[513];
    __shared__ int s_wh[kSortCta / 32][512];
    pdl_enter();
    if (static_cast<int>(blockIdx.x) >= sort_blocks) {
        // Passenger work: the sort keeps a few dozen CTAs busy for ~10 us; the blocks behind them rotate the tokens' rows (which
        // does not depend on the routing) for the row-copy gather that follows, instead of a launch of their own.
        moe_gather_items<uint32_t>(rot_x, rot_ldx, rot_h, nullptr, static_cast<uint32_t>(rot_rows), 1, rot_vec, rot_out,
                                   static_cast<int>(blockIdx.x) - sort_blocks, static_cast<int>(gridDim.x) - sort_blocks);
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lo = blockIdx.x * kSortCta;
    for (int i = tid; i < e; i += kSortCta) s_cnt[i] = 0;
    for (int i = tid; i < (kSortCta / 32) * 512; i += kSortCta) (&s_wh[0][0])[i] = 0;
    __syncthreads();
    const bool vec = (reinterpret_cast<uintptr_t>(idx) & 15) == 0;
    auto count_range = [&](int a, int b) {   // a is a multiple of 256
        if (vec) {
            const int b4 = a + ((b - a) & ~3);
            for (int i = a + tid * 4; i < b4; i += kSortCta * 4) {
                const int4 v = *reinterpret_cast<const int4*>(idx + i);
                if (v.x >= 0 && v.x < e) atomicAdd(&s_cnt[v.x], 1);
                if (v.y >= 0 && v.y < e) atomicAdd(&s_cnt[v.y], 1);
                if (v.z >= 0 && v.z < e) atomicAdd(&s_cnt[v.z], 1);
                if (v.w >= 0 && v.w < e) atomicAdd(&s_cnt[v.w], 1);
            }
            a = b4;
        }
        for (int i = a + tid; i < b; i += kSortCta) {
            const int v = idx[i];
            if (v >= 0 && v < e) atomicAdd(&s_cnt[v], 1);
        }
    };
    count_range(0, min(lo, pairs));
    __syncthreads();
    for (int i = tid; i < e; i += kSortCta) s_prev[i] = s_cnt[i];
    __syncthreads();
    count_range(min(lo, pairs), pairs);
    __syncthreads();
    // exclusive scans over the experts (one warp, each lane a contiguous run of experts)
    if (warp == 0) {
        const int per = (e + 31) / 32;
        const int b0 = min(lane * per, e), b1 = min(b0 + per, e);
        int sc = 0, st = 0;
        for (int i = b0; i < b1; ++i) {
            sc += s_cnt[i];
            st += (s_cnt[i] + kTileX - 1) / kTileX;
        }
        int ic = sc, it = st;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, o), ut = __shfl_up_sync(0xFFFFFFFFu, it, o);
            if (lane >= o) {
                ic += uc;
                it += ut;
            }
        }
        int rc = ic - sc, rt = it - st;
        for (int i = b0; i < b1; ++i) {
            s_off[i] = rc;
            s_tx[i] = rt;
            rc += s_cnt[i];
            rt += (s_cnt[i] + kTileX - 1) / kTileX;
        }
        if (lane == 31) {
            s_off[e] = ic;
            s_tx[e] = it;
        }
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int i = tid; i <= e; i += kSortCta) expert_off[i] = s_off[i];
        if (tid == 0) {
            tile_counts[0] = s_tx[e] * ((gu_rows + kTileW - 1) / kTileW);
            tile_counts[1] = s_tx[e] * ((dn_rows + kTileW - 1) / kTileW);
        }
    }
    // tile lists: weight tiles fastest inside an activation tile, so consecutive tiles re-read the same activations
    for (int ex = blockIdx.x; ex < e && (tiles_gu != nullptr || tiles_dn != nullptr); ex += sort_blocks) {
        const int cnt = s_cnt[ex], ntx = s_tx[ex + 1] - s_tx[ex];
        for (int which = 0; which < 2; ++which) {
            const int rows = which == 0 ? gu_rows : dn_rows;
            qwc_moe_tile* tiles = which == 0 ? tiles_gu : tiles_dn;
            if (tiles == nullptr) continue;
            const int ntw = (rows + kTileW - 1) / kTileW;
            for (int it = tid; it < ntx * ntw; it += kSortCta) {
                const int mt = it / ntw, j = it - mt * ntw;
                tiles[(s_tx[ex] + mt) * ntw + j] = moe_make_tile(ex, rows, j, which == 0 && gu_paired, s_off[ex] + mt * kTileX,
                                                                 min(kTileX, cnt - mt * kTileX));
            }
        }
    }
    // this CTA's pairs
    const int p = lo + tid;
    const int v = p < pairs ? idx[p] : -1;
    const bool valid = v >= 0 && v < e;
    const unsigned same = __match_any_sync(0xFFFFFFFFu, valid ? v : (0x40000000 | lane));
    const int rank_w = __popc(same & ((1u << lane) - 1u));
    if (valid && rank_w == 0) s_wh[warp][v] = __popc(same);
    __syncthreads();
    for (int i = tid; i < e; i += kSortCta) {
        int run = s_prev[i];
#pragma unroll
        for (int w = 0; w < kSortCta / 32; ++w) {
            const int t = s_wh[w][i];
            s_wh[w][i] = run;
            run += t;
        }
    }
    __syncthreads();
    if (p < pairs) {
        if (valid) {
            const int pos = s_off[v] + s_wh[warp][v] + rank_w;
            sorted_pair[pos] = p;
            sorted_tok[pos] = p / k;
            inv_perm[p] = pos;
        } else {
            inv_perm[p] = -1;
        }
    }
}

// Decode-time plan (at most 8 tokens, so an expert holds at most 8 sorted rows): one list entry per (active expert,
// block of output columns) for the gate/up and for the down matmul, each entry served by one CTA of the streaming GEMV
// in segment mode (the twin of the reference's per-(token, route) GEMVs with expert de-duplication,
// Sources/Operators/QWGEMM/QWGemmMoE.swift:117-199).  Entry layout = qwc_gemv_seg of qwc_gemv.cu.
struct MoeSeg {
    int32_t w_row0, col0, cols, x_row0, m, pad0, pad1, pad2;
};

__global__ void __launch_bounds__(512) qwc_moe_decode_plan_kernel(const int32_t* __restrict__ expert_off, int e, int inter, int h,
                                                                  int cols_gu, int cols_dn, MoeSeg* __restrict__ segs_gu,
                                                                  MoeSeg* __restrict__ segs_dn, int32_t* __restrict__ seg_counts) {
    pdl_enter();
    __shared__ int s_warp[16];
    const int ex = threadIdx.x, lane = ex & 31, warp = ex >> 5;
    const int cnt = ex < e ? expert_off[ex + 1] - expert_off[ex] : 0;
    const unsigned act = __ballot_sync(0xFFFFFFFFu, cnt > 0);
    if (lane == 0) s_warp[warp] = __popc(act);
    __syncthreads();
    int before = __popc(act & ((1u << lane) - 1u)), total = 0;
    for (int w = 0; w < 16; ++w) {
        if (w < warp) before += s_warp[w];
        total += s_warp[w];
    }
    const int ngu = (inter + cols_gu - 1) / cols_gu, ndn = (h + cols_dn - 1) / cols_dn;
    if (ex == 0) {
        seg_counts[0] = total * ngu;
        seg_counts[1] = total * ndn;
    }
    if (cnt <= 0) return;
    const int x0 = expert_off[ex];
    for (int j = 0; j < ngu; ++j) {
        MoeSeg sg{ex * 2 * inter, j * cols_gu, min(cols_gu, inter - j * cols_gu), x0, min(cnt, 8), 0, 0, 0};
        segs_gu[before * ngu + j] = sg;
    }
    for (int j = 0; j < ndn; ++j) {
        MoeSeg sg{ex * h, j * cols_dn, min(cols_dn, h - j * cols_dn), x0, min(cnt, 8), 0, 0, 0};
        segs_dn[before * ndn + j] = sg;
    }
}

// xs[p, :] = xr[sorted_tok[p], :] for rows that are rotated already: one warp per sorted row, 16 bytes per lane and step, four
// steps in flight.  A token's row is rotated once (not once per route) and the gather is a plain copy; rows and both bases
// 16-byte aligned, h a multiple of 8.
__global__ void __launch_bounds__(256) qwc_moe_gather_rows_kernel(const __half* __restrict__ xr, int64_t ldx, int h,
                                                                  const int32_t* __restrict__ sorted_tok,
                                                                  const int32_t* __restrict__ expert_off, int e, __half* __restrict__ xs) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int rows = expert_off[e];
    const int nwarps = static_cast<int>(gridDim.x) * (blockDim.x >> 5);
    const int chunks = h / 8;   // 16-byte chunks per row
    for (int pr = static_cast<int>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); pr < rows; pr += nwarps) {
        const uint4* src = reinterpret_cast<const uint4*>(xr + static_cast<int64_t>(sorted_tok[pr]) * ldx);
        uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<int64_t>(pr) * h);
        int c = lane;
        for (; c + 96 < chunks; c += 128) {
            const uint4 a = src[c], b = src[c + 32], cc = src[c + 64], d = src[c + 96];
            dst[c] = a;
            dst[c + 32] = b;
            dst[c + 64] = cc;
            dst[c + 96] = d;
        }
        for (; c < chunks; c += 32) dst[c] = src[c];
    }
}

// h[p, i] = fwht32(f16(silu(g) * u)) over expert-sorted rows; one warp per (row, 32-wide slice of inter).
__global__ void __launch_bounds__(256) qwc_moe_silu_mul_kernel(const __half* __restrict__ gu, const int32_t* __restrict__ row_count,
                                                               int64_t rows_cap, int inter, int rotate, __half* __restrict__ hout) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int units = inter / 32;
    const int64_t rows = row_count != nullptr ? static_cast<int64_t>(*row_count) : rows_cap;
    const int64_t total = rows * units;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t it = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); it < total; it += warps) {
        const int64_t r = it / units;
        const int c = static_cast<int>(it % units) * 32 + lane;
        const float g = __half2float(gu[r * 2 * inter + c]);
        const float u = __half2float(gu[r * 2 * inter + inter + c]);
        float v = __half2float(__float2half_rn((g / (1.0f + expf(-g))) * u));
        if (rotate) {
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) v = fwht_xor_stage(v, s, (lane & s) != 0);
            v = __fmul_rn(v, qwc_inv_sqrt32());
        }
        hout[r * inter + c] = __float2half_rn(v);
    }
}

// out[t, :] = sum_k wts[t, k] * dn[inv_perm[t, k], :] (+ gate[t] * shared[t, :], the shared-expert term of the
// reference's qwg_moe_down_reduce_combine_f32); one thread per (token, VEC columns) with 16-byte loads when VEC
// elements of DnT are 16 bytes (VEC = 8 for f16 rows, 4 for f32 rows; VEC = 2 is the fallback for odd shapes),
// f32 accumulate in route order.
template <typename DnT, typename OutT, int VEC>
__global__ void __launch_bounds__(256) qwc_moe_combine_kernel(const DnT* __restrict__ dn, const int32_t* __restrict__ inv_perm,
                                                              const float* __restrict__ wts, const float* __restrict__ shared,
                                                              const float* __restrict__ gate, int t_rows, int k, int h,
                                                              OutT* __restrict__ out) {
    pdl_enter();
    const int per_row = h / VEC;
    const int64_t total = static_cast<int64_t>(t_rows) * per_row;
    for (int64_t it = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; it < total;
         it += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(it / per_row);
        const int c = static_cast<int>(it % per_row) * VEC;
        float acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
        // eight routes at a time: all positions and weights first, then all rows, then the sums in route order, so the
        // loads of a batch are in flight together instead of one dependent pair after the other
        constexpr int kBatch = 8;
        for (int j0 = 0; j0 < k; j0 += kBatch) {
            int pos[kBatch];
            float w[kBatch];
            float v[kBatch][VEC];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const bool in = j0 + u < k;
                pos[u] = in ? inv_perm[static_cast<int64_t>(t) * k + j0 + u] : -1;
                w[u] = in ? wts[static_cast<int64_t>(t) * k + j0 + u] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[u][i] = 0.0f;
                if (pos[u] < 0) continue;
                const DnT* src = dn + static_cast<int64_t>(pos[u]) * h + c;
                if (sizeof(DnT) == 2) {
                    if (VEC == 8) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(src);
                        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[u][2 * i] = __low2float(h2[i]);
                            v[u][2 * i + 1] = __high2float(h2[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < VEC / 2; ++i) {
                            const __half2 hv = reinterpret_cast<const __half2*>(src)[i];
                            v[u][2 * i] = __low2float(hv);
                            v[u][2 * i + 1] = __high2float(hv);
                        }
                    }
                } else {
                    if (VEC == 4) {
                        const float4 raw = *reinterpret_cast<const float4*>(src);
                        v[u][0] = raw.x; v[u][1] = raw.y; v[u][2] = raw.z; v[u][3] = raw.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < VEC; ++i) v[u][i] = reinterpret_cast<const float*>(src)[i];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
                if (pos[u] >= 0) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
                }
        }
        if (shared != nullptr) {
            const float g = gate[t];
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = fmaf(g, shared[static_cast<int64_t>(t) * h + c + i], acc[i]);
        }
        OutT* dst = out + static_cast<int64_t>(t) * h + c;
        if (sizeof(OutT) == 2) {
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) reinterpret_cast<__half2*>(dst)[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) reinterpret_cast<float2*>(dst)[i] = make_float2(acc[2 * i], acc[2 * i + 1]);
        }
    }
}

int grid_for(const qwc_hal* hal, int64_t items, int per_block, int waves) {
    int64_t g = (items + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * waves;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Scratch layout of qwc_moe_forward (every region 256-byte aligned).
struct MoeScratch {
    size_t idx, wts, counts, expert_off, sorted_pair, sorted_tok, inv_perm, tiles_gu, tiles_dn, tile_counts, xs, gu, hs, dn, total;
};

MoeScratch moe_layout(int64_t t, int64_t e, int64_t k, int64_t h, int64_t inter) {
    MoeScratch s{};
    const int64_t pairs = t * k;
    size_t at = 0;
    auto take = [&](size_t bytes) {
        const size_t o = at;
        at = align_up(at + bytes, 256);
        return o;
    };
    s.idx = take(pairs * 4);
    s.wts = take(pairs * 4);
    s.counts = take((e + 1) * 4);
    s.expert_off = take((e + 1) * 4);
    s.sorted_pair = take(pairs * 4);
    s.sorted_tok = take(pairs * 4);
    s.inv_perm = take(pairs * 4);
    s.tiles_gu = take(qwc_moe_max_tiles(pairs, e, 2 * inter) * sizeof(qwc_moe_tile));
    s.tiles_dn = take(qwc_moe_max_tiles(pairs, e, h) * sizeof(qwc_moe_tile));
    s.tile_counts = take(16);
    s.xs = take(pairs * h * 2);
    s.gu = take(pairs * 2 * inter * 2);
    s.hs = take(pairs * inter * 2);
    s.dn = take(pairs * h * 2);
    s.total = at;
    return s;
}

}  // namespace

extern "C" {

int32_t qwc_moe_tile_rows(int64_t pairs, int64_t e) { return moe_tile_rows(pairs, e > 0 ? e : 1); }

int64_t qwc_moe_max_tiles(int64_t pairs, int64_t e, int64_t rows_per_expert) {
    // sum over experts of ceil(cnt / tile rows) <= min(pairs, e + pairs / tile rows)
    int64_t tx = e + pairs / moe_tile_rows(pairs, e);
    if (tx > pairs) tx = pairs;
    return tx * ((rows_per_expert + kTileW - 1) / kTileW);
}

int qwc_moe_router_gemm(qwc_hal* hal, qwc_stream stream, const void* x, int32_t x_dtype, int64_t ldx, int64_t t, int64_t h,
                        const void* w, int32_t w_dtype, int64_t e, float* logits) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    // QWGemmMoERouter.swift:82: the router GEMM needs K % 32 == 0
    if (h <= 0 || h % 32 != 0) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "hidden=%lld must be a positive multiple of 32", (long long)h);
    if (e <= 0 || t < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "bad extents");
    if (t == 0) return QWC_OK;
    if (ldx < h) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx < hidden");
    if (!x || !w || !logits) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    if (x_dtype != QWC_F16 && x_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "activations must be f16 or f32");
    if (w_dtype != QWC_F16 && w_dtype != QWC_F32 && w_dtype != QWC_BF16) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "router weights must be bf16, f16 or f32");
    const dim3 grid(static_cast<unsigned>((e + 63) / 64), static_cast<unsigned>((t + 63) / 64));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int ti = static_cast<int>(t), ei = static_cast<int>(e), hi = static_cast<int>(h);
#define QWC_ROUTER_LAUNCH(XT, WT) \
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_router_gemm_kernel<XT, WT>, grid, dim3(256), 0, st, static_cast<const XT*>(x), ldx, static_cast<const WT*>(w), ti, ei, hi, logits))
    if (x_dtype == QWC_F32) {
        if (w_dtype == QWC_F32) QWC_ROUTER_LAUNCH(float, float);
        else if (w_dtype == QWC_F16) QWC_ROUTER_LAUNCH(float, __half);
        else QWC_ROUTER_LAUNCH(float, unsigned short);
    } else {
        if (w_dtype == QWC_F32) QWC_ROUTER_LAUNCH(__half, float);
        else if (w_dtype == QWC_F16) QWC_ROUTER_LAUNCH(__half, __half);
        else QWC_ROUTER_LAUNCH(__half, unsigned short);
    }
#undef QWC_ROUTER_LAUNCH
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

int qwc_moe_route(qwc_hal* hal, qwc_stream stream, const float* logits, int64_t t, int64_t e, int64_t k, int32_t norm_topk,
                  float routed_scale, int32_t* idx, float* wts) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    // the reference's limits (QWGemmMoERouter.swift:22): e <= 512, k <= 16
    if (e <= 0 || e > 512) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "experts=%lld must be in 1..512", (long long)e);
    if (k <= 0 || k > 16 || k > e) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "top-k=%lld must be in 1..16 and <= experts", (long long)k);
    if (t < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "t is negative");
    if (t == 0) return QWC_OK;
    if (!logits || !idx || !wts) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    const int blocks = static_cast<int>((t + 3) / 4);
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_route_kernel, dim3(blocks), dim3(128), 0, static_cast<cudaStream_t>(stream), logits,
                                static_cast<int>(t), static_cast<int>(e), static_cast<int>(k), norm_topk, routed_scale, idx, wts));
    return QWC_OK;
}

// A rotation job that rides on the sort launch (see qwc_moe_sort_kernel): out[r, :] = rot(x[r, :]) for `rows` rows of h.
struct MoeRotateJob {
    const __half* x;
    int64_t ldx;
    int h, rows, vec;
    __half* out;
};
static int moe_group_pairs_impl(qwc_hal* hal, qwc_stream stream, const int32_t* idx, int64_t pairs, int64_t e, int64_t k,
                                int32_t* expert_off, int32_t* sorted_pair, int32_t* sorted_tok, int32_t* inv_perm,
                                int64_t gu_rows, int64_t dn_rows, int32_t gu_epilogue, qwc_moe_tile* tiles_gu, qwc_moe_tile* tiles_dn,
                                int32_t* tile_counts, const MoeRotateJob* rot, bool* rot_done);

int qwc_moe_group_pairs(qwc_hal* hal, qwc_stream stream, const int32_t* idx, int64_t pairs, int64_t e, int64_t k,
                        int32_t* expert_off, int32_t* sorted_pair, int32_t* sorted_tok, int32_t* inv_perm,
                        int64_t gu_rows, int64_t dn_rows, int32_t gu_epilogue, qwc_moe_tile* tiles_gu, qwc_moe_tile* tiles_dn,
                        int32_t* tile_counts) {
    return moe_group_pairs_impl(hal, stream, idx, pairs, e, k, expert_off, sorted_pair, sorted_tok, inv_perm, gu_rows, dn_rows,
                                gu_epilogue, tiles_gu, tiles_dn, tile_counts, nullptr, nullptr);
}

// rot != nullptr: the one-launch sort also carries the rotation job; *rot_done says whether it did (the three-pass sort of long
// pair lists does not).
static int moe_group_pairs_impl(qwc_hal* hal, qwc_stream stream, const int32_t* idx, int64_t pairs, int64_t e, int64_t k,
                                int32_t* expert_off, int32_t* sorted_pair, int32_t* sorted_tok, int32_t* inv_perm,
                                int64_t gu_rows, int64_t dn_rows, int32_t gu_epilogue, qwc_moe_tile* tiles_gu, qwc_moe_tile* tiles_dn,
                                int32_t* tile_counts, const MoeRotateJob* rot, bool* rot_done) {
    qwc_clear_error();
    if (rot_done) *rot_done = false;
    const int paired = gu_epilogue != QWC_EPI_NONE;
    if (paired && gu_rows % kTileW != 0)
        return qwc_fail(QWC_ERR_BAD_GEOMETRY, "a SwiGLU epilogue needs inter %% 64 == 0, got gate||up rows = %lld", (long long)gu_rows);
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (e <= 0 || e > 512) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "experts=%lld must be in 1..512", (long long)e);
    if (k <= 0 || pairs < 0 || pairs % k != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "pairs=%lld is not a multiple of k=%lld", (long long)pairs, (long long)k);
    if (pairs >= (int64_t(1) << 30)) return qwc_fail(QWC_ERR_BAD_SHAPE, "too many pairs");
    if (!idx || !expert_off || !sorted_pair || !sorted_tok || !inv_perm || !tile_counts) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pairs <= (int64_t(1) << 18)) {
        // one launch: every CTA reads the whole pair list (<= 1 MB, L2-resident)
        int grid = static_cast<int>(pairs > 0 ? (pairs + kSortCta - 1) / kSortCta : 1);
        // the tile lists are written expert by expert, experts dealt over the CTAs: a short pair list still gets 32 CTAs for that
        if ((tiles_gu != nullptr || tiles_dn != nullptr) && grid < 32 && grid < e) grid = static_cast<int>(e < 32 ? e : 32);
        const int rot_blocks = rot != nullptr ? grid_for(hal, static_cast<int64_t>(rot->rows) * (rot->h / 32), 64, 16) : 0;
        QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_sort_kernel, dim3(grid + rot_blocks), dim3(kSortCta), 0, st, idx, static_cast<int>(pairs),
                                    static_cast<int>(e), static_cast<int>(k), moe_tile_rows(pairs, e), static_cast<int>(gu_rows),
                                    static_cast<int>(dn_rows), paired, expert_off, sorted_pair, sorted_tok, inv_perm, tiles_gu, tiles_dn,
                                    tile_counts, grid, rot != nullptr ? rot->x : static_cast<const __half*>(nullptr),
                                    rot != nullptr ? rot->ldx : int64_t(0), rot != nullptr ? rot->h : 0, rot != nullptr ? rot->rows : 0,
                                    rot != nullptr ? rot->vec : 0, rot != nullptr ? rot->out : static_cast<__half*>(nullptr)));
        if (rot_done) *rot_done = rot != nullptr;
        return QWC_OK;
    }
    // larger lists: three passes, one warp per expert.
    // expert_off doubles as the count buffer of pass 1; the plan kernel reads all counts before it writes offsets
    const int warps = static_cast<int>(e) + 1;
    qwc_moe_count_kernel<<<(warps + 15) / 16, 512, 0, st>>>(idx, static_cast<int>(pairs), static_cast<int>(e), expert_off, inv_perm);
    QWC_CUDA_TRY(cudaGetLastError());
    qwc_moe_plan_kernel<<<1, 512, 0, st>>>(expert_off, static_cast<int>(e), moe_tile_rows(pairs, e), expert_off, static_cast<int>(gu_rows),
                                           static_cast<int>(dn_rows), paired, tiles_gu, tiles_dn, tile_counts);
    QWC_CUDA_TRY(cudaGetLastError());
    qwc_moe_place_kernel<<<(static_cast<int>(e) + 15) / 16, 512, 0, st>>>(idx, static_cast<int>(pairs), static_cast<int>(e),
                                                                       static_cast<int>(k), expert_off, sorted_pair, sorted_tok, inv_perm);
    QWC_CUDA_TRY(cudaGetLastError());
    return QWC_OK;
}

static int moe_gather_impl(qwc_hal* hal, qwc_stream stream, const void* x_f16, int64_t ldx, int64_t h, const int32_t* sorted_tok,
                           const int32_t* expert_off, int64_t e, int64_t pairs, int32_t x_is_rotated, void* xs_f16, int64_t t,
                           void* tmp, size_t tmp_bytes);

int qwc_moe_gather(qwc_hal* hal, qwc_stream stream, const void* x_f16, int64_t ldx, int64_t h, const int32_t* sorted_tok,
                   const int32_t* expert_off, int64_t e, int64_t pairs, int32_t x_is_rotated, void* xs_f16) {
    return moe_gather_impl(hal, stream, x_f16, ldx, h, sorted_tok, expert_off, e, pairs, x_is_rotated, xs_f16, 0, nullptr, 0);
}

// t > 0 with a temp of t * h f16 (16-byte aligned): standard-basis rows are rotated once per token into the temp and the gather
// is a row copy (a token has k routes: the per-route rotation of the one-pass kernel was k times the butterfly work and
// bounded that kernel by its instruction stream, 27 us at 2048 tokens x 8 routes x 2048 wide against ~10 us of copying).
static int moe_gather_impl(qwc_hal* hal, qwc_stream stream, const void* x_f16, int64_t ldx, int64_t h, const int32_t* sorted_tok,
                           const int32_t* expert_off, int64_t e, int64_t pairs, int32_t x_is_rotated, void* xs_f16, int64_t t,
                           void* tmp, size_t tmp_bytes) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (h <= 0 || h % 32 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "hidden=%lld must be a positive multiple of 32", (long long)h);
    if (ldx < h) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx < hidden");
    if (pairs == 0) return QWC_OK;
    if (!x_f16 || !sorted_tok || !expert_off || !xs_f16) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    const int vec = reinterpret_cast<uintptr_t>(x_f16) % 16 == 0 && ldx % 8 == 0;
    if (reinterpret_cast<uintptr_t>(xs_f16) % 16 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "xs must be 16-byte aligned");
    const bool aligned_out = h % 8 == 0;
    const bool temp_ok = t > 0 && tmp != nullptr && reinterpret_cast<uintptr_t>(tmp) % 16 == 0 &&
                         tmp_bytes >= static_cast<size_t>(t) * static_cast<size_t>(h) * 2 && t * (h / 32) < (1ll << 31);
    if (aligned_out && pairs < (1ll << 31) && ((x_is_rotated && vec) || (!x_is_rotated && temp_ok && pairs > t))) {
        const __half* rows_src = static_cast<const __half*>(x_f16);
        int64_t rows_ld = ldx;
        if (!x_is_rotated) {
            const int g0 = grid_for(hal, t * (h / 32), 64, 16);
            QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_gather_kernel<uint32_t>, dim3(g0), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                        static_cast<const __half*>(x_f16), ldx, static_cast<int>(h), static_cast<const int32_t*>(nullptr),
                                        expert_off, static_cast<int>(t), 1, vec, static_cast<__half*>(tmp)));
            rows_src = static_cast<const __half*>(tmp);
            rows_ld = h;
        }
        const int g1 = grid_for(hal, pairs, 8, 8);
        QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_gather_rows_kernel, dim3(g1), dim3(256), 0, static_cast<cudaStream_t>(stream), rows_src, rows_ld,
                                    static_cast<int>(h), sorted_tok, expert_off, static_cast<int>(e), static_cast<__half*>(xs_f16)));
        return QWC_OK;
    }
    const int grid = grid_for(hal, pairs * (h / 32), 64, 16);
    // 32-bit item indices while the last item plus one grid step of the loop still fits
    const bool idx32 = pairs * (h / 32) + static_cast<int64_t>(grid) * 64 < (1ll << 32);
    if (idx32)
        QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_gather_kernel<uint32_t>, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                    static_cast<const __half*>(x_f16), ldx, static_cast<int>(h), sorted_tok, expert_off, static_cast<int>(e),
                                    static_cast<int>(!x_is_rotated), vec, static_cast<__half*>(xs_f16)));
    else
        QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_gather_kernel<int64_t>, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                    static_cast<const __half*>(x_f16), ldx, static_cast<int>(h), sorted_tok, expert_off, static_cast<int>(e),
                                    static_cast<int>(!x_is_rotated), vec, static_cast<__half*>(xs_f16)));
    return QWC_OK;
}

int qwc_moe_grouped_gemm(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* bank, const void* xs_f16, int64_t pairs,
                         const qwc_moe_tile* tiles, const int32_t* tile_count, int64_t max_tiles, int32_t x_tile_rows, void* y,
                         int32_t y_dtype, int64_t ldy, int32_t epilogue) {
    qwc_clear_error();
    if (epilogue < QWC_EPI_NONE || epilogue > QWC_EPI_SILU_PAIR_FWHT) return qwc_fail(QWC_ERR_BAD_SHAPE, "unknown epilogue %d", epilogue);
    if (x_tile_rows != 64 && x_tile_rows != 128 && x_tile_rows != 192 && x_tile_rows != 256)
        return qwc_fail(QWC_ERR_BAD_GEOMETRY, "x_tile_rows must be 64, 128, 192 or 256 (qwc_moe_tile_rows)");
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (!bank || !bank->blocks) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "bank is null");
    if (pairs <= 0 || max_tiles <= 0) return QWC_OK;
    if (!xs_f16 || !tiles || !tile_count || !y) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    if (y_dtype != QWC_F16 && y_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "y dtype must be f16 or f32");
    // The grouped door uses the tensor-core kernel only: K % 128 == 0, HQ4_G32_M5 or HQ8_G32, 16-byte aligned bank.
    if (int rc0 = qwc_check_view(bank)) return rc0;
    if (!qwc_gemm_tc_supported(hal, bank, 17, QWC_EPI_NONE))
        return qwc_fail(QWC_ERR_BLOCKED, "grouped expert GEMM needs an HQ4_G32_M5 / HQ8_G32 bank with k %% 128 == 0 or an HQ4_G64 bank with k %% 256 == 0, 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(xs_f16) % 16 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "xs must be 16-byte aligned");
    return qwc_launch_gemm_tc_grouped(hal, static_cast<cudaStream_t>(stream), bank, xs_f16, pairs, tiles, tile_count, max_tiles, y,
                                      y_dtype, ldy, x_tile_rows, epilogue);
}

int qwc_moe_silu_mul(qwc_hal* hal, qwc_stream stream, const void* gu_f16, int64_t rows, int64_t inter, int32_t rotate,
                     void* h_f16) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (inter <= 0 || inter % 32 != 0) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "inter=%lld must be a positive multiple of 32", (long long)inter);
    if (rows <= 0) return QWC_OK;
    if (!gu_f16 || !h_f16) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_silu_mul_kernel, dim3(grid_for(hal, rows * (inter / 32), 8, 16)), dim3(256), 0,
                                static_cast<cudaStream_t>(stream), static_cast<const __half*>(gu_f16), static_cast<const int32_t*>(nullptr),
                                rows, static_cast<int>(inter), static_cast<int>(rotate), static_cast<__half*>(h_f16)));
    return QWC_OK;
}

int qwc_moe_combine_shared(qwc_hal* hal, qwc_stream stream, const void* dn, int32_t dn_dtype, const int32_t* inv_perm,
                            const float* wts, const float* shared_f32, const float* gate_f32, int64_t t, int64_t k, int64_t h,
                            void* out, int32_t out_dtype) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (h <= 0 || h % 2 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "hidden must be even");
    if ((dn_dtype != QWC_F16 && dn_dtype != QWC_F32) || (out_dtype != QWC_F16 && out_dtype != QWC_F32))
        return qwc_fail(QWC_ERR_BAD_SHAPE, "dtypes must be f16 or f32");
    if ((shared_f32 == nullptr) != (gate_f32 == nullptr)) return qwc_fail(QWC_ERR_BAD_SHAPE, "shared rows and their gate come together");
    if (t <= 0) return QWC_OK;
    if (!dn || !inv_perm || !wts || !out) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int ti = static_cast<int>(t), ki = static_cast<int>(k), hi = static_cast<int>(h);
    const int wide = dn_dtype == QWC_F16 ? 8 : 4;   // elements of a 16-byte load
    const bool vec = h % wide == 0 && reinterpret_cast<uintptr_t>(dn) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0;
    const int grid = grid_for(hal, t * (h / (vec ? wide : 2)), 256, 16);
    cudaError_t e;
#define QWC_COMBINE(DT, OT, V)                                                                                                  \
    e = qwc_launch_pdl(qwc_moe_combine_kernel<DT, OT, V>, dim3(grid), dim3(256), 0, st, static_cast<const DT*>(dn), inv_perm, wts, \
                       shared_f32, gate_f32, ti, ki, hi, static_cast<OT*>(out))
    if (dn_dtype == QWC_F16 && out_dtype == QWC_F32) { if (vec) QWC_COMBINE(__half, float, 8); else QWC_COMBINE(__half, float, 2); }
    else if (dn_dtype == QWC_F16) { if (vec) QWC_COMBINE(__half, __half, 8); else QWC_COMBINE(__half, __half, 2); }
    else if (out_dtype == QWC_F32) { if (vec) QWC_COMBINE(float, float, 4); else QWC_COMBINE(float, float, 2); }
    else { if (vec) QWC_COMBINE(float, __half, 4); else QWC_COMBINE(float, __half, 2); }
#undef QWC_COMBINE
    QWC_CUDA_TRY(e);
    return QWC_OK;
}

int qwc_moe_combine(qwc_hal* hal, qwc_stream stream, const void* dn, int32_t dn_dtype, const int32_t* inv_perm,
                    const float* wts, int64_t t, int64_t k, int64_t h, void* out, int32_t out_dtype) {
    return qwc_moe_combine_shared(hal, stream, dn, dn_dtype, inv_perm, wts, nullptr, nullptr, t, k, h, out, out_dtype);
}

size_t qwc_moe_scratch_bytes(int64_t t, int64_t e, int64_t k, int64_t h, int64_t inter) {
    if (t <= 0 || e <= 0 || k <= 0 || h <= 0 || inter <= 0) return 0;
    return moe_layout(t, e, k, h, inter).total;
}

int qwc_moe_forward(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* bank_gu, const qwc_weight_view* bank_dn,
                    int64_t e, int64_t inter, const void* x_f16, int64_t t, int64_t ldx, int32_t x_is_rotated,
                    const float* logits, int64_t k, int32_t norm_topk, float routed_scale, void* out, int32_t out_dtype,
                    void* scratch, size_t scratch_bytes) {
    qwc_clear_error();
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (!bank_gu || !bank_dn) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "expert banks are null");
    const int64_t h = bank_gu->k;
    if (e <= 0 || e > 512) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "experts=%lld must be in 1..512", (long long)e);
    if (k <= 0 || k > 16 || k > e) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "top-k=%lld must be in 1..16 and <= experts", (long long)k);
    if (inter <= 0 || h <= 0) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "empty expert banks");
    // Bank geometry (QWMoEOperator.Weights, QWMoEOperator.swift:10-130): gate||up is [e * 2 * inter, h], down is [e * h, inter].
    if (bank_gu->n != e * 2 * inter) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "gate/up bank has %lld rows, expected e * 2 * inter = %lld", (long long)bank_gu->n, (long long)(e * 2 * inter));
    if (bank_dn->n != e * h || bank_dn->k != inter) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "down bank must be [e * hidden, inter] = [%lld, %lld]", (long long)(e * h), (long long)inter);
    if (t < 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "t is negative");
    if (t == 0) return QWC_OK;
    if (!x_f16 || !logits || !out) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    const MoeScratch L = moe_layout(t, e, k, h, inter);
    if (!scratch || scratch_bytes < L.total) return qwc_fail(QWC_ERR_BAD_SHAPE, "scratch of %zu bytes needed (qwc_moe_scratch_bytes), got %zu", L.total, scratch_bytes);
    if (reinterpret_cast<uintptr_t>(scratch) % 256 != 0) return qwc_fail(QWC_ERR_BAD_SHAPE, "scratch must be 256-byte aligned");
    // Every refusal comes before the first launch (QWGemm.swift:216-217; Tests/QWGEMMTests/QWGEMMTests.swift:221-248): the
    // checks of the doors called below are made here, for the path this call will take.
    if (int rc0 = qwc_check_view(bank_gu)) return rc0;
    if (int rc0 = qwc_check_view(bank_dn)) return rc0;
    if (h % 32 != 0 || inter % 32 != 0) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "hidden and inter must be multiples of 32");
    if (ldx < h) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx < hidden");
    if (out_dtype != QWC_F16 && out_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "out dtype must be f16 or f32");
    if (t * k >= (int64_t(1) << 30)) return qwc_fail(QWC_ERR_BAD_SHAPE, "too many pairs");
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    const int64_t pairs = t * k;
    int32_t* idx = reinterpret_cast<int32_t*>(sc + L.idx);
    float* wts = reinterpret_cast<float*>(sc + L.wts);
    int32_t* expert_off = reinterpret_cast<int32_t*>(sc + L.expert_off);
    int32_t* sorted_pair = reinterpret_cast<int32_t*>(sc + L.sorted_pair);
    int32_t* sorted_tok = reinterpret_cast<int32_t*>(sc + L.sorted_tok);
    int32_t* inv_perm = reinterpret_cast<int32_t*>(sc + L.inv_perm);
    qwc_moe_tile* tiles_gu = reinterpret_cast<qwc_moe_tile*>(sc + L.tiles_gu);
    qwc_moe_tile* tiles_dn = reinterpret_cast<qwc_moe_tile*>(sc + L.tiles_dn);
    int32_t* tile_counts = reinterpret_cast<int32_t*>(sc + L.tile_counts);
    int rc;
    // ---- decode / verify sizes: per-expert streaming GEMVs over a device-side segment list
    const int64_t rb_gu = (h / bank_gu->group) * qwc_block_bytes(bank_gu->kind, bank_gu->bits, bank_gu->group);
    const int64_t rb_dn = (inter / bank_dn->group) * qwc_block_bytes(bank_dn->kind, bank_dn->bits, bank_dn->group);
    const bool no_decode_path = tune_env("QWC_MOE_NO_DECODE_PATH", 0) != 0;
    bool decode_path = t <= 8 && !no_decode_path && rb_gu % 16 == 0 && rb_dn % 16 == 0 && 8 * h * 2 <= 112 * 1024 &&
                       8 * inter * 2 <= 112 * 1024 && reinterpret_cast<uintptr_t>(bank_gu->blocks) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(bank_dn->blocks) % 16 == 0;
    int cols_gu = 0, cols_dn = 0;
    int64_t max_gu = 0, max_dn = 0;
    if (decode_path) {
        // as many column blocks per expert as keep one wave of CTAs busy when every pair names a different expert
        // (whole 32-column blocks; the floors keep the lists inside the tile-list regions of the scratch)
        const int64_t act = pairs < e ? pairs : e;
        auto pick_cols = [&](int64_t n_out, int64_t floor_cols) {
            const int64_t nseg = hal->sm_count / act > 1 ? hal->sm_count / act : 1;
            int64_t c = ((n_out + nseg - 1) / nseg + 31) / 32 * 32;
            if (c < floor_cols) c = floor_cols;
            return static_cast<int>(c);
        };
        cols_gu = pick_cols(inter, 64);
        cols_dn = pick_cols(h, 128);
        max_gu = act * ((inter + cols_gu - 1) / cols_gu);
        max_dn = act * ((h + cols_dn - 1) / cols_dn);
        decode_path = static_cast<size_t>(max_gu) * sizeof(MoeSeg) <= static_cast<size_t>(qwc_moe_max_tiles(pairs, e, 2 * inter)) * sizeof(qwc_moe_tile) &&
                      static_cast<size_t>(max_dn) * sizeof(MoeSeg) <= static_cast<size_t>(qwc_moe_max_tiles(pairs, e, h)) * sizeof(qwc_moe_tile);
    }
    if (!decode_path && (!qwc_gemm_tc_supported(hal, bank_gu, 17, QWC_EPI_NONE) || !qwc_gemm_tc_supported(hal, bank_dn, 17, QWC_EPI_NONE)))
        return qwc_fail(QWC_ERR_BLOCKED, "the grouped expert GEMMs need HQ4_G32_M5 / HQ8_G32 banks with k %% 128 == 0 or HQ4_G64 banks with k %% 256 == 0, "
                                         "16-byte aligned");
    if ((rc = qwc_moe_route(hal, stream, logits, t, e, k, norm_topk, routed_scale, idx, wts))) return rc;
    if (decode_path) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if ((rc = qwc_moe_group_pairs(hal, stream, idx, pairs, e, k, expert_off, sorted_pair, sorted_tok, inv_perm, 2 * inter, h,
                                      QWC_EPI_NONE, nullptr, nullptr, tile_counts))) return rc;
        MoeSeg* segs_gu = reinterpret_cast<MoeSeg*>(tiles_gu);
        MoeSeg* segs_dn = reinterpret_cast<MoeSeg*>(tiles_dn);
        QWC_CUDA_TRY(qwc_launch_pdl(qwc_moe_decode_plan_kernel, dim3(1), dim3(512), 0, st, expert_off, static_cast<int>(e),
                                    static_cast<int>(inter), static_cast<int>(h), cols_gu, cols_dn, segs_gu, segs_dn, tile_counts + 2));
        if ((rc = qwc_moe_gather(hal, stream, x_f16, ldx, h, sorted_tok, expert_off, e, pairs, x_is_rotated, sc + L.xs))) return rc;
        if ((rc = qwc_launch_gemv_segments(hal, st, bank_gu, sc + L.xs, h, sc + L.hs, QWC_F16, inter, QWC_EPI_SILU_PAIR_FWHT, inter,
                                           cols_gu, segs_gu, tile_counts + 2, max_gu))) return rc;
        if ((rc = qwc_launch_gemv_segments(hal, st, bank_dn, sc + L.hs, inter, sc + L.dn, QWC_F16, h, QWC_EPI_NONE, h, cols_dn,
                                           segs_dn, tile_counts + 3, max_dn))) return rc;
        return qwc_moe_combine(hal, stream, sc + L.dn, QWC_F16, inv_perm, wts, t, k, h, out, out_dtype);
    }
    // SwiGLU + FWHT run in the gate/up GEMM's epilogue when the tiles can pair 64 gate rows with their up rows
    const int32_t gu_epi = inter % 64 == 0 ? QWC_EPI_SILU_PAIR_FWHT : QWC_EPI_NONE;
    // The gate/up region of the scratch is idle until the gate/up GEMM writes it (never, with the fused epilogue): it holds the
    // rotated copy of x that the row-copy gather reads.  The rotation rides on the sort launch when it can.
    const size_t tmp_bytes = static_cast<size_t>(pairs) * 2 * inter * 2;
    MoeRotateJob rot{static_cast<const __half*>(x_f16), ldx, static_cast<int>(h), static_cast<int>(t),
                     reinterpret_cast<uintptr_t>(x_f16) % 16 == 0 && ldx % 8 == 0, reinterpret_cast<__half*>(sc + L.gu)};
    const bool want_rot = !x_is_rotated && k > 1 && h % 32 == 0 && tmp_bytes >= static_cast<size_t>(t) * h * 2 && t * (h / 32) < (1ll << 31);
    bool rotated_here = false;
    if ((rc = moe_group_pairs_impl(hal, stream, idx, pairs, e, k, expert_off, sorted_pair, sorted_tok, inv_perm, 2 * inter, h, gu_epi,
                                   tiles_gu, tiles_dn, tile_counts, want_rot ? &rot : nullptr, &rotated_here))) return rc;
    if (rotated_here) {
        if ((rc = moe_gather_impl(hal, stream, sc + L.gu, h, h, sorted_tok, expert_off, e, pairs, 1, sc + L.xs, 0, nullptr, 0))) return rc;
    } else if ((rc = moe_gather_impl(hal, stream, x_f16, ldx, h, sorted_tok, expert_off, e, pairs, x_is_rotated, sc + L.xs, t, sc + L.gu,
                                     tmp_bytes))) {
        return rc;
    }
    const int32_t xrows = qwc_moe_tile_rows(pairs, e);
    if (gu_epi != QWC_EPI_NONE) {
        if ((rc = qwc_moe_grouped_gemm(hal, stream, bank_gu, sc + L.xs, pairs, tiles_gu, tile_counts, qwc_moe_max_tiles(pairs, e, 2 * inter),
                                       xrows, sc + L.hs, QWC_F16, inter, gu_epi))) return rc;
    } else {
        if ((rc = qwc_moe_grouped_gemm(hal, stream, bank_gu, sc + L.xs, pairs, tiles_gu, tile_counts, qwc_moe_max_tiles(pairs, e, 2 * inter),
                                       xrows, sc + L.gu, QWC_F16, 2 * inter, QWC_EPI_NONE))) return rc;
        if ((rc = qwc_moe_silu_mul(hal, stream, sc + L.gu, pairs, inter, 1, sc + L.hs))) return rc;
    }
    if ((rc = qwc_moe_grouped_gemm(hal, stream, bank_dn, sc + L.hs, pairs, tiles_dn, tile_counts + 1, qwc_moe_max_tiles(pairs, e, h),
                                   xrows, sc + L.dn, QWC_F16, h, QWC_EPI_NONE))) return rc;
    return qwc_moe_combine(hal, stream, sc + L.dn, QWC_F16, inv_perm, wts, t, k, h, out, out_dtype);
}

}  // extern "C"
