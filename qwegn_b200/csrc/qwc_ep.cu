// Expert-parallel exchange of the mixture-of-experts block over peer memory (no counterpart in the reference, which
// runs on one device; the places where the exchange sits are the reference's own stages: the pair sort, where rows
// are grouped by expert -- Sources/QWMetal/gemm/qwgemm_moe_group_f32.metal:10-148 -- and the weighted combine, where
// the experts' outputs return to their tokens -- Sources/QWMetal/gemm/qwgemm_moe_nax_f16.metal:7-126; the chain is
// QWMoEOperator.encodeResident, Sources/Operators/QWGEMM/QWMoEOperator.swift:246-362).
//
// Experts [r * E / R, (r + 1) * E / R) live on rank r; every rank routes its own tokens.  Three phases per call, each
// an entry point, all on the caller's stream, no host synchronisation and no NCCL:
//   dispatch  route -> pair sort by (global) expert -> one kernel rotates each sorted row and stores it straight into
//             the receive buffer of the rank that owns its expert (plain peer stores over NVLink), with the per-expert
//             row counts; the last CTA to finish raises this rank's flag on every peer;
//   experts   waits (bounded) for every peer's flag, regroups the received rows by local expert (prefix sums over the
//             count tables, tile lists of the grouped GEMMs, one copy), runs the two grouped expert GEMMs and stores
//             every result row back into the return buffer of the rank it came from, at the position the row had in
//             that rank's sorted order; then raises the return flag on every peer;
//   combine   waits (bounded) for every peer's return flag and runs the weighted combine over the returned rows.
// A rank's buffers are reused from call to call: a peer can only start the next call's dispatch after its own combine,
// which needs this rank's return flag, which is raised after this rank has read everything the peer sent.  Flags carry
// the call number, so stale values never match.  With fewer GPUs than ranks the phases can be run rank after rank on
// one device (each wait then finds its flags already raised), which is how the protocol is tested on a single GPU.
#include "qwc_common.cuh"

int qwc_launch_gemm_tc_grouped(const qwc_hal*, cudaStream_t, const qwc_weight_view*, const void*, int64_t, const qwc_moe_tile*,
                               const int32_t*, int64_t, void*, int, int64_t, int, int);
bool qwc_gemm_tc_supported(const qwc_hal*, const qwc_weight_view*, int64_t, int);

namespace {

constexpr int kTileW = 128;   // weight rows per grouped-GEMM tile (as in qwc_moe.cu)
constexpr int kMaxWorld = 8;
constexpr int kMaxExperts = 512;

struct EpPeers {
    __half* recv[kMaxWorld];      // rank r's receive buffer: f16 [world][capacity][hidden]; slot [s] is written by rank s
    int32_t* counts[kMaxWorld];   // rank r's count table: i32 [world][experts_local + 2]; row [s] is written by rank s:
                                  //   rows per local expert, then rank s's first sorted row for rank r, then the total
    __half* ret[kMaxWorld];       // rank r's return buffer: f16 [capacity][hidden], in rank r's own sorted order
    uint32_t* flags[kMaxWorld];   // rank r's flags: u32 [2][world] (dispatch arrived / results arrived, per source) + 2 tickets
};

// Flag accesses are relaxed (volatile) and the ordering comes from ONE system-scope fence on each side: a system fence, a
// release store or an acquire load each cost about 3.5 us on B200, and a poll loop of acquire loads pays that per poll.
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// "Last CTA done": the CTA's stores are ordered before its barrier; one thread per CTA then fences at system scope
// (cumulative over what the barrier ordered before it: one fence per CTA, not one per thread) and takes a ticket; the CTA
// that takes the last one resets the ticket, fences again and raises `word` (call number) on every peer.
__device__ __forceinline__ void raise_flags_when_grid_done(uint32_t* ticket, const EpPeers& peers, int world, int flag_index, uint32_t epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1u) {
            *ticket = 0u;
            __threadfence_system();
            for (int d = 0; d < world; ++d) st_relaxed_sys(peers.flags[d] + flag_index, epoch);   // after the fence above
        }
    }
}

// The call number: counted by the host (epoch_state == null) or by the device (*epoch_state + 1: the form for calls
// captured in a CUDA graph, where a host value would repeat at every replay).  Read after pdl_enter(), when every
// kernel of the previous call has completed.
__device__ __forceinline__ uint32_t ep_epoch(const uint32_t* epoch_state, uint32_t host_epoch) {
    return epoch_state != nullptr ? *reinterpret_cast<const volatile uint32_t*>(epoch_state) + 1u : host_epoch;
}

// Waits (bounded) until flags[base + s] == epoch for every s < world; one warp, lane s polls flag s.  bump != 0 (the
// last kernel of a call that needs the call number): stores the new number into the device-side counter.
__global__ void __launch_bounds__(32) qwc_ep_wait_kernel(const uint32_t* flags, int base, int world, uint32_t* epoch_state,
                                                         uint32_t host_epoch, int bump, uint64_t limit_ns, int32_t* status) {
    pdl_enter();
    const int lane = threadIdx.x;
    const uint32_t epoch = ep_epoch(epoch_state, host_epoch);
    if (lane < world) {
        bool got = false;
        const uint64_t t0 = qwc_globaltimer_ns();
        for (uint32_t spin = 0;; ++spin) {
            if (ld_relaxed_sys(flags + base + lane) == epoch) {
                got = true;
                break;
            }
            if ((spin & 15u) == 15u && qwc_globaltimer_ns() - t0 > limit_ns) break;
            __nanosleep(spin < 256 ? 40 : 250);
        }
        if (!got) atomicCAS(status, 0, QWC_DEV_WAIT_PEER_TIMEOUT);
        __threadfence_system();   // acquire side: what the peer wrote before it raised the flag is ordered before what follows
    }
    __syncwarp();
    if (bump && epoch_state != nullptr && lane == 0) *reinterpret_cast<volatile uint32_t*>(epoch_state) = epoch;
}

// Dispatch: xs row p (sorted order) = rot(x[sorted_tok[p], :]) goes to the rank that owns its expert.  A quad of lanes
// handles one (row, 32-element unit) as in the single-device gather kernel.
__global__ void __launch_bounds__(256) qwc_ep_dispatch_kernel(const __half* __restrict__ x, int64_t ldx, int h,
                                                              const int32_t* __restrict__ sorted_tok,
                                                              const int32_t* __restrict__ expert_off, int e_total, int e_local,
                                                              int rotate, int vec, EpPeers peers, int rank, int world,
                                                              int64_t capacity, const uint32_t* epoch_state, uint32_t host_epoch) {
    __shared__ int s_base[kMaxWorld + 1];   // first sorted row of every destination rank
    pdl_enter();
    const uint32_t epoch = ep_epoch(epoch_state, host_epoch);
    if (threadIdx.x <= world) s_base[threadIdx.x] = expert_off[threadIdx.x * e_local];
    __syncthreads();
    // the count tables: CTA 0 writes this rank's row of every destination's table
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i < world * (e_local + 2); i += blockDim.x) {
            const int d = i / (e_local + 2), le = i - d * (e_local + 2);
            int v;
            if (le < e_local) v = expert_off[d * e_local + le + 1] - expert_off[d * e_local + le];
            else if (le == e_local) v = s_base[d];
            else v = s_base[d + 1] - s_base[d];
            peers.counts[d][rank * (e_local + 2) + le] = v;
        }
    }
    const int lane = threadIdx.x & 31, t4 = lane & 3, q8 = lane >> 2;
    const int units = h / 32;
    const int64_t total = static_cast<int64_t>(s_base[world]) * units;
    const int64_t step = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5) * 8;
    for (int64_t base = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 8; base < total; base += step) {
        const int64_t it = base + q8;
        const bool live = it < total;
        const int64_t pr = live ? it / units : 0;
        const int u = live ? static_cast<int>(it % units) : 0;
        const __half* src = x + static_cast<int64_t>(live ? sorted_tok[pr] : 0) * ldx + u * 32 + 8 * t4;
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
        if (live) {
            int d = 0;
            while (d + 1 < world && pr >= s_base[d + 1]) ++d;
            const int64_t i = pr - s_base[d];
            if (i < capacity)
                *reinterpret_cast<uint4*>(peers.recv[d] + (static_cast<int64_t>(rank) * capacity + i) * h + u * 32 + 8 * t4) = raw;
        }
    }
    raise_flags_when_grid_done(peers.flags[rank] + 2 * world, peers, world, rank, epoch);
}

// Regroup on the receiving rank: rows arrive per source rank in that rank's expert-sorted order; the grouped GEMMs want
// each local expert's rows contiguous.  Every CTA rebuilds the (tiny) offset tables from the count tables in shared
// memory; CTA 0 publishes the expert offsets and the tile counts; the tile lists are written expert by expert; the rows
// are copied one warp per row.  ret_src[row] = (source rank, row inside that rank's segment) for the way back.
__global__ void __launch_bounds__(256) qwc_ep_regroup_kernel(const __half* __restrict__ recv, const int32_t* __restrict__ counts, int world,
                                                             int e_local, int h, int64_t capacity, int kTileX, int gu_rows, int dn_rows,
                                                             int gu_paired, int32_t* __restrict__ expert_off_local,
                                                             qwc_moe_tile* __restrict__ tiles_gu, qwc_moe_tile* __restrict__ tiles_dn,
                                                             int32_t* __restrict__ tile_counts, int32_t* __restrict__ ret_src,
                                                             __half* __restrict__ xs, int64_t max_rows, int max_tiles_gu, int max_tiles_dn) {
    __shared__ int s_cnt[kMaxExperts];          // [s][le] rows, then reused as the destination row of (s, le)
    __shared__ int s_seg[kMaxExperts + kMaxWorld];   // [s][le] first row of expert le inside source s's segment, + total per source
    __shared__ int s_off[kMaxExperts + 1];      // local expert offsets
    __shared__ int s_tx[kMaxExperts + 1];       // activation-tile prefix
    __shared__ int s_srcbase[kMaxWorld + 1];    // prefix of the rows received per source
    pdl_enter();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cw = e_local + 2;
    for (int i = tid; i < world * e_local; i += blockDim.x) {
        const int s = i / e_local, le = i - s * e_local;
        int v = counts[s * cw + le];
        v = v < 0 ? 0 : (v > capacity ? static_cast<int>(capacity) : v);   // a stale table (a peer that gave up) must not index out of range
        s_cnt[i] = v;
    }
    __syncthreads();
    // per source: exclusive prefix over the local experts (one warp per source)
    if (warp < world) {
        const int s = warp;
        const int per = (e_local + 31) / 32;
        const int b0 = min(lane * per, e_local), b1 = min(b0 + per, e_local);
        int sum = 0;
        for (int i = b0; i < b1; ++i) sum += s_cnt[s * e_local + i];
        int inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += up;
        }
        int run = inc - sum;
        for (int i = b0; i < b1; ++i) {
            s_seg[s * e_local + i] = run;
            run += s_cnt[s * e_local + i];
        }
        if (lane == 31) s_seg[world * e_local + s] = min(inc, static_cast<int>(capacity));
    }
    __syncthreads();
    // local expert totals, their prefix and the tile prefix (warp 0), then the destination row of every (source, expert)
    if (warp == 0) {
        const int per = (e_local + 31) / 32;
        const int b0 = min(lane * per, e_local), b1 = min(b0 + per, e_local);
        int sc = 0, st = 0;
        for (int i = b0; i < b1; ++i) {
            int c = 0;
            for (int s = 0; s < world; ++s) c += s_cnt[s * e_local + i];
            sc += c;
            st += (c + kTileX - 1) / kTileX;
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
            int c = 0;
            for (int s = 0; s < world; ++s) c += s_cnt[s * e_local + i];
            s_off[i] = rc;
            s_tx[i] = rt;
            rc += c;
            rt += (c + kTileX - 1) / kTileX;
        }
        if (lane == 31) {
            s_off[e_local] = ic;
            s_tx[e_local] = it;
        }
        if (lane == 0) {
            int run = 0;
            for (int s = 0; s < world; ++s) {
                s_srcbase[s] = run;
                run += s_seg[world * e_local + s];
            }
            s_srcbase[world] = run;
        }
    }
    __syncthreads();
    for (int le = tid; le < e_local; le += blockDim.x) {
        int run = s_off[le];
        for (int s = 0; s < world; ++s) {
            const int c = s_cnt[s * e_local + le];
            s_cnt[s * e_local + le] = run;   // from here on: destination row of the first row of (s, le)
            run += c;
        }
    }
    __syncthreads();
    // Count tables that do not add up (a peer gave up and its table is stale) must not drive the kernels that follow
    // out of their buffers: then this rank does nothing for this call (the status word already says why).
    const bool sane = s_off[e_local] <= max_rows && s_srcbase[world] == s_off[e_local] &&
                      s_tx[e_local] * ((gu_rows + kTileW - 1) / kTileW) <= max_tiles_gu &&
                      s_tx[e_local] * ((dn_rows + kTileW - 1) / kTileW) <= max_tiles_dn;
    if (blockIdx.x == 0) {
        for (int i = tid; i <= e_local; i += blockDim.x) expert_off_local[i] = sane ? s_off[i] : 0;
        if (tid == 0) {
            tile_counts[0] = sane ? s_tx[e_local] * ((gu_rows + kTileW - 1) / kTileW) : 0;
            tile_counts[1] = sane ? s_tx[e_local] * ((dn_rows + kTileW - 1) / kTileW) : 0;
            tile_counts[2] = sane ? s_off[e_local] : 0;   // rows received in all
        }
    }
    if (!sane) return;
    // tile lists (weight tiles fastest inside an activation tile), experts dealt over the CTAs
    for (int ex = blockIdx.x; ex < e_local; ex += gridDim.x) {
        const int cnt = s_off[ex + 1] - s_off[ex], ntx = s_tx[ex + 1] - s_tx[ex];
        for (int which = 0; which < 2; ++which) {
            const int rows = which == 0 ? gu_rows : dn_rows;
            qwc_moe_tile* tiles = which == 0 ? tiles_gu : tiles_dn;
            const int ntw = (rows + kTileW - 1) / kTileW;
            const int paired = which == 0 && gu_paired;
            for (int it = tid; it < ntx * ntw; it += blockDim.x) {
                const int mt = it / ntw, j = it - mt * ntw;
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
                tl.x_row0 = s_off[ex] + mt * kTileX;
                tl.x_rows = min(kTileX, cnt - mt * kTileX);
                tl.expert = ex;
                tiles[(s_tx[ex] + mt) * ntw + j] = tl;
            }
        }
    }
    // the rows: one warp per received row
    const int total = s_srcbase[world];
    const int warps = gridDim.x * (blockDim.x >> 5);
    const int chunks = h / 8;   // 16-byte pieces per row
    for (int g = blockIdx.x * (blockDim.x >> 5) + warp; g < total; g += warps) {
        int s = 0;
        while (s + 1 < world && g >= s_srcbase[s + 1]) ++s;
        const int j = g - s_srcbase[s];
        // local expert of row j of source s: the last le with seg[s][le] <= j among the experts that hold rows
        int lo = 0, hi = e_local - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_seg[s * e_local + mid] <= j) lo = mid; else hi = mid - 1;
        }
        const int dst = s_cnt[s * e_local + lo] + (j - s_seg[s * e_local + lo]);
        const uint4* src = reinterpret_cast<const uint4*>(recv + (static_cast<int64_t>(s) * capacity + j) * h);
        uint4* out = reinterpret_cast<uint4*>(xs + static_cast<int64_t>(dst) * h);
        for (int c = lane; c < chunks; c += 32) out[c] = src[c];
        if (lane == 0) {
            ret_src[2 * dst] = s;
            ret_src[2 * dst + 1] = j;
        }
    }
}

// The way back: result row r (local expert order) goes to the rank it came from, at that rank's sorted position.
__global__ void __launch_bounds__(256) qwc_ep_return_kernel(const __half* __restrict__ dn, const int32_t* __restrict__ ret_src,
                                                            const int32_t* __restrict__ total_rows, const int32_t* __restrict__ counts,
                                                            int e_local, int h, int64_t capacity, EpPeers peers, int rank, int world,
                                                            const uint32_t* epoch_state, uint32_t host_epoch) {
    pdl_enter();
    const uint32_t epoch = ep_epoch(epoch_state, host_epoch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = *total_rows;
    const int warps = gridDim.x * (blockDim.x >> 5);
    const int chunks = h / 8;
    const int cw = e_local + 2;
    for (int r = blockIdx.x * (blockDim.x >> 5) + warp; r < total; r += warps) {
        const int s = ret_src[2 * r], j = ret_src[2 * r + 1];
        if (s < 0 || s >= world) continue;
        const int64_t pos = static_cast<int64_t>(counts[s * cw + e_local]) + j;   // position in rank s's sorted order
        if (pos < 0 || pos >= capacity) continue;
        const uint4* src = reinterpret_cast<const uint4*>(dn + static_cast<int64_t>(r) * h);
        uint4* out = reinterpret_cast<uint4*>(peers.ret[s] + pos * h);
        for (int c = lane; c < chunks; c += 32) out[c] = src[c];
    }
    raise_flags_when_grid_done(peers.flags[rank] + 2 * world + 1, peers, world, world + rank, epoch);
}

size_t ep_align(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct EpScratch {
    size_t idx, wts, expert_off, sorted_pair, sorted_tok, inv_perm, tile_counts, expert_off_local, tiles_gu, tiles_dn, ret_src, xs, hs, dn, total;
};

// Rows per activation tile: chosen for the balanced case (every rank receives about as many rows as it sends), while
// the buffers and tile lists are sized for the worst case (every row of every rank lands here).
int64_t ep_tile_rows(int64_t capacity, int64_t e_local) { return qwc_moe_tile_rows(capacity, e_local); }
int64_t ep_max_tiles(int64_t rmax, int64_t capacity, int64_t e_local, int64_t rows_per_expert) {
    return (e_local + rmax / ep_tile_rows(capacity, e_local)) * ((rows_per_expert + kTileW - 1) / kTileW);
}

EpScratch ep_layout(int64_t t, int64_t e_total, int64_t e_local, int64_t k, int64_t h, int64_t inter, int64_t world, int64_t capacity) {
    EpScratch s{};
    const int64_t pairs = t * k, rmax = world * capacity;
    size_t at = 0;
    auto take = [&](size_t bytes) {
        const size_t o = at;
        at = ep_align(at + bytes);
        return o;
    };
    s.idx = take(pairs * 4);
    s.wts = take(pairs * 4);
    s.expert_off = take((e_total + 1) * 4);
    s.sorted_pair = take(pairs * 4);
    s.sorted_tok = take(pairs * 4);
    s.inv_perm = take(pairs * 4);
    s.tile_counts = take(16);
    s.expert_off_local = take((e_local + 1) * 4);
    s.tiles_gu = take(ep_max_tiles(rmax, capacity, e_local, 2 * inter) * sizeof(qwc_moe_tile));
    s.tiles_dn = take(ep_max_tiles(rmax, capacity, e_local, h) * sizeof(qwc_moe_tile));
    s.ret_src = take(rmax * 8);
    s.xs = take(rmax * h * 2);
    s.hs = take(rmax * inter * 2);
    s.dn = take(rmax * h * 2);
    s.total = at;
    return s;
}

int ep_check_ctx(const qwc_hal* hal, const qwc_ep_ctx* ctx, int64_t e_total) {
    if (!hal) return qwc_fail(QWC_ERR_BAD_SHAPE, "hal is null");
    if (!ctx) return qwc_fail(QWC_ERR_BAD_SHAPE, "expert-parallel context is null");
    if (ctx->world < 1 || ctx->world > kMaxWorld || ctx->rank < 0 || ctx->rank >= ctx->world)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "rank %d / world %d: 1..8 ranks", ctx->rank, ctx->world);
    if (e_total <= 0 || e_total > kMaxExperts || e_total % ctx->world != 0)
        return qwc_fail(QWC_ERR_BAD_GEOMETRY, "experts=%lld must be in 1..512 and divide over %d ranks", (long long)e_total, ctx->world);
    if (ctx->capacity_rows <= 0 || ctx->capacity_rows >= (int64_t(1) << 28)) return qwc_fail(QWC_ERR_BAD_SHAPE, "capacity_rows out of range");
    for (int r = 0; r < ctx->world; ++r)
        if (!ctx->recv[r] || !ctx->counts[r] || !ctx->ret[r] || !ctx->flags[r]) return qwc_fail(QWC_ERR_BAD_SHAPE, "peer buffer %d is null", r);
    return QWC_OK;
}

EpPeers ep_peers(const qwc_ep_ctx* ctx) {
    EpPeers p{};
    for (int r = 0; r < ctx->world; ++r) {
        p.recv[r] = static_cast<__half*>(ctx->recv[r]);
        p.counts[r] = static_cast<int32_t*>(ctx->counts[r]);
        p.ret[r] = static_cast<__half*>(ctx->ret[r]);
        p.flags[r] = static_cast<uint32_t*>(ctx->flags[r]);
    }
    return p;
}

uint64_t ep_limit_ns(const qwc_ep_ctx* ctx) {
    return ctx->wait_us > 0 ? static_cast<uint64_t>(ctx->wait_us) * 1000ull : static_cast<uint64_t>(QWC_WAIT_LIMIT_NS);
}

int ep_grid(const qwc_hal* hal, int64_t items, int per_block) {
    int64_t g = (items + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(hal->sm_count) * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

}  // namespace

extern "C" {

size_t qwc_ep_scratch_bytes(const qwc_ep_ctx* ctx, int64_t t, int64_t e_total, int64_t k, int64_t h, int64_t inter) {
    if (!ctx || t < 0 || e_total <= 0 || k <= 0 || h <= 0 || inter <= 0 || ctx->world < 1 || ctx->world > kMaxWorld || e_total % ctx->world) return 0;
    return ep_layout(t, e_total, e_total / ctx->world, k, h, inter, ctx->world, ctx->capacity_rows).total;
}

size_t qwc_ep_recv_bytes(int32_t world, int64_t capacity_rows, int64_t h) { return static_cast<size_t>(world) * capacity_rows * h * 2; }
size_t qwc_ep_ret_bytes(int64_t capacity_rows, int64_t h) { return static_cast<size_t>(capacity_rows) * h * 2; }
size_t qwc_ep_counts_bytes(int32_t world, int64_t e_total) { return static_cast<size_t>(world) * (e_total / (world > 0 ? world : 1) + 2) * 4; }
size_t qwc_ep_flags_bytes(int32_t world) { return static_cast<size_t>(2 * world + 2) * 4; }

int qwc_ep_dispatch(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, int64_t e_total, const void* x_f16, int64_t t,
                    int64_t ldx, int64_t h, int32_t x_is_rotated, const float* logits, int64_t k, int32_t norm_topk,
                    float routed_scale, void* scratch, size_t scratch_bytes, int64_t inter) {
    qwc_clear_error();
    if (int rc = ep_check_ctx(hal, ctx, e_total)) return rc;
    if (k <= 0 || k > 16 || k > e_total) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "top-k=%lld must be in 1..16 and <= experts", (long long)k);
    if (h <= 0 || h % 32 != 0 || inter <= 0 || inter % 32 != 0) return qwc_fail(QWC_ERR_BAD_GEOMETRY, "hidden and inter must be positive multiples of 32");
    if (t < 0 || t * k > ctx->capacity_rows) return qwc_fail(QWC_ERR_BAD_SHAPE, "t * k = %lld rows exceed the context's capacity of %lld", (long long)(t * k), (long long)ctx->capacity_rows);
    if (ldx < h) return qwc_fail(QWC_ERR_BAD_SHAPE, "ldx < hidden");
    if (t > 0 && (!x_f16 || !logits)) return qwc_fail(QWC_ERR_BAD_SHAPE, "null buffer");
    const int64_t e_local = e_total / ctx->world;
    const EpScratch L = ep_layout(t, e_total, e_local, k, h, inter, ctx->world, ctx->capacity_rows);
    if (!scratch || scratch_bytes < L.total || reinterpret_cast<uintptr_t>(scratch) % 256 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "scratch of %zu bytes (256-byte aligned) needed (qwc_ep_scratch_bytes), got %zu", L.total, scratch_bytes);
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    int32_t* idx = reinterpret_cast<int32_t*>(sc + L.idx);
    float* wts = reinterpret_cast<float*>(sc + L.wts);
    int32_t* expert_off = reinterpret_cast<int32_t*>(sc + L.expert_off);
    int32_t* sorted_pair = reinterpret_cast<int32_t*>(sc + L.sorted_pair);
    int32_t* sorted_tok = reinterpret_cast<int32_t*>(sc + L.sorted_tok);
    int32_t* inv_perm = reinterpret_cast<int32_t*>(sc + L.inv_perm);
    int32_t* tile_counts = reinterpret_cast<int32_t*>(sc + L.tile_counts);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (t > 0) {
        if ((rc = qwc_moe_route(hal, stream, logits, t, e_total, k, norm_topk, routed_scale, idx, wts))) return rc;
    }
    // the pair sort also serves t == 0 (all offsets zero): every rank must raise its flags in every call
    if ((rc = qwc_moe_group_pairs(hal, stream, idx, t * k, e_total, k, expert_off, sorted_pair, sorted_tok, inv_perm, 2 * inter, h,
                                  QWC_EPI_NONE, nullptr, nullptr, tile_counts))) return rc;
    const int vec = x_f16 != nullptr && reinterpret_cast<uintptr_t>(x_f16) % 16 == 0 && ldx % 8 == 0;
    const int grid = ep_grid(hal, t * k * (h / 32), 64);
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_ep_dispatch_kernel, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(x_f16), ldx,
                                static_cast<int>(h), static_cast<const int32_t*>(sorted_tok), static_cast<const int32_t*>(expert_off),
                                static_cast<int>(e_total), static_cast<int>(e_local), static_cast<int>(!x_is_rotated), vec, ep_peers(ctx),
                                ctx->rank, ctx->world, ctx->capacity_rows, static_cast<const uint32_t*>(ctx->epoch_state), ctx->epoch));
    return QWC_OK;
}

int qwc_ep_experts(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, const qwc_weight_view* bank_gu_local,
                   const qwc_weight_view* bank_dn_local, int64_t e_total, int64_t inter, int64_t t, int64_t k, void* scratch,
                   size_t scratch_bytes) {
    qwc_clear_error();
    if (int rc = ep_check_ctx(hal, ctx, e_total)) return rc;
    if (!bank_gu_local || !bank_dn_local) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "expert banks are null");
    if (int rc = qwc_check_view(bank_gu_local)) return rc;
    if (int rc = qwc_check_view(bank_dn_local)) return rc;
    const int64_t e_local = e_total / ctx->world, h = bank_gu_local->k;
    if (bank_gu_local->n != e_local * 2 * inter) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "local gate/up bank has %lld rows, expected %lld", (long long)bank_gu_local->n, (long long)(e_local * 2 * inter));
    if (bank_dn_local->n != e_local * h || bank_dn_local->k != inter) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "local down bank must be [%lld, %lld]", (long long)(e_local * h), (long long)inter);
    if (inter % 64 != 0 || h % 32 != 0)
        return qwc_fail(QWC_ERR_BLOCKED, "the expert-parallel chain needs inter %% 64 == 0 (SwiGLU fused into the gate/up GEMM) and hidden %% 32 == 0");
    if (!qwc_gemm_tc_supported(hal, bank_gu_local, 17, QWC_EPI_NONE) || !qwc_gemm_tc_supported(hal, bank_dn_local, 17, QWC_EPI_NONE))
        return qwc_fail(QWC_ERR_BLOCKED, "the grouped expert GEMMs need HQ4_G32_M5 / HQ8_G32 banks with k %% 128 == 0 or HQ4_G64 banks with k %% 256 == 0, 16-byte aligned");
    const EpScratch L = ep_layout(t, e_total, e_local, k, h, inter, ctx->world, ctx->capacity_rows);
    if (!scratch || scratch_bytes < L.total || reinterpret_cast<uintptr_t>(scratch) % 256 != 0)
        return qwc_fail(QWC_ERR_BAD_SHAPE, "scratch of %zu bytes (256-byte aligned) needed (qwc_ep_scratch_bytes), got %zu", L.total, scratch_bytes);
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    int32_t* tile_counts = reinterpret_cast<int32_t*>(sc + L.tile_counts);
    int32_t* expert_off_local = reinterpret_cast<int32_t*>(sc + L.expert_off_local);
    qwc_moe_tile* tiles_gu = reinterpret_cast<qwc_moe_tile*>(sc + L.tiles_gu);
    qwc_moe_tile* tiles_dn = reinterpret_cast<qwc_moe_tile*>(sc + L.tiles_dn);
    int32_t* ret_src = reinterpret_cast<int32_t*>(sc + L.ret_src);
    __half* xs = reinterpret_cast<__half*>(sc + L.xs);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t rmax = static_cast<int64_t>(ctx->world) * ctx->capacity_rows;
    const int32_t gu_epi = QWC_EPI_SILU_PAIR_FWHT;
    const int xrows = static_cast<int>(ep_tile_rows(ctx->capacity_rows, e_local));
    const int64_t max_gu = ep_max_tiles(rmax, ctx->capacity_rows, e_local, 2 * inter), max_dn = ep_max_tiles(rmax, ctx->capacity_rows, e_local, h);
    const EpPeers peers = ep_peers(ctx);
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_ep_wait_kernel, dim3(1), dim3(32), 0, st, static_cast<const uint32_t*>(peers.flags[ctx->rank]), 0, ctx->world,
                                static_cast<uint32_t*>(ctx->epoch_state), ctx->epoch, 0, ep_limit_ns(ctx), hal->status));
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_ep_regroup_kernel, dim3(ep_grid(hal, rmax, 8)), dim3(256), 0, st,
                                static_cast<const __half*>(peers.recv[ctx->rank]), static_cast<const int32_t*>(peers.counts[ctx->rank]), ctx->world,
                                static_cast<int>(e_local), static_cast<int>(h), ctx->capacity_rows, xrows, static_cast<int>(2 * inter),
                                static_cast<int>(h), 1, expert_off_local, tiles_gu, tiles_dn, tile_counts, ret_src, xs, rmax,
                                static_cast<int>(max_gu), static_cast<int>(max_dn)));
    int rc;
    if ((rc = qwc_launch_gemm_tc_grouped(hal, st, bank_gu_local, xs, rmax, tiles_gu, tile_counts, max_gu, sc + L.hs, QWC_F16, inter, xrows, gu_epi))) return rc;
    if ((rc = qwc_launch_gemm_tc_grouped(hal, st, bank_dn_local, sc + L.hs, rmax, tiles_dn, tile_counts + 1, max_dn, sc + L.dn, QWC_F16, h, xrows, QWC_EPI_NONE))) return rc;
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_ep_return_kernel, dim3(ep_grid(hal, rmax, 8)), dim3(256), 0, st, reinterpret_cast<const __half*>(sc + L.dn),
                                static_cast<const int32_t*>(ret_src), static_cast<const int32_t*>(tile_counts + 2),
                                static_cast<const int32_t*>(peers.counts[ctx->rank]), static_cast<int>(e_local), static_cast<int>(h),
                                ctx->capacity_rows, peers, ctx->rank, ctx->world, static_cast<const uint32_t*>(ctx->epoch_state), ctx->epoch));
    return QWC_OK;
}

int qwc_ep_combine(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, int64_t e_total, int64_t inter, int64_t t, int64_t k,
                   int64_t h, void* out, int32_t out_dtype, void* scratch, size_t scratch_bytes) {
    qwc_clear_error();
    if (int rc = ep_check_ctx(hal, ctx, e_total)) return rc;
    if (out_dtype != QWC_F16 && out_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "out dtype must be f16 or f32");
    if (t > 0 && !out) return qwc_fail(QWC_ERR_BAD_SHAPE, "out is null");
    const int64_t e_local = e_total / ctx->world;
    const EpScratch L = ep_layout(t, e_total, e_local, k, h, inter, ctx->world, ctx->capacity_rows);
    if (!scratch || scratch_bytes < L.total) return qwc_fail(QWC_ERR_BAD_SHAPE, "scratch too small");
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    const EpPeers peers = ep_peers(ctx);
    QWC_CUDA_TRY(qwc_launch_pdl(qwc_ep_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                                static_cast<const uint32_t*>(peers.flags[ctx->rank]), ctx->world, ctx->world,
                                static_cast<uint32_t*>(ctx->epoch_state), ctx->epoch, 1, ep_limit_ns(ctx), hal->status));
    if (t == 0) return QWC_OK;
    return qwc_moe_combine(hal, stream, peers.ret[ctx->rank], QWC_F16, reinterpret_cast<const int32_t*>(sc + L.inv_perm),
                           reinterpret_cast<const float*>(sc + L.wts), t, k, h, out, out_dtype);
}

int qwc_ep_moe(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, const qwc_weight_view* bank_gu_local,
               const qwc_weight_view* bank_dn_local, int64_t e_total, int64_t inter, const void* x_f16, int64_t t, int64_t ldx,
               int32_t x_is_rotated, const float* logits, int64_t k, int32_t norm_topk, float routed_scale, void* out,
               int32_t out_dtype, void* scratch, size_t scratch_bytes) {
    if (!bank_gu_local) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "expert banks are null");
    const int64_t h = bank_gu_local->k;
    // the checks of the later phases come first, so that nothing has been launched when one of them refuses
    if (int rc = ep_check_ctx(hal, ctx, e_total)) return rc;
    if (!bank_dn_local) return qwc_fail(QWC_ERR_BAD_WEIGHTS, "expert banks are null");
    if (int rc = qwc_check_view(bank_gu_local)) return rc;
    if (int rc = qwc_check_view(bank_dn_local)) return rc;
    if (inter % 64 != 0) return qwc_fail(QWC_ERR_BLOCKED, "the expert-parallel chain needs inter %% 64 == 0 (fused SwiGLU epilogue)");
    if (!qwc_gemm_tc_supported(hal, bank_gu_local, 17, QWC_EPI_NONE) || !qwc_gemm_tc_supported(hal, bank_dn_local, 17, QWC_EPI_NONE))
        return qwc_fail(QWC_ERR_BLOCKED, "the grouped expert GEMMs need HQ4_G32_M5 / HQ8_G32 banks with k %% 128 == 0 or HQ4_G64 banks with k %% 256 == 0, 16-byte aligned");
    const int64_t e_local = e_total / ctx->world;
    if (bank_gu_local->n != e_local * 2 * inter || bank_dn_local->n != e_local * h || bank_dn_local->k != inter)
        return qwc_fail(QWC_ERR_BAD_WEIGHTS, "local expert banks do not match experts / world, hidden and inter");
    if (out_dtype != QWC_F16 && out_dtype != QWC_F32) return qwc_fail(QWC_ERR_BAD_SHAPE, "out dtype must be f16 or f32");
    if (t > 0 && !out) return qwc_fail(QWC_ERR_BAD_SHAPE, "out is null");
    int rc;
    if ((rc = qwc_ep_dispatch(hal, stream, ctx, e_total, x_f16, t, ldx, h, x_is_rotated, logits, k, norm_topk, routed_scale, scratch,
                              scratch_bytes, inter))) return rc;
    if ((rc = qwc_ep_experts(hal, stream, ctx, bank_gu_local, bank_dn_local, e_total, inter, t, k, scratch, scratch_bytes))) return rc;
    return qwc_ep_combine(hal, stream, ctx, e_total, inter, t, k, h, out, out_dtype, scratch, scratch_bytes);
}

}  // extern "C"
