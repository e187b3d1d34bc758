/*
 * qwc.h -- C ABI of the B200 (sm_100a) quantized-matmul library, libqwcuda.so.
 *
 * Every entry point is the CUDA twin of one "door" of the reference's Swift
 * operator layer (Sources/Operators/QWGEMM).  The reference encodes kernels
 * into an MTLComputeCommandEncoder and addresses memory through
 * QWTensorValue / QWWeightView; here an encoder becomes a CUDA stream and a
 * tensor value becomes a raw device pointer plus extents.  Rules carried over
 * from the reference ("Encode path allocates nothing",
 * Sources/Operators/QWGEMM/QWGemm.swift:216-217):
 *
 *   - the caller owns every buffer, scratch included;
 *   - no encode-class call allocates, synchronises or copies host<->device;
 *   - every refusal happens before the first launch and leaves the stream
 *     untouched (the orchestrating doors check, up front, everything the
 *     doors they call would check); the status code mirrors QWGemmError
 *     (Sources/Operators/QWGEMM/QWGemm.swift:66-80) and qwc_last_error()
 *     returns the message (thread-local).
 *
 * Paths in comments are paths inside the reference project.
 */
#ifndef QWC_H
#define QWC_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qwc_hal qwc_hal; /* device context: replaces QWHal (Sources/Foundation/QWHAL/QWHal.swift:81-235) */
typedef void* qwc_stream;       /* a cudaStream_t; replaces the MTLComputeCommandEncoder argument */

/* QWGemmError cases (QWGemm.swift:66-80) plus a CUDA runtime failure. */
enum {
    QWC_OK = 0,
    QWC_ERR_BLOCKED = 1,      /* .f3Blocked: the plan has no kernel for this shape */
    QWC_ERR_BAD_WEIGHTS = 2,  /* .badWeights */
    QWC_ERR_BAD_SHAPE = 3,    /* .badShape */
    QWC_ERR_BAD_GEOMETRY = 4, /* .badGeometry */
    QWC_ERR_CUDA = 5
};

/* QWWeightView.ContainerKind (Sources/Foundation/QWAlloc/QWWeightView.swift:11-31). */
enum {
    QWC_KIND_HQ4_G32_M5 = 0, /* .incumbentHQ4G32: 20-byte block, interleaved nibbles, +1024 decode */
    QWC_KIND_ROTATED_HQ = 1  /* .rotatedHQ(bits, group): f16 scale, f16 bias, linear bit stream */
};

/* QWDType subset used by this path (Sources/Foundation/QWCore/QWDType.swift:5-23). */
enum { QWC_F16 = 0, QWC_F32 = 1, QWC_BF16 = 2 /* raw router planes only */ };

/* QWEpilogue (QWGemm.swift:19-22) plus the fused-FWHT mode bit of
 * qwg_gemv_q4g_silu_pair_dx_h16 (Sources/QWMetal/gemm/qwgemm.metal:204-379). */
enum { QWC_EPI_NONE = 0, QWC_EPI_SILU_PAIR = 1, QWC_EPI_SILU_PAIR_FWHT = 2 };

/* QWGemmFamily (QWGemm.swift:11-17). */
enum { QWC_FAMILY_F1_DECODE_GEMV = 1, QWC_FAMILY_F2_LMHEAD_GEMV = 2, QWC_FAMILY_F3_PREFILL_GEMM = 3,
       QWC_FAMILY_F4_BLOCKED_GEMM = 4, QWC_FAMILY_F5_SKINNY_GEMM = 5 };

/* Which kernel a plan selects. */
enum { QWC_BACKEND_BLOCKED = 0, QWC_BACKEND_STREAM_MMA = 1, QWC_BACKEND_TCGEN05 = 2, QWC_BACKEND_ROWWISE = 3 };

/* QWWeightView (QWWeightView.swift:9-152): one weight bank, row-major [n][k/group] blocks. */
typedef struct {
    const void* blocks; /* device pointer to the first block */
    int64_t n, k;
    int32_t kind, bits, group;
} qwc_weight_view;

/* QWGemmPlan (QWGemm.swift:35-64). */
typedef struct {
    int32_t family, backend, epilogue, threads_per_cta;
    char kernel[48];
} qwc_plan;

/* ---- context -------------------------------------------------------------- */
/* QWHal.init (QWHal.swift:81-145).  Allocates a small device status word; the only allocation in the library. */
int qwc_hal_create(int device, qwc_hal** out);
void qwc_hal_destroy(qwc_hal* hal);
const char* qwc_last_error(void);
/* Synchronises the device and returns the kernels' status word: 0, or the code of the first bounded wait that
 * gave up (the CUDA stand-in for MTLCommandBuffer.error, Sources/Runtime/QWEngine/Driver/DriverDecode.swift:142-158). */
int qwc_hal_device_status(qwc_hal* hal, int32_t* status_out);
int qwc_sm_count(const qwc_hal* hal);
/* The reference loads its weight planes once and never writes them again (Sources/Foundation/QWLoad/PlaneIO.swift:64-198;
 * the decode loop only reads QWWeightView banks).  A caller that keeps that discipline can say so: with enabled != 0
 * the decode / verify kernels are launched with programmatic stream serialization and start streaming their packed
 * weights while the previous kernel of the stream is still finishing; activations, outputs and scratch are still
 * touched only after the previous work has completed.  Leave it off (the default) if a weight bank may still be
 * written by work in flight on the same stream when a matmul door is called (e.g. quantize-then-multiply). */
int qwc_hal_set_static_weights(qwc_hal* hal, int32_t enabled);

/* ---- weights -------------------------------------------------------------- */
/* QWWeightView.init? (QWWeightView.swift:108-152): fills *view or refuses (k % group, bank too short, unknown kind). */
int qwc_weight_view_init(qwc_weight_view* view, const void* blocks, size_t bank_bytes, int64_t n, int64_t k,
                         int32_t kind, int32_t bits, int32_t group);
int64_t qwc_block_bytes(int32_t kind, int32_t bits, int32_t group);

/* ---- dispatch table ------------------------------------------------------- */
/* QWGemm.plan (QWGemm.swift:92-133): pure function of the shape. */
int qwc_gemm_plan(int64_t m, int64_t n, int64_t k, int32_t kind, int32_t bits, int32_t group, int32_t epilogue,
                  int64_t vocab, qwc_plan* out);

/* ---- kernels -------------------------------------------------------------- */
/* QWGemm.encodeFwht32 (QWGemm.swift:285-300): in-place f16 Walsh-Hadamard per aligned 32 block; count % 32 == 0. */
int qwc_fwht32_f16(qwc_hal* hal, qwc_stream stream, void* x_f16, int64_t count);

/* RMSNorm with rotated f16 output, the step before every quantized matmul in the reference's engine (qwg_rmsnorm /
 * qwg_rmsnorm_residual, Sources/QWMetal/mlp_norm_rope/qwnorm.metal:27-79, 249-259; encodeRMSNormFast /
 * encodeRMSNormResidualFast, Sources/Runtime/QWEngine/Driver/EncodeKernels.swift:339-404):
 *   s = x, or s = f16(x + residual) written back to residual when residual != NULL;
 *   y = f16(fwht32(s * rsqrt(mean(s^2) + eps) * (1 + gamma)))   (rotate == 0 leaves out the rotation).
 * x, y, residual f16 [rows, hidden] dense; gamma f16 [hidden] stored raw (the +1 is applied here); hidden % 256 == 0.
 * Feed y to qwc_gemm with x_is_rotated = 1. */
int qwc_rmsnorm_fwht(qwc_hal* hal, qwc_stream stream, const void* x_f16, const void* gamma_f16, void* y_f16,
                     void* residual_f16, int64_t rows, int64_t hidden, float eps, int32_t rotate);

/* QWGemm.encodeCast (QWGemm.swift:302-320): the f32 -> f16 cast seam after an f32-emitting GEMV; count % 8 == 0. */
int qwc_cast_f32_to_f16(qwc_hal* hal, qwc_stream stream, const float* x_f32, void* y_f16, int64_t count);

/* Greedy head: tokens[r] = argmax_c logits[r, c] in the reference's key order (value, then lower column; NaN lowest, +0
 * above -0) — the pair encodeHQ4F32V4Argmax + encodeArgmaxFin (Sources/Operators/QWGEMM/QWGemmF32.swift:201-307; kernels
 * Sources/QWMetal/include/qw_gemm_f32_common.metalh:31-57, Sources/QWMetal/head_sampling/qwhead.metal:241-270) after the
 * LM-head GEMV: call qwc_gemm with f32 logits [rows, n], then this.  logits f32, row stride ld; tokens i32 [rows]. */
int qwc_head_argmax(qwc_hal* hal, qwc_stream stream, const float* logits, int64_t ld, int64_t rows, int64_t n,
                    int32_t* tokens);

/* Host decode twin Pack.dequantHQ4Slab / dequantHQBlockSlab (Sources/Foundation/QWQuant/QWPack.swift:205-321),
 * on the device: blocks -> [n, k] values, bit-exact with the reference decode.  standard_domain != 0 applies the
 * inverse rotation (FWHT-32).  out_dtype QWC_F32, or QWC_F16 (one extra rounding). */
int qwc_dequant(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, void* out, int32_t out_dtype,
                int32_t standard_domain);

/* Load-time quantizer: HQ4Quantizer / qwg_quantize_bf16_to_hq4_g32_m5 (Sources/Foundation/QWLoad,
 * Sources/QWMetal/quant/qw_online_quant.metal:17-55) and the Python packers it mirrors
 * (Scripts/quantize/hq4.py:54-123, hq_blocks.py:436-517).  w: f32 [n, k] row-major on the device; blocks_out
 * receives n * (k/group) blocks whose bytes equal the Python packer's.  A non-finite weight sets the device
 * status word (the Python packer raises). */
int qwc_quantize(qwc_hal* hal, qwc_stream stream, const float* w_f32, int64_t n, int64_t k, int32_t kind, int32_t bits,
                 int32_t group, void* blocks_out);

/* The single matmul door: QWGemm.encode / encodeH16 (QWGemm.swift:135-283), QWGemmAQ.encode / encodeDecodeT4
 * (Sources/Operators/QWGEMM/QWGemmAQ.swift:192-304), the batched verify doors
 * (Sources/Runtime/QWEngine/SpeculativeMTP/QWMTPBatchedMLP.swift:92-288) and the prefill doors
 * QWGemm.encodeNaxF32 / encodeDenseProjF32 (Sources/Operators/QWGEMM/QWGemmF32.swift:366-441).
 *   y[m, n_out] = epilogue( rot(x)[m, k] . W_rot[n, k]^T ),  f32 accumulate.
 * x: f16 [m, k] rows ldx apart.  x_is_rotated == 0: x is in the standard basis and is rotated inside the call
 * (FWHT-32 along k, rounded once to f16); != 0: x already is (the reference's dataflow).
 * epilogue NONE: n_out = n.  SILU_PAIR: rows [0, n/2) are gate, [n/2, n) up; n_out = n/2,
 * y = silu(gate) * up.  SILU_PAIR_FWHT: same, then FWHT-32 along n_out (n_out % 32 == 0).
 * y: f16 or f32 [m, n_out] rows ldy apart.  workspace may be NULL when qwc_gemm_workspace_bytes() is 0.  The workspace holds
 * what the chosen kernel needs: the rotated (or, below 16 tokens, copied) activations of the tensor-core kernel, which takes
 * calls of 9 tokens and more (8 for HQ8_G32), or the K-slice sums of the streaming kernel; 16-byte aligned.  Numeric class of
 * every door: f16 weights (decoded exactly as the reference decodes them) x f16 activations, f32 accumulate. */
int qwc_gemm(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const void* x_f16, int64_t m, int64_t ldx,
             void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated, void* workspace,
             size_t workspace_bytes);
size_t qwc_gemm_workspace_bytes(const qwc_hal* hal, const qwc_weight_view* w, int64_t m, int32_t epilogue,
                                int32_t x_is_rotated);

/* The f32-activation matmul door: QWGemmF32.encodeHQ4F32V4 / encodeHQ4F32BM (Sources/Operators/QWGEMM/QWGemmF32.swift:
 * 143-199, 309-350; bodies Sources/QWMetal/include/qw_gemm_f32_common.metalh:59-225) with the f32 rotation
 * encodeH32F32 (QWGemmF32.swift:46-54) folded in when x_is_rotated == 0.
 *   y[m, n] = epi( x_rot[m, k] . W_rot[n, k]^T ),  x f32 rows ldx apart, rounded once to f16 after the (f32) rotation.
 * epilogue, the reference's codes (qw_gemm_f32_common.metalh:15-20, 131-133): 0 none, 1 silu(y / scale), 2 sigmoid(y),
 * 3 silu(y / scale) then FWHT-32 along n (n % 32 == 0).  y: f16 or f32 [m, n] rows ldy apart.  workspace: 256-byte
 * aligned, qwc_gemm_f32_workspace_bytes() bytes.  Activations beyond the f16 range (|x_rot| > 65504) become infinite. */
int qwc_gemm_f32(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const float* x_f32, int64_t m, int64_t ldx,
                 void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, float scale, int32_t x_is_rotated,
                 void* workspace, size_t workspace_bytes);
size_t qwc_gemm_f32_workspace_bytes(const qwc_hal* hal, const qwc_weight_view* w, int64_t m, int32_t epilogue);

/* No counterpart in the reference.  The small-M matmul door (m <= 16, same arguments and results as qwc_gemm) for
 * callers that cannot allocate device memory where they call it -- an operator inside an engine whose arena was
 * frozen at load time, a thread that must not risk the device-wide synchronisation of cudaMalloc, a host running
 * under a memory budget already handed out.  When the call needs scratch (9..16 tokens with K processed in slices)
 * it comes from a fixed 2 MiB array inside the library's device image, held by every GPU that loads the library.
 * Needs beyond qwc_static_scratch_capacity() are refused (QWC_ERR_BAD_SHAPE).  The first call on a device looks up
 * the array's device address: make it before any stream capture, with that device current.  All calls share the
 * array, so calls that could overlap on the GPU must be ordered by the caller.  Never allocates. */
int qwc_gemm_static_scratch(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w, const void* x_f16, int64_t m,
                            int64_t ldx, void* y, int32_t y_dtype, int64_t ldy, int32_t epilogue, int32_t x_is_rotated);
size_t qwc_static_scratch_capacity(void);

/* ---- peer-visible device memory (load time) ----------------------------------------------------------------------
 * (No counterpart in the reference.)  The fused collectives below store into the other ranks' buffers directly; one
 * process drives one GPU.  qwc_peer_alloc: a zeroed device buffer of this rank and its 64-byte handle, which the host
 * hands to the peers by its own channel; qwc_peer_open: maps a peer's buffer from its handle (peer access is enabled on
 * first use).  These calls allocate and synchronise: make them once, before the first encode call. */
int qwc_peer_alloc(qwc_hal* hal, size_t bytes, void** ptr_out, void* handle_out_64);
int qwc_peer_open(qwc_hal* hal, const void* handle_64, void** ptr_out);
int qwc_peer_close(qwc_hal* hal, void* ptr);
int qwc_peer_free(qwc_hal* hal, void* ptr);

/* ---- tensor parallel: row-parallel matmul fused with its all-reduce ---------------------------------------------
 * (No counterpart in the reference, which runs on one device; the format decides the design: a K shard of the bank per
 * rank, f32 partial sums, one sum over the ranks.)  One kernel does both: every CTA stores its partial sums straight
 * into the inbox of every rank (ordinary peer stores over NVLink), each as ONE 8-byte store of (value, call number), and
 * then reads the world slots of its own rows from its own inbox, waiting (bounded) until each carries this call's number,
 * and sums them in rank order, so every rank ends with the same bits.  No fences and no flags: a slot that carries the
 * call's number holds the call's value.  The caller provides peer-mapped memory (qwc_peer_alloc / qwc_peer_open):
 *   inbox[r]: rank r's inbox, [world][m][n] slots of 8 bytes (f32 value, u32 call number), zero before the first call.
 *   Two inbox buffers are used in turn, so that a fast rank's next call does not overwrite a slot a slow rank has not
 *   read yet.  Either the host counts: epoch = a non-zero value that differs from the previous two calls' and inbox[r]
 *   points at the buffer of THIS call (epoch_state = NULL); or the device counts: epoch_state points at two zero-initialised
 *   u32 words in this rank's memory, inbox[r] points at the FIRST of two buffers inbox_floats apart, and the kernel takes
 *   call number *epoch_state + 1, picks the buffer by its parity and stores the new number when it is done -- the form to
 *   use when calls are captured in a CUDA graph and replayed, where host values would repeat.
 *   Every rank of the group must make the same calls (same shapes, same order). */
typedef struct {
    int32_t rank, world;      /* 2 <= world <= 8 */
    uint32_t epoch;
    int32_t reserved;         /* > 0: limit of the wait for the peers' values in microseconds (0: the library's default, 1 s) */
    void* inbox[8];           /* 8-byte aligned */
    void* flags[8];           /* not used (kept for the layout of earlier callers) */
    int64_t inbox_floats;     /* capacity of one inbox buffer in floats: even, >= 2 * world * m * n */
    int64_t flag_words;       /* not used */
    void* epoch_state;        /* NULL, or this rank's device-side call counter (two u32 words, zero before the first call) */
} qwc_allreduce_ctx;

/* y[m, n] = sum over ranks of rot(x_local[m, k_local]) . W_local^T (no epilogue), m <= 8 (decode / verify), banks with
 * 16-byte rows.  Returns QWC_ERR_BLOCKED for shapes this form does not take (use qwc_gemm + an all-reduce then). */
int qwc_gemm_allreduce(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* w_local, const void* x_f16, int64_t m,
                       int64_t ldx, void* y, int32_t y_dtype, int64_t ldy, int32_t x_is_rotated,
                       const qwc_allreduce_ctx* ctx);

/* ---- expert parallel: the MoE block with its token exchange over peer memory ------------------------------------
 * (No counterpart in the reference, which runs on one device.  The exchange sits where the reference's own stages sit:
 * the pair sort, Sources/QWMetal/gemm/qwgemm_moe_group_f32.metal:10-148, and the weighted combine,
 * Sources/QWMetal/gemm/qwgemm_moe_nax_f16.metal:7-126; chain: QWMoEOperator.encodeResident,
 * Sources/Operators/QWGEMM/QWMoEOperator.swift:246-362.)  Experts [r * E / R, (r + 1) * E / R) live on rank r; every
 * rank routes its own t tokens.  dispatch: route, pair sort, and one kernel that rotates every sorted row and stores it
 * into the receive buffer of the rank that owns its expert (plain peer stores), then raises this rank's flag on every
 * peer.  experts: waits (bounded) for every peer's flag, regroups the received rows by local expert, runs the two grouped
 * expert GEMMs (SwiGLU + FWHT fused; inter % 64 == 0) and stores every result row into the return buffer of the rank it
 * came from; raises the return flags.  combine: waits (bounded) for the return flags, then the weighted combine.  No host
 * synchronisation, no NCCL.  The caller provides peer-mapped memory, zero before the first call:
 *   recv[r]   rank r's receive buffer, f16 [world][capacity_rows][hidden]      (qwc_ep_recv_bytes)
 *   counts[r] rank r's count tables, i32 [world][experts / world + 2]          (qwc_ep_counts_bytes)
 *   ret[r]    rank r's return buffer, f16 [capacity_rows][hidden]              (qwc_ep_ret_bytes)
 *   flags[r]  rank r's flags, u32 [2 * world + 2]                              (qwc_ep_flags_bytes)
 * capacity_rows >= the largest t * k of any rank.  Every rank must make the same calls in the same order (t may differ
 * per rank, also 0).  The call number is epoch (host counted, must differ from the previous call's) or, with epoch_state
 * != NULL (one zero-initialised u32 in this rank's memory), *epoch_state + 1, stored back by the combine phase: the form
 * for calls captured in a CUDA graph.  A wait that runs out (wait_us, default 1 s) sets status 105; the rank then
 * finishes the call without touching memory outside its buffers.  With fewer GPUs than ranks the three phases can be
 * called rank after rank on one device, each rank with its own buffers: every wait then finds its flags raised. */
typedef struct {
    int32_t rank, world;      /* 1 <= world <= 8 */
    uint32_t epoch;
    int32_t wait_us;
    int64_t capacity_rows;
    void* recv[8];
    void* counts[8];
    void* ret[8];
    void* flags[8];
    void* epoch_state;
} qwc_ep_ctx;

size_t qwc_ep_recv_bytes(int32_t world, int64_t capacity_rows, int64_t h);
size_t qwc_ep_ret_bytes(int64_t capacity_rows, int64_t h);
size_t qwc_ep_counts_bytes(int32_t world, int64_t e_total);
size_t qwc_ep_flags_bytes(int32_t world);
size_t qwc_ep_scratch_bytes(const qwc_ep_ctx* ctx, int64_t t, int64_t e_total, int64_t k, int64_t h, int64_t inter);
int qwc_ep_dispatch(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, int64_t e_total, const void* x_f16, int64_t t,
                    int64_t ldx, int64_t h, int32_t x_is_rotated, const float* logits, int64_t k, int32_t norm_topk,
                    float routed_scale, void* scratch, size_t scratch_bytes, int64_t inter);
int qwc_ep_experts(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, const qwc_weight_view* bank_gu_local,
                   const qwc_weight_view* bank_dn_local, int64_t e_total, int64_t inter, int64_t t, int64_t k, void* scratch,
                   size_t scratch_bytes);
int qwc_ep_combine(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, int64_t e_total, int64_t inter, int64_t t, int64_t k,
                   int64_t h, void* out, int32_t out_dtype, void* scratch, size_t scratch_bytes);
/* The three phases in one call (what a rank of a real group makes). */
int qwc_ep_moe(qwc_hal* hal, qwc_stream stream, const qwc_ep_ctx* ctx, const qwc_weight_view* bank_gu_local,
               const qwc_weight_view* bank_dn_local, int64_t e_total, int64_t inter, const void* x_f16, int64_t t, int64_t ldx,
               int32_t x_is_rotated, const float* logits, int64_t k, int32_t norm_topk, float routed_scale, void* out,
               int32_t out_dtype, void* scratch, size_t scratch_bytes);

/* ---- mixture of experts ---------------------------------------------------------------------------------------
 * The operator chain of QWMoEOperator.encodeResident (Sources/Operators/QWGEMM/QWMoEOperator.swift:206-442), grouped
 * path: route -> pair sort + tile plan -> gather -> grouped gate/up GEMM -> SwiGLU + FWHT -> grouped down GEMM ->
 * weighted combine.  All scratch is caller-allocated (QWMoEOperator.Scratch, :131-192). */

/* One tile of a grouped expert GEMM (the tile list of Sources/QWMetal/gemm/qwgemm_moe_group_f32.metal:82-115,
 * with 128 expert weight rows x up to qwc_moe_tile_rows() expert-sorted activation rows per tile). */
typedef struct {
    int32_t w_row0; /* first weight row of the tile in the stacked expert bank */
    int32_t w_rows; /* valid weight rows (<= 128) */
    int32_t x_row0; /* first expert-sorted activation row */
    int32_t x_rows; /* valid activation rows (<= 256) */
    int32_t y_col0; /* output column of the tile's first weight row */
    int32_t expert;
    int32_t pad0;   /* paired tiles (pad1 != 0): first up row; rows w_row0.. are 64 gate rows, rows pad0.. the 64 up rows */
    int32_t pad1;   /* 1 for a paired gate/up tile feeding a SwiGLU epilogue, else 0 */
} qwc_moe_tile;

/* QWGemm.encodeFnRouterGemm (Sources/Operators/QWGEMM/QWGemmMoERouter.swift:78-125; kernel qwg_router_gemm,
 * Sources/QWMetal/subsystems/qwrouter.metal:460-520): logits f32 [t, e] = x [t, h] . w [e, h]^T with f32 accumulate.  x:
 * the plain (un-rotated) hidden states, f16 or f32, row stride ldx; w: the raw router plane, bf16 / f16 / f32 (never
 * rotated or quantized, Scripts/quantize/pack.py:332).  h % 32 == 0. */
int qwc_moe_router_gemm(qwc_hal* hal, qwc_stream stream, const void* x, int32_t x_dtype, int64_t ldx, int64_t t, int64_t h,
                        const void* w, int32_t w_dtype, int64_t e, float* logits);

/* QWGemm.encodeFnMoeRoute (Sources/Operators/QWGEMM/QWGemmMoERouter.swift:78-113; kernel qwg_moe_route,
 * Sources/QWMetal/subsystems/qwrouter.metal:84-168): f32 softmax over all experts, top-k by repeated argmax (ties to
 * the lower id, non-finite logits never chosen, idx = -1 when none is left), optional renormalisation over the k
 * chosen, times routed_scale (<= 0 means 1).  logits f32 [t, e]; idx i32 [t, k]; wts f32 [t, k].  e <= 512, k <= 16. */
int qwc_moe_route(qwc_hal* hal, qwc_stream stream, const float* logits, int64_t t, int64_t e, int64_t k, int32_t norm_topk,
                  float routed_scale, int32_t* idx, float* wts);

/* QWGemm.encodeMoEGroupPairsF32 (Sources/Operators/QWGEMM/QWGemmMoE.swift:24-99; kernel qwg_moe_group_pairs_f32):
 * counting sort of the t*k (token, route) pairs by expert, slot order inside an expert = ascending pair index.
 * expert_off i32 [e + 1]; sorted_pair, sorted_tok, inv_perm i32 [pairs] (inv_perm = -1 for dropped pairs).  Also
 * writes the tile lists of the two grouped GEMMs (gate/up with gu_rows = 2 * inter rows per expert, down with dn_rows
 * = hidden rows per expert): tiles_gu / tiles_dn hold up to qwc_moe_max_tiles() entries, tile_counts i32 [2].
 * gu_epilogue: QWC_EPI_NONE lists plain 128-row gate/up tiles; a SwiGLU epilogue (the one the gate/up grouped GEMM will
 * be called with; needs inter % 64 == 0) lists tiles of 64 gate rows + their 64 up rows. */
int qwc_moe_group_pairs(qwc_hal* hal, qwc_stream stream, const int32_t* idx, int64_t pairs, int64_t e, int64_t k,
                        int32_t* expert_off, int32_t* sorted_pair, int32_t* sorted_tok, int32_t* inv_perm,
                        int64_t gu_rows, int64_t dn_rows, int32_t gu_epilogue, qwc_moe_tile* tiles_gu, qwc_moe_tile* tiles_dn,
                        int32_t* tile_counts);
int64_t qwc_moe_max_tiles(int64_t pairs, int64_t e, int64_t rows_per_expert);
/* Activation rows per tile the plan uses for this problem size (128 while an expert holds up to ~85 rows on average, else
 * 192; the kernel also takes 64). */
int32_t qwc_moe_tile_rows(int64_t pairs, int64_t e);

/* Gather + rotate: xs[p, :] = f16(fwht32(x[sorted_tok[p], :])) for the sorted pairs (x_is_rotated != 0: plain copy).
 * Stands where the gather-A of qwg_moe_nax_gemm (Sources/QWMetal/include/qw_gemm_nax.metalh:436-470) and the bridge
 * (QWGemmMoE.swift:334-377) stand. */
int qwc_moe_gather(qwc_hal* hal, qwc_stream stream, const void* x_f16, int64_t ldx, int64_t h, const int32_t* sorted_tok,
                   const int32_t* expert_off, int64_t e, int64_t pairs, int32_t x_is_rotated, void* xs_f16);

/* QWGemm.encodeMoEGateUpNax / encodeMoENaxSplitF32 (QWGemmMoE.swift:201-296): grouped expert GEMM over the tile list.
 * bank: stacked expert bank [e * rows_per_expert, k]; xs: expert-sorted rotated activations f16 [pairs, k];
 * y: f16 or f32 [pairs, rows_per_expert].  x_tile_rows = qwc_moe_tile_rows() of the call that built the list.
 * epilogue: QWC_EPI_NONE, or (gate/up bank with a paired tile list) QWC_EPI_SILU_PAIR / QWC_EPI_SILU_PAIR_FWHT: y is
 * then h = f16(silu(gate) * up) [pairs, inter], rotated per 32 columns for the FWHT form — the fused twin of the
 * reference's gemmBatchedH16SwiGLU (Sources/Runtime/QWEngine/Driver/EncodeKernels.swift:156-228). */
int qwc_moe_grouped_gemm(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* bank, const void* xs_f16, int64_t pairs,
                         const qwc_moe_tile* tiles, const int32_t* tile_count, int64_t max_tiles, int32_t x_tile_rows, void* y,
                         int32_t y_dtype, int64_t ldy, int32_t epilogue);

/* QWGemm.encodeSiluMulSplitF16 (Sources/Operators/QWGEMM/QWGemmF32.swift:96-105; kernels
 * Sources/QWMetal/gemm/qwgemm_batched.metal:55-97): h[p, i] = fwht32(f16(silu(gu[p, i]) * gu[p, inter + i])). */
int qwc_moe_silu_mul(qwc_hal* hal, qwc_stream stream, const void* gu_f16, int64_t rows, int64_t inter, int32_t rotate,
                     void* h_f16);

/* QWGemm.encodeMoEDownReduceCombineF32 (QWGemmMoE.swift:298-332; kernel qwg_moe_down_reduce_combine_f32):
 * out[t, :] = sum_k wts[t, k] * dn[inv_perm[t * k_top + k], :] (dropped pairs skipped), f32 accumulate. */
int qwc_moe_combine(qwc_hal* hal, qwc_stream stream, const void* dn, int32_t dn_dtype, const int32_t* inv_perm,
                    const float* wts, int64_t t, int64_t k, int64_t h, void* out, int32_t out_dtype);
/* The same with the reference kernel's shared-expert term (Sources/QWMetal/gemm/qwgemm_moe_nax_f16.metal:7-126):
 * out[t, :] += gate[t] * shared[t, :], shared f32 [t, h] (the shared expert's output), gate f32 [t].  Both NULL: as above. */
int qwc_moe_combine_shared(qwc_hal* hal, qwc_stream stream, const void* dn, int32_t dn_dtype, const int32_t* inv_perm,
                           const float* wts, const float* shared_f32, const float* gate_f32, int64_t t, int64_t k, int64_t h,
                           void* out, int32_t out_dtype);

/* QWMoEOperator.encodeResident (QWMoEOperator.swift:206-442), grouped path with no shared expert: the whole chain
 * above on one stream.  x f16 [t, h] (standard basis unless x_is_rotated); logits f32 [t, e]; bank_gu = stacked
 * [e * 2 * inter, h] gate||up banks, bank_dn = stacked [e * h, inter]; out f32 or f16 [t, h].  scratch must hold
 * qwc_moe_scratch_bytes() bytes, 256-byte aligned. */
int qwc_moe_forward(qwc_hal* hal, qwc_stream stream, const qwc_weight_view* bank_gu, const qwc_weight_view* bank_dn,
                    int64_t e, int64_t inter, const void* x_f16, int64_t t, int64_t ldx, int32_t x_is_rotated,
                    const float* logits, int64_t k, int32_t norm_topk, float routed_scale, void* out, int32_t out_dtype,
                    void* scratch, size_t scratch_bytes);
size_t qwc_moe_scratch_bytes(int64_t t, int64_t e, int64_t k, int64_t h, int64_t inter);

#ifdef __cplusplus
}
#endif
#endif /* QWC_H */
