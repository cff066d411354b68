/*
 * rknpu_b200_ext.h -- entry points that exist only in the B200 library.
 *
 * The original project's W4A8 interface is blocking and takes host tensors.  A caller
 * whose activations already live in GPU memory (an inference engine running a
 * decoder layer on its own CUDA stream) needs neither the copies nor the host wait,
 * so the same operators are also exposed in an enqueue form: device pointers in, work
 * queued on the caller's stream, nothing allocated, nothing waited for.  None of
 * these has a counterpart in the original project.
 */
#ifndef RKNPU_B200_EXT_H
#define RKNPU_B200_EXT_H

#include "rknpu_b200_w4a8.h"
#include "rknpu_b200_rmsnorm.h"

#ifdef __cplusplus
extern "C" {
#endif

/* CUDA ordinal the context runs on; -1 for NULL or an offline context. */
int rk_npu_b200_device(const rk_npu_ctx *ctx);
/* The driver version the context writes into tuning-cache keys (the CUDA driver version of an online
 * context; what rk_npu_b200_open_offline was given for an offline one); 0 for NULL. */
uint32_t rk_npu_b200_driver_version(const rk_npu_ctx *ctx);

/* A context with no GPU behind it, for tools that inspect or write tuning caches and
 * query memory requirements on a machine without a device.  driver_version is the value
 * the cache key should carry.  Only the tuning-cache, profile and *_query functions
 * accept it; rk_npu_iommu_domain_create returns NULL for it.  Close with rk_npu_close. */
rk_npu_ctx *rk_npu_b200_open_offline(uint32_t driver_version);

/* ---- A group of GPUs: column sharding inside the library ------------------------------------------
 * The original splits a GEMM's output columns over its NPU cores in contiguous runs of 64-column blocks
 * (src/rk_npu_i4_plan.cpp:37-43).  A group context does the same over the GPUs of a box, one process per
 * GPU: rank 0 calls rk_npu_b200_group_id, hands the 128 bytes to the other ranks by whatever means the
 * application has (MPI, a file, torch.distributed ...), and every rank opens its context with
 * rk_npu_b200_open_group(dev, rank, world, id).  From then on the ordinary interface applies unchanged:
 *   - rk_npu_w4a8_weights_create[_tuned] takes the FULL B[K,N] and w_scale[N] on every rank and keeps this
 *     rank's columns (N % 128 == 0: the same slice of both halves of N, so a [gate | up] packing keeps its
 *     SwiGLU pairs on one GPU; otherwise one contiguous run);
 *   - workspaces are created with the full (M, N, K);
 *   - rk_npu_w4a8_run_f32 / _f16 and their enqueue forms take the full A on every rank (activations are
 *     replicated), compute this rank's columns, all-gather them over NVLink (NCCL, C API, loaded on first
 *     use) and leave the full C on every rank;
 *   - rk_npu_w4a8_run_swiglu_f32 / _ffn_f32 (N % 128 == 0 for the gate/up weights) do the same for the
 *     middle tensor; the down projection's row scales are the all-reduced (integer maximum) row maxima.
 * Results are bit-identical to a single GPU's for any group size.  Every rank must make the same calls in
 * the same order (they contain collectives).  A rank whose communicator cannot be created gets NULL from
 * rk_npu_b200_open_group before any GPU work.  None of this has a counterpart in the original project. */
#define RK_NPU_B200_GROUP_ID_BYTES 128
int rk_npu_b200_group_id(unsigned char *id);
rk_npu_ctx *rk_npu_b200_open_group(const char *dev, int rank, int world, const unsigned char *id);
int rk_npu_b200_group_rank(const rk_npu_ctx *ctx);   /* 0 outside a group; -1 for NULL */
int rk_npu_b200_group_size(const rk_npu_ctx *ctx);   /* 1 outside a group; 0 for NULL */
/* The partition rule itself: [*n0, *n1) of `rank` among `world` for N columns. */
int rk_npu_b200_shard_columns(int N, int world, int rank, int *n0, int *n1);
/* A caller that keeps column-parallel outputs sharded (tensor-parallel attention heads, a row-parallel layer
 * behind) needs no exchange per linear.  rk_npu_b200_w4a8_workspace_shard tells which columns this rank
 * computes: [*n0, *n1) of N, or with *two_range the same [*n0, *n1) of both halves of N; *columns in all.
 * rk_npu_b200_w4a8_enqueue_local_f16 / _f32 queue the linear and write only those columns, compact
 * [M][*columns], to dLocal -- no collective.  rk_npu_b200_group_all_gather is the group's all-gather for
 * whatever the caller batches up: every rank's piece of bytes_per_rank bytes already lies at
 * dBuffer + rank * bytes_per_rank (in place), afterwards every rank holds all pieces. */
int rk_npu_b200_w4a8_workspace_shard(const rk_npu_w4a8_workspace *workspace, int *two_range, int *n0, int *n1, int *columns);
int rk_npu_b200_w4a8_enqueue_local_f16(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                       const uint16_t *dA, uint16_t *dLocal, void *cuda_stream);
int rk_npu_b200_w4a8_enqueue_local_f32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                       const float *dA, float *dLocal, void *cuda_stream);
int rk_npu_b200_group_all_gather(rk_npu_ctx *ctx, void *dBuffer, size_t bytes_per_rank, void *cuda_stream);

/* Queue one W4A8 linear on `cuda_stream` (a cudaStream_t; NULL = the legacy default
 * stream).  dA / dC are device pointers on the context's GPU with the shapes of the
 * blocking calls.  Returns after queuing.  The workspace must not be used by another
 * call until the queued work has finished.  Argument errors are reported as in the
 * blocking calls; a non-finite activation is only known once the work has run: call
 * rk_npu_b200_w4a8_finish after synchronising. */
int rk_npu_b200_w4a8_enqueue_f32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                 const float *dA, float *dC, void *cuda_stream);
int rk_npu_b200_w4a8_enqueue_f16(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                 const uint16_t *dA, uint16_t *dC, void *cuda_stream);
int rk_npu_b200_w4a8_enqueue_swiglu_f32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                        const float *dA, float *dMiddle, void *cuda_stream);
/* gate/up -> SwiGLU -> down in one queue; a non-finite middle makes the down kernels
 * return without writing and is reported by rk_npu_b200_w4a8_finish(down).
 * On a group context dMiddle may be NULL when the caller does not need the middle tensor (feature count a
 * multiple of 64 x group size): the GPUs then agree on the row maxima, quantise their own feature slice and
 * all-gather int8 codes -- a quarter of the bytes of the fp32 middle -- with bit-identical results. */
int rk_npu_b200_w4a8_enqueue_ffn_f32(rk_npu_w4a8_workspace *gate_up, const rk_npu_w4a8_weights *gate_up_weights,
                                     rk_npu_w4a8_workspace *down, const rk_npu_w4a8_weights *down_weights,
                                     const float *dA, float *dMiddle, float *dC, void *cuda_stream);

/* Several INDEPENDENT linears in one launch.  On a stream, every queued linear waits for the one in front, so a
 * decoder layer's q / k / v projections (or gate and up), which read the same activations and do not depend on
 * each other, pay the dependent latency of a small-batch launch three times.  This call queues up to four
 * linears of up to eight tokens (the same token count for all, binary16, workspaces of the single-launch decode
 * family) as ONE kernel launch: they wait once for whatever is in front of them on the stream and then run
 * side by side.  Outputs are written as by rk_npu_b200_w4a8_enqueue_local_f16 (on one GPU: the whole
 * [M,N]; in a group: this rank's columns, compact).  The caller states the independence: no dLocal[i] may
 * be read as a dA[j] of the same call.  The launch is counted on the first workspace.
 * RK_NPU_ERR_PARAM for other workspace families, mixed token counts or repeated workspaces / outputs.
 * No counterpart in the original project. */
int rk_npu_b200_w4a8_enqueue_batch_f16(int count, rk_npu_w4a8_workspace *const *workspaces,
                                       const rk_npu_w4a8_weights *const *weights, const uint16_t *const *dA,
                                       uint16_t *const *dLocal, void *cuda_stream);

/* ---- Column-sharded FFN: the pieces around the exchange between GPUs ----------------------
 * When gate/up and down are sharded by output columns over g GPUs (each GPU holds the gate and
 * up columns of one feature slice f0..f1 and a column slice of down), a GPU produces
 * middle[:, f0:f1] but the down projection needs the whole row, quantised with the scale of the
 * whole row.  The three calls below let the caller exchange int8 codes instead of the fp32
 * middle (a quarter of the bytes) and still obtain bit-identical results:
 *   1. rk_npu_b200_w4a8_enqueue_swiglu_collect_f32: the SwiGLU projection of this GPU's slice;
 *      additionally maxes the bit patterns of max|middle[m, f0:f1]| into dRowMaxima[M]
 *      (caller-owned device words that must be zero before the call).
 *   2. the caller combines dRowMaxima across GPUs with an integer maximum (e.g. ncclAllReduce,
 *      ncclMax on 32-bit integers: the patterns are non-negative) on the same stream;
 *   3. rk_npu_b200_w4a8_enqueue_quantize_slice: dMiddle[M, f1-f0] -> dCodes[M, f1-f0] int8 with the
 *      combined maxima (the rule of the down projection's own quantiser); dRowMaxima is only read;
 *   4. the caller all-gathers the code slices: [g][M][F/g] on every GPU;
 *   5. rk_npu_b200_w4a8_enqueue_codes_f32 on the down workspace: dCodes is [parts][M][K/parts]
 *      (parts = g; K/parts a multiple of 16; parts = 1 accepts a plain [M,K] matrix), scales come
 *      from dRowMaxima, which is cleared for the next step.  A non-finite middle shows as a
 *      non-finite maximum: the GEMM returns without writing and rk_npu_b200_w4a8_finish(down)
 *      reports RK_NPU_ERR_PARAM, as in the single-GPU FFN.
 * None of these has a counterpart in the original project, whose FFN runs on one device. */
int rk_npu_b200_w4a8_enqueue_swiglu_collect_f32(rk_npu_w4a8_workspace *gate_up, const rk_npu_w4a8_weights *gate_up_weights,
                                                const float *dA, float *dMiddle, uint32_t *dRowMaxima, void *cuda_stream);
int rk_npu_b200_w4a8_enqueue_quantize_slice(rk_npu_w4a8_workspace *gate_up, const float *dMiddle,
                                            const uint32_t *dRowMaxima, int8_t *dCodes, void *cuda_stream);
int rk_npu_b200_w4a8_enqueue_codes_f32(rk_npu_w4a8_workspace *down, const rk_npu_w4a8_weights *down_weights,
                                       const int8_t *dCodes, int parts, uint32_t *dRowMaxima, float *dC, void *cuda_stream);

/* After the caller has synchronised the stream: RK_NPU_OK, RK_NPU_ERR_PARAM (non-finite
 * activation or middle in the last queued call) or RK_NPU_ERR_SUBMIT (a bounded device
 * wait ran out).  Clears the recorded status. */
int rk_npu_b200_w4a8_finish(rk_npu_w4a8_workspace *workspace);

/* Diagnostic: the same linear as rk_npu_w4a8_run_f32 / _f16 (activation_is_f16 selects
 * the input type) but the exact int32 sums sum_k q*B are returned in acc[M,N] instead of
 * the dequantised output.  Blocking; host or device pointers. */
int rk_npu_b200_w4a8_run_acc_i32(rk_npu_w4a8_workspace *workspace, const rk_npu_w4a8_weights *weights,
                                 const void *A, int activation_is_f16, int32_t *acc);

/* Diagnostic: the per-token scales of the last call on this workspace and the int8 codes
 * [M,K] its activations were quantised to (host pointers; either may be NULL).  The codes
 * are those of the last rk_npu_b200_w4a8_run_acc_i32 call when the workspace runs the
 * single-kernel small-batch path, which otherwise keeps them in shared memory only. Blocking. */
int rk_npu_b200_w4a8_last_quant(rk_npu_w4a8_workspace *workspace, float *scales, int8_t *codes);

/* Scheduling override for experiments and tuning.  variant: 0 = keep, else the workspace's kernel family
 * (1 quantise + mma.sync GEMM, 2 quantise + tcgen05 GEMM, 3 single-kernel split-K small batch, 4 quantise +
 * persistent tcgen05 streaming GEMM, 5 single-kernel decode with whole-K CTAs; chosen at creation,
 * RK_NPU_B200_VARIANT overrides where the geometry allows).  The family is fixed with the activation-code layout at
 * creation, except that a workspace of up to eight tokens may move between 3 and 5, which share it.
 * split_k: 0 = automatic, else the number of CTAs that cooperate on a column tile: the split-K factor (1..8 for
 * family 3; 1, 2, 4, 8 for 1 and 2) or the decode kernel's cluster size (1, 2, 4, 8); ignored by family 4.
 * Returns RK_NPU_ERR_PARAM when the workspace geometry cannot run the request.
 * rk_npu_b200_w4a8_schedule reads both back (either pointer may be NULL). */
int rk_npu_b200_w4a8_set_schedule(rk_npu_w4a8_workspace *workspace, int variant, int split_k);
int rk_npu_b200_w4a8_schedule(const rk_npu_w4a8_workspace *workspace, int *variant, int *split_k);

/* Diagnostics: with tracing enabled the kernels record device stamps of their latest launch.
 * Single-kernel small-batch path: eight stamps per CTA -- start (global timer, ns), then cycles
 * since the CTA's start at: weights requested, dependency met, scales known, slice quantised,
 * contraction done, partials exchanged -- and the end (ns); trace_read copies stamps[ctas][8]
 * (CTA index = blockIdx.y * gridDim.x + blockIdx.x, at most 16384 CTAs).
 * Persistent large-batch GEMM: CTA pair 0 records per tile j < 16 at [8 j + 0..6] the cycles since
 * kernel start at which the MMA issuer begins, issues its first MMA, commits the last, the epilogue
 * sees the accumulator, hands tensor memory back, has stored the tile, and the cycles the issuer
 * waited for operands; [128 + 2 j], [129 + 2 j], [160 + j] the cycles one unpack warp waited for
 * weights, for a free tensor-memory buffer and for activations; [200] the CTA pairs in the grid.
 * The caller synchronises first.  `bench.py --case decode|prefill --stamps` prints both. */
int rk_npu_b200_w4a8_trace_enable(rk_npu_w4a8_workspace *workspace, int enable);
int rk_npu_b200_w4a8_trace_read(rk_npu_w4a8_workspace *workspace, unsigned long long *stamps, int ctas);

/* One W4A8 linear (binary16 in and out) that allocates nothing.  It has no counterpart in the
 * original project.  It is meant for callers that are not allowed to allocate when they need
 * the result -- an engine that carved up its device memory once and forbids cudaMalloc from
 * then on, a plugin inside a latency-critical loop -- and therefore cannot create a workspace.
 * The scratch a workspace would own (activation codes, per-token scales, status) lives in a
 * fixed 2 MiB + 4 KiB array inside the library image; every GPU that loads the library holds
 * it until the process exits.
 *   weights      an existing weight object (its creation did allocate; this call does not)
 *   dA, dC       device pointers on the weights' GPU: [M,K] activations, [M,N] output
 *   M            1..32 tokens, and 32 x K (K rounded up to 128; 8 or 16 x K for M <= 8 / 16)
 *                must fit in 2 MiB, i.e. K <= 65536 for M > 16; larger sizes return
 *                RK_NPU_ERR_NOMEM and do nothing
 *   cuda_stream  a cudaStream_t; the work is queued, not waited for
 * The first call on a device looks up the array's device address; make that first call before
 * any stream capture starts.  All calls share the one array, which keeps the previous call's
 * contents (the parts that must start at zero are cleared on the stream first): two calls
 * whose GPU work overlaps -- different streams, no ordering between them -- race on it.
 * A row of dA holding NaN or Inf leaves dC unwritten, and a bounded wait inside the kernels that
 * ran out leaves dC undefined; neither is known when the call returns (RK_NPU_OK once queued):
 * ask rk_npu_b200_w4a8_static_status after synchronising.  The caller's current CUDA device is
 * the same after the call as before it. */
int rk_npu_b200_w4a8_enqueue_f16_static(const rk_npu_w4a8_weights *weights, const uint16_t *dA, uint16_t *dC, int M,
                                        void *cuda_stream);
/* Verdict of the last rk_npu_b200_w4a8_enqueue_f16_static call on the weights' GPU, read from the
 * same fixed array (no allocation; a 16-byte blocking copy).  Call it after synchronising the stream
 * the linear was queued on.  *bad_input: 1 when a row of dA held NaN or Inf (dC was not written);
 * *device_error: 1 when a bounded wait ran out (dC undefined).  Returns RK_NPU_OK, RK_NPU_ERR_PARAM
 * (bad input) or RK_NPU_ERR_SUBMIT (device error or the copy failed).  No counterpart in the
 * original project. */
int rk_npu_b200_w4a8_static_status(const rk_npu_w4a8_weights *weights, int *bad_input, int *device_error);

/* ---- Residual add + RMSNorm on device tensors ------------------------------------------------------------
 * The operator of rk_npu_add_rmsnorm_f16_run on the caller's own device tensors and stream: the kernel is queued,
 * nothing is copied or waited for.  row_major = 0: the original's block-8 layout (D/8, M, 8); row_major = 1: plain
 * [M, D] rows, the layout rk_npu_b200_w4a8_enqueue_f16 takes, so that the normalised rows feed the quantised FFN
 * without a transpose.  rows: 1..plan M (a smaller batch than the plan was made for is allowed).  The tensors must
 * be 16-byte aligned; an output must not overlap an input or the other output.  RK_NPU_ERR_PARAM / RK_NPU_ERR_SUBMIT
 * as for the blocking call.  No counterpart in the original project. */
int rk_npu_b200_add_rmsnorm_f16_enqueue(rk_npu_add_rmsnorm_f16_plan *plan, int rows, int row_major, const uint16_t *dX,
                                        const uint16_t *dResidual, uint16_t *dResidualOut, uint16_t *dNormOut,
                                        void *cuda_stream);

/* ---- Test hooks: failures produced on the host, or by a wait that is allowed to run out ---------------
 * None of these faults, traps or hangs a GPU.
 * rk_npu_b200_test_fail_allocation(n): the (n+1)-th device allocation from now on fails as if memory were
 *   exhausted (constructors return NULL and release what they had); n < 0 switches the hook off.  Process-wide.
 * rk_npu_b200_w4a8_test_starve(ws, 1): launches of a decode-kernel workspace make the first weight barrier of
 *   every CTA expect 16 bytes that no copy brings, so the bounded wait on it runs out after the workspace's
 *   timeout_ms, the kernel records the error and returns (all real copies have landed), and the call reports
 *   RK_NPU_ERR_SUBMIT; (ws, 0) restores normal launches.  RK_NPU_ERR_PARAM for other kernel families.
 * rk_npu_b200_w4a8_test_device_error(ws): sets the workspace's device-side error word from the host, as a kernel
 *   whose wait ran out would; the next status read reports RK_NPU_ERR_SUBMIT and clears it. */
void rk_npu_b200_test_fail_allocation(long long after);
int rk_npu_b200_w4a8_test_starve(rk_npu_w4a8_workspace *workspace, int on);
int rk_npu_b200_w4a8_test_device_error(rk_npu_w4a8_workspace *workspace);

/* Kernels this workspace has launched since creation (for launch accounting). */
uint64_t rk_npu_b200_w4a8_launch_count(const rk_npu_w4a8_workspace *workspace);

#ifdef __cplusplus
}
#endif
#endif /* RKNPU_B200_EXT_H */
