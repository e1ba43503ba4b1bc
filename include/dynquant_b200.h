/*
 * dynquant_b200 -- C ABI of the packed decode path for NVIDIA B200 (sm_100a).
 *
 * Plain pointers, sizes and a CUDA stream handle; no torch, no C++ types.
 * Every tensor pointer is a DEVICE pointer unless the parameter name ends in
 * `_host`.  All entry points are asynchronous on `stream` (a cudaStream_t
 * passed as void*; NULL is the legacy default stream) except the `_host`
 * variants, which synchronise that stream before returning.
 *
 * Every function that can fail returns a dq_status.  On a non-zero status
 * dq_last_error() returns a message for the calling thread; the messages keep
 * the wording the reference's operators raise, so callers that match on them
 * ("exceeds the kernel's limit", "resolved positive count") keep working.
 *
 * "Reference" citations name files of the kambojvikram/dynquant project by
 * their path inside that project.
 */
#ifndef DYNQUANT_B200_H_
#define DYNQUANT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define DQ_API
#else
#define DQ_API __attribute__((visibility("default")))
#endif

/* Same numbers as packages/dynquant-kernels/csrc/include/dynquant/abi.h:23-39. */
#define DQ_ABI_VERSION 2
#define DQ_GROUP_SIZE_ALIGNMENT 32
#define DQ_GEMV_MAX_ROWS 8
#define DQ_GEMV_CHUNKED_MAX_ROWS 64 /* dq_gemv_shards_rows: row chunks of <= 8, above it dequant + dense wins */
/* Most tokens one expert may receive in a single dq_moe_* call. */
#define DQ_MOE_MAX_TOKENS 64
/* Size of the scratch buffer built into the library for dq_moe_gemv_static (2 MiB). */
#define DQ_MOE_STATIC_SCRATCH_BYTES (2 * 1024 * 1024)

typedef enum dq_status {
  DQ_OK = 0,
  DQ_ERR_INVALID = 1,     /* argument / geometry check failed (reference: TORCH_CHECK) */
  DQ_ERR_CUDA = 2,        /* a CUDA runtime call or the launch failed */
  DQ_ERR_UNSUPPORTED = 3, /* legal input this build has no kernel for */
  DQ_ERR_DEVICE = 4       /* a kernel reported an error through its status word */
} dq_status;

typedef enum dq_dtype { DQ_F16 = 0, DQ_BF16 = 1, DQ_F32 = 2 } dq_dtype;

/*
 * One packed tensor: the (packed, scales, offsets, bits, group_values,
 * in_features) tuple the reference passes to every operator
 * (packages/dynquant-kernels/csrc/bindings.cpp:204-214), plus the shapes that
 * at::Tensor carries implicitly there.
 *
 *   packed   int32 [rows, words_per_row], row-major, bit patterns unsigned
 *   scales   [rows, num_groups] in meta_dtype
 *   offsets  same shape and dtype, or NULL meaning zero
 *   group_values  resolved values per group, never the -1 per-row sentinel
 *   in_features   unpadded reduction length
 */
typedef struct dq_weight {
  const void* packed;
  const void* scales;
  const void* offsets;
  int64_t rows;
  int64_t words_per_row;
  int64_t num_groups;
  int64_t group_values;
  int64_t in_features;
  int32_t bits;
  int32_t meta_dtype; /* dq_dtype */
} dq_weight;

/* Derived sizes; mirrors nbit::RowGeometry,
 * packages/dynquant-kernels/csrc/include/dynquant/geometry.h:47-57. */
typedef struct dq_geometry {
  int32_t group_values;
  int32_t num_groups;
  int32_t words_per_group;
  int32_t words_per_row;
  int32_t in_features;
  int32_t blocks_per_group;
  int32_t blocks_per_row;
} dq_geometry;

/* ---- metadata (reference: bindings.cpp:188-197 abi_version, built_with_cuda,
 *      compiled_architectures, gemv_max_rows) -------------------------------- */
DQ_API int32_t dq_abi_version(void);
DQ_API int32_t dq_built_with_cuda(void);
DQ_API const char* dq_compiled_architectures(void);
DQ_API int32_t dq_gemv_max_rows(void);

/* Kernels this library has launched in this process so far, over all entry
 * points (monotonic; counted at launch, also during stream capture).  No
 * reference counterpart: the reference launches one kernel per operator call
 * (csrc/cuda/gemv.cu:231-275), here one call may be one launch for several
 * matrices or several launches for one, and benchmarks report the real number. */
DQ_API int64_t dq_launch_count(void);
/* Name of the kernel the calling thread's most recent GEMV or MoE entry point launched last
 * ("gemv_mma_stream_kernel", "gemv_mma_stream_multi_kernel", "gemv_mma_stream_sliced_kernel", "gemv_mma_tile_kernel",
 * "gemv_mma_kernel", "gemv_fast_kernel",
 * "gemv_general_kernel", "gemv_plan_kernel", "gemv_rows_kernel", "moe_grouped_kernel", "moe_combine_kernel",
 * "moe_down_token_kernel"; "" before the first launch).  No reference
 * counterpart: the reference has two kernels and a documented rule between them
 * (csrc/gemv/gemv.cu:566-598); here a test uses this to prove which kernel it exercised. */
DQ_API const char* dq_last_kernel(void);
DQ_API int32_t dq_moe_max_tokens(void);
DQ_API const char* dq_last_error(void);

/* ---- geometry (reference: resolve_geometry, geometry.h:63-132) -------------
 * Host-only validation; reads no device memory.  `op` prefixes the message. */
DQ_API int32_t dq_resolve_geometry(const char* op, const dq_weight* w, dq_geometry* out);

/* ---- dequant (reference: dequant_cuda, csrc/quant/dequant.cu:130-165) ------
 * out [rows, in_features] in out_dtype.  The reference writes the scales
 * dtype; any dq_dtype is accepted here.  w = float(q)*scale, then + offset,
 * in fp32, one rounding to out_dtype. */
DQ_API int32_t dq_dequant(const dq_weight* w, void* out, int32_t out_dtype, void* stream);

/* ---- achievable-bandwidth probes (reference: achievable_bandwidth,
 *      packages/dynquant-core/src/dynquant/commands/bench.py:95-120, which times
 *      a large read and a large copy in the session it benchmarks in) ----------
 * dq_probe_read streams `bytes` (a multiple of 16, 16-byte aligned buffer) from
 * HBM once and XORs every 32-bit word read into *sink (device memory, 8-byte
 * aligned; the low 32 bits carry the XOR of all words, so a caller can check
 * that the whole buffer was read).  dq_probe_copy copies `bytes` between two
 * non-overlapping 16-byte aligned device buffers.  Both enqueue one kernel on
 * `stream`; the caller times them with events. */
DQ_API int32_t dq_probe_read(const void* src, int64_t bytes, uint64_t* sink, void* stream);
DQ_API int32_t dq_probe_copy(void* dst, const void* src, int64_t bytes, void* stream);

/* ---- gemv (reference: gemv_cuda, csrc/gemv/gemv.cu:695-756) ----------------
 * x [m, in_features] in x_dtype, contiguous, m <= DQ_GEMV_MAX_ROWS.
 * out [m, rows] in out_dtype (the reference writes x's dtype; DQ_F32 gives the
 * unrounded fp32 accumulators).  x_dtype may differ from w->meta_dtype.
 * fp32 accumulation, fixed summation order: bit-identical run to run. */
DQ_API int32_t dq_gemv(const void* x, int32_t x_dtype, int64_t m, const dq_weight* w, void* out,
                       int32_t out_dtype, void* stream);

/* Several shards of one fused layer from one call (replaces the per-shard loop
 * plus concat of integration/vllm_plugin/linear.py:172-186 and
 * integration/serving_common/fuse.py:41-53).  Shard i writes columns
 * [sum(rows[0..i)), +rows[i]) of out [m, out_stride]; every shard shares x and
 * in_features.  bias [sum rows] in out_dtype or NULL.  Up to four shards at a
 * time, of any mix of widths, run as ONE kernel launch. */
DQ_API int32_t dq_gemv_shards(const void* x, int32_t x_dtype, int64_t m, const dq_weight* shards,
                              int32_t num_shards, const void* bias, void* out, int64_t out_stride,
                              int32_t out_dtype, void* stream);
/* dq_gemv_shards for up to DQ_GEMV_CHUNKED_MAX_ROWS activation rows (the 9..64-row band in which
 * the reference already pays for dequantize + dense matmul, runtime/ops.py:205-231).  A shard
 * with 128-value groups and enough work to fill half of the SMs goes through the many-rows kernel:
 * one pass over its weights per 32 rows, a step's fragments decoded once for all of them (shards
 * of few rows slice the reduction axis over a thread-block cluster).  Otherwise the rows are cut
 * into ceil(m / 8) chunks of equal size (+-1) and up to four (chunk, shard) pairs leave as one
 * launch of the tiled kernel, so that a matrix is read from HBM once and by the other chunks from
 * L2; matrices long enough for the streaming kernel go chunk by chunk.  Same arguments and
 * results as dq_gemv_shards. */
DQ_API int32_t dq_gemv_shards_rows(const void* x, int32_t x_dtype, int64_t m, const dq_weight* shards,
                                   int32_t num_shards, const void* bias, void* out, int64_t out_stride,
                                   int32_t out_dtype, void* stream);

/* One GEMV of a sequence; see dq_gemv_sequence. */
typedef struct dq_gemv_job {
  const void* x;    /* [m, weight.in_features] in x_dtype */
  void* out;        /* [m, out_stride] in out_dtype; this job writes columns [out_col0, +rows) */
  const void* bias; /* [>= out_col0 + rows] in out_dtype, indexed by output column, or NULL */
  int64_t m;
  int64_t out_stride;
  int64_t out_col0;
  int32_t x_dtype;
  int32_t out_dtype;
  dq_weight weight;
} dq_gemv_job;

/* Launch `num_jobs` GEMVs back to back on `stream`, in order, from one host
 * call: what one decode step of a model does through the reference runtime's
 * per-module quantized_matmul calls
 * (packages/dynquant-core/src/dynquant/runtime/ops.py:184-231), without a
 * host round trip per module.  Every launch carries the programmatic
 * dependent-launch attribute, so job i+1 streams its first weights while job
 * i drains and reads its activation only after job i has completed.
 * Consecutive jobs that read the SAME activation (same x pointer, m and dtypes:
 * the q/k/v or gate/up shards of a layer) cannot depend on one another; up to
 * four of them are issued as one launch, so their outputs must not overlap.
 * All jobs are validated before the first launch. */
DQ_API int32_t dq_gemv_sequence(const dq_gemv_job* jobs, int32_t num_jobs, void* stream);

/* ---- whole-step plans: a job list compiled once, run by ONE persistent kernel ------------
 * Same semantics as dq_gemv_sequence over the same job list (reference: one
 * quantized_matmul call per module per decode step,
 * packages/dynquant-core/src/dynquant/runtime/ops.py:184-231; its own profile of a decode
 * step -- experiments/four_point/RESULTS.md:884-906 -- is host and launch time around
 * single-digit-microsecond kernels).  Consecutive jobs that read the same activation form a
 * stage; a stage may read what the stage before it wrote.  One grid of one CTA per SM walks
 * the stages: weights stream ahead of the arithmetic across stage boundaries, and a stage
 * reads its activation only after the stage before it has stored every output -- a
 * completion counter in `workspace`, polled with a BOUNDED spin.  If the bound runs out
 * (the grid was not resident at once, or a test asked for it) the kernel sets a status word
 * and returns; dq_plan_status reports DQ_ERR_DEVICE.
 *
 * Requirements, checked by dq_plan_create (DQ_ERR_UNSUPPORTED names the first job that
 * fails them; launch such lists with dq_gemv_sequence): fp16/bf16 activations of one dtype,
 * 1..DQ_GEMV_MAX_ROWS rows, 16-byte aligned with in_features a multiple of 8; fp16/bf16
 * scales; 128-value groups, an even number per row; 16-byte aligned packed rows.
 *
 * `workspace` is caller-owned device memory (dq_plan_workspace_bytes, 256-byte aligned)
 * that must stay alive and untouched for the life of the plan; the job list's tensors are
 * referenced, not copied.  A plan belongs to the device that was current at creation.
 * Launches of ONE plan must not overlap on the GPU (they share the counters); launches of
 * different plans may.  dq_plan_launch enqueues one persistent kernel per run of consecutive
 * stages, and hands a matrix long enough to fill the machine many row tiles deep (a vocabulary
 * projection) to the streaming GEMV as a launch of its own -- dq_plan_info.launches in all,
 * two for a decoder stack followed by its lm_head; all of it is capturable. */
typedef struct dq_plan dq_plan;
typedef struct dq_plan_info {
  int32_t num_stages;
  int32_t num_jobs;
  int32_t grid;       /* CTAs = SMs of the device */
  int32_t threads;    /* per CTA */
  int32_t ring_slots; /* weight slots each warp keeps in flight */
  int32_t launches;   /* kernels one dq_plan_launch enqueues (see below) */
  int64_t shared_bytes;
} dq_plan_info;
DQ_API int32_t dq_plan_workspace_bytes(int32_t num_jobs, int64_t* bytes);
DQ_API int32_t dq_plan_create(const dq_gemv_job* jobs, int32_t num_jobs, void* workspace,
                              int64_t workspace_bytes, void* stream, dq_plan** plan);
DQ_API int32_t dq_plan_launch(dq_plan* plan, void* stream);
/* Synchronises `stream` and reads the plan's status word: DQ_OK, or DQ_ERR_DEVICE with the
 * stage that gave up in dq_last_error() (the word and the counters are then cleared, so the
 * plan can be launched again). */
DQ_API int32_t dq_plan_status(dq_plan* plan, void* stream);
DQ_API int32_t dq_plan_describe(const dq_plan* plan, dq_plan_info* info);
/* Slicing chosen for one stage: warps along the reduction axis, steps per ring slot and the
 * CTAs given to each of its (up to four) jobs.  Any out pointer may be NULL. */
DQ_API int32_t dq_plan_stage_shape(const dq_plan* plan, int32_t stage, int32_t* k_slices,
                                   int32_t* slot_steps, int32_t* cta_counts);
/* Failure-handling hook: overwrite the count stage `stage` waits for (negative: keep it) and
 * the spin bound of every wait.  A count the previous stage can never reach makes the wait
 * run out -- the way the tests exercise the error path without faulting anything. */
DQ_API int32_t dq_plan_set_wait(dq_plan* plan, int32_t stage, int32_t wait_target,
                                int32_t spin_limit, void* stream);
DQ_API void dq_plan_destroy(dq_plan* plan);

/* Same as dq_gemv with x and out in HOST memory: copies x to the device,
 * launches, copies the result back and synchronises.  `x_dev` / `out_dev` are
 * caller-provided device staging buffers of at least the same sizes. */
DQ_API int32_t dq_gemv_host(const void* x_host, int32_t x_dtype, int64_t m, const dq_weight* w,
                            void* out_host, int32_t out_dtype, void* x_dev, void* out_dev,
                            void* stream);

/* ---- MoE grouped GEMV -------------------------------------------------------
 * No reference kernel or operator exists for this (the reference refuses fused-MoE
 * layers: integration/vllm_plugin/config.py:107-112, runtime/linear.py:442-456).  The
 * weight layout is the reference's: a stacked bank [E, out, in] folded to rows
 * (quant/tensor.py:253-255), expert e owning rows [e*out, (e+1)*out); gate_up is
 * [E, 2*inter, hidden] with an expert's gate rows before its up rows and down is
 * [E, hidden, inter] (graph/experts.py:35-43).
 *
 *   y[t] = sum_k topk_w[t,k] * W_down[e] ( silu(W_gate[e] x[t]) * (W_up[e] x[t]) ),  e = topk_ids[t,k]
 *
 * x [tokens, hidden] in x_dtype (fp16 or bf16), tokens <= DQ_MOE_MAX_TOKENS;
 * topk_ids [tokens, topk] int32, ids outside [0, num_experts) are skipped (an
 * expert-parallel rank passes its local expert numbers and -1 for the rest); the ids of one
 * token must be distinct, so that no expert receives more than `tokens` assignments;
 * topk_w [tokens, topk] fp32; y [tokens, hidden] in y_dtype.  The intermediate
 * silu(g)*u is rounded once to x_dtype.  fp32 accumulation, no atomics: bit-identical
 * run to run.  `scratch` is caller-owned device memory of at least
 * dq_moe_scratch_bytes() bytes, 256-byte aligned; its contents are overwritten. */
DQ_API int32_t dq_moe_scratch_bytes(int64_t tokens, int64_t topk, int64_t hidden, int64_t inter,
                                    int64_t num_experts, int32_t act_dtype, int64_t* bytes);
DQ_API int32_t dq_moe_gemv(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids,
                           const float* topk_w, int64_t topk, int64_t num_experts,
                           const dq_weight* gate_up, const dq_weight* down, int64_t hidden,
                           int64_t inter, void* y, int32_t y_dtype, void* scratch,
                           int64_t scratch_bytes, void* stream);

/* dq_moe_gemv for one rank of an expert-parallel layer: topk_ids carry GLOBAL expert numbers and
 * the banks hold experts [first_expert, first_expert + num_experts) only; every other id is
 * skipped, so y is this rank's partial sum.  Saves the host framework the elementwise pass that
 * renumbers the ids per rank. */
DQ_API int32_t dq_moe_gemv_shard(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids,
                                 const float* topk_w, int64_t topk, int64_t first_expert,
                                 int64_t num_experts, const dq_weight* gate_up, const dq_weight* down,
                                 int64_t hidden, int64_t inter, void* y, int32_t y_dtype, void* scratch,
                                 int64_t scratch_bytes, void* stream);
/* dq_moe_gemv without a scratch argument and without any allocation.  This entry point has
 * no counterpart in the reference.
 *
 * Who needs it: host code that must not, or cannot, obtain device memory at call time --
 * for example a serving worker written against this C ABI (no torch allocator in reach)
 * that has already handed all free HBM to its KV-cache pool, where a cudaMalloc would
 * fail or stall the device, or a caller bound to a fixed memory plan that forbids new
 * allocations once serving has started.  Inputs and outputs are still the caller's.
 *
 * The scratch lives inside the library: DQ_MOE_STATIC_SCRATCH_BYTES (2 MiB) of device
 * memory per GPU that loads the library, held until the process exits.  A problem whose
 * dq_moe_scratch_bytes() exceeds that is rejected with DQ_ERR_INVALID and a message
 * naming both numbers (8 tokens x top-8 of a 2048/768 expert layer needs ~0.6 MiB).
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * The first call on each device looks up the buffer's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before any
 * stream capture begins.  On EVERY call the device that owns `stream`, x and y must be the
 * current device: the address is looked up for the current device, and kernels launched on
 * another device's stream would be handed an address that is not theirs.  Every call on a device shares the one buffer: it still holds the
 * previous call's intermediates (the rounded silu(g)*u rows and the per-assignment down
 * projections) when the next call starts -- each call rewrites everything it reads, nothing
 * has to start at zero -- so two calls that may overlap on the GPU (different streams, no
 * ordering between them) race on it.  Order them, or give the overlapping one its own scratch
 * through dq_moe_gemv. */
DQ_API int32_t dq_moe_gemv_static(const void* x, int32_t x_dtype, int64_t tokens,
                                  const int32_t* topk_ids, const float* topk_w, int64_t topk,
                                  int64_t num_experts, const dq_weight* gate_up,
                                  const dq_weight* down, int64_t hidden, int64_t inter, void* y,
                                  int32_t y_dtype, void* stream);

/* ---- exchanges of the sharded paths over peer memory ------------------------------------
 * No reference counterpart: the reference issues no collective (tensor parallelism there is
 * weight placement only, integration/vllm_plugin/parameter.py:102-154; the gathers are the
 * host framework's).  These replace a host-issued library collective where the payload is a
 * few KB and the call is made hundreds of times per decode step: the output slabs of a
 * column-sharded layer (all-gather) and the partial sums of an expert-parallel layer
 * (reduce-scatter).  Each enqueues ordinary kernels on `stream` (capturable): a rank STORES
 * its piece into every peer's exchange buffer through peer-mapped pointers, raises a flag
 * there, and waits -- a bounded number of polls -- for the peers' flags in its own buffer.
 * Only local memory is ever read; no TMA, no multicast.
 *
 * `buffers`: DEVICE array of `world` pointers, entry i = rank i's exchange buffer as mapped
 * into this process (CUDA IPC / symmetric memory), every buffer `buffer_bytes` long, zeroed
 * before first use, 16-byte aligned.  The first dq_peer_header_bytes() bytes hold flags,
 * epochs and a status word; the rest is two halves used alternately, each of which must hold
 * `world` pieces.  All ranks must issue the same sequence of exchanges on a group.  If a
 * peer's flag does not arrive within `spin_limit` polls (0: a default of about a second) the
 * kernel sets the status word and returns; dq_peer_status then reports DQ_ERR_DEVICE. */
typedef struct dq_peer_group {
  void* const* buffers;
  int64_t buffer_bytes;
  int32_t world, rank;
  int32_t spin_limit;
  int32_t reserved;
} dq_peer_group;
DQ_API int64_t dq_peer_header_bytes(void);
/* Every rank contributes `bytes` (a multiple of 16) at `src`; `out` receives world * bytes,
 * rank i's piece at out + i * bytes. */
DQ_API int32_t dq_peer_all_gather(const dq_peer_group* group, const void* src, int64_t bytes,
                                  void* out, void* stream);
/* Up to four tensors gathered by ONE exchange launch (an expert layer's token rows, expert ids and
 * routing weights travel together): part i contributes bytes[i] (a multiple of 16) from srcs[i],
 * and outs[i] receives world * bytes[i], rank r's copy at outs[i] + r * bytes[i].  srcs, bytes and
 * outs are HOST arrays. */
DQ_API int32_t dq_peer_all_gather_parts(const dq_peer_group* group, const void* const* srcs,
                                        const int64_t* bytes, void* const* outs, int32_t parts,
                                        void* stream);
/* `partial` holds world * count floats: the rows this rank computed for rank i's elements at
 * partial + i * count.  `out` (count elements of out_dtype) receives the sum over source ranks
 * of the rows that belong to this rank, added in rank order, rounded once. */
DQ_API int32_t dq_peer_reduce_scatter_f32(const dq_peer_group* group, const float* partial,
                                          int64_t count, void* out, int32_t out_dtype, void* stream);
/* Synchronises `stream` and reads the status word of this rank's own buffer (`local_buffer` =
 * the pointer that is buffers[rank]). */
DQ_API int32_t dq_peer_status(const dq_peer_group* group, const void* local_buffer, void* stream);

/* ---- a column-sharded stage and its all-gather as ONE launch ----
 *
 * Replaces, for a stage of a tensor-parallel decode step, the pair "GEMV over this rank's row
 * slab, then the host framework's all-gather" (vLLM: the gather after a ColumnParallelLinear
 * whose weights were placed by integration/vllm_plugin/parameter.py:102-154) -- and this
 * library's own pair dq_gemv_sequence + dq_peer_all_gather.  The GEMV kernel's CTAs copy their
 * output rows into EVERY rank's window with ordinary stores through peer-mapped pointers
 * (nothing is read from a peer; no TMA, no multicast), the launch's last CTA raises this rank's
 * flag in every window and waits, a bounded number of polls, for the other ranks' flags in its
 * own.  When the launch completes, the stage's gathered output is complete on this GPU.
 *
 * `windows`: HOST array of `world` (<= 8) device pointers, every rank's window as mapped on this
 * GPU (symmetric memory, IPC), windows[rank] the local one; all offsets below are bytes from a
 * window's base and identical on every rank.  Data of this exchange: 2 halves x world pieces of
 * `piece_bytes` at `data_offset`; the exchange with epoch e (1, 2, ... counted on the device in
 * state[0]) lands in half e & 1, rank r's piece at + r * piece_bytes, laid out exactly like the
 * jobs' output buffer.  `flags_offset`: u32[world]; `state_offset`: u32[2] {epoch, arrived};
 * `status_offset`: u32, nonzero once a wait ran out (1 | rank waited for << 8).  The host zeroes
 * flags, state and status once before first use; every exchange needs its own data, flags and
 * state; the status word may be shared. */
typedef struct dq_peer_push {
  void* const* windows;
  int32_t world, rank;
  int64_t data_offset;
  int64_t piece_bytes;
  int64_t flags_offset;
  int64_t state_offset;
  int64_t status_offset;
  int32_t spin_limit; /* polls per awaited rank; <= 0: a default of about a second */
  int32_t reserved;
} dq_peer_push;
/* `jobs`: 1..4 jobs of one stage -- the same x, m and dtypes, and the same out / out_stride
 * (distinct columns): that [m, out_stride] buffer is the piece (piece_bytes >= its size).  They
 * must leave as ONE launch of the tiled or the streaming tensor-core kernel; otherwise
 * DQ_ERR_UNSUPPORTED is returned and nothing was launched (the caller then uses
 * dq_gemv_sequence + dq_peer_all_gather).  Every rank must issue the same exchanges in the same
 * order.  Captures into CUDA graphs. */
DQ_API int32_t dq_gemv_stage_push(const dq_gemv_job* jobs, int32_t num_jobs, const dq_peer_push* push,
                                  void* stream);
/* Synchronises `stream` and reads the window's status word. */
DQ_API int32_t dq_peer_push_status(const dq_peer_push* push, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DYNQUANT_B200_H_ */
