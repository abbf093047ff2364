/* lumen_b200 — C ABI of the B200 (sm_100a) execution backend for lumen's compiled graphs.
 *
 * These entry points are what lumen's CUDA device target binds for its compiled-graph hot path: the three launch
 * hooks the plan steps call (lumen/runtime/kernel/cuda/mod.rs:22-76: LAUNCH, GEMM, ATTENTION), plus the hooks the
 * reference's CUDA backend lacks and its Triton backend generates kernels for (reductions/rows, attention
 * backward, gather/scatter rows).
 *
 * Conventions
 *  - Every function returns 0 on success and a non-zero lb_status otherwise; lb_last_error() gives the message
 *    of the calling thread's last failure (the reference returns Result<_, String>).
 *  - Tensors are borrowed for the duration of the call. The library never frees caller memory and never
 *    synchronises the host: work is queued on the given stream (the reference launches on its one stream and
 *    never waits, lumen/runtime/README.md:32-34).
 *  - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *  - No CPU fallback: without a usable GPU every compute entry fails with LB_ERR_CUDA.
 */
#ifndef LUMEN_B200_H
#define LUMEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    LB_OK = 0,
    LB_ERR_INVALID = 1,     /* bad argument / type error, message names the primitive */
    LB_ERR_UNSUPPORTED = 2, /* a graph or layout this backend has no kernel for */
    LB_ERR_CUDA = 3,        /* CUDA driver/runtime/NVRTC failure */
    LB_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out (status word set by the kernel) */
} lb_status;

/* dtype codes; names as in lumen (lumen/tensor/dtype.rs) */
typedef enum {
    LB_BOOL = 0, LB_I8, LB_I16, LB_I32, LB_I64, LB_U8, LB_U16, LB_U32, LB_U64, LB_F16, LB_BF16, LB_F32, LB_F64,
} lb_dtype;

#define LB_MAX_RANK 8

/* Replaces the reference's Tensor view at the launch seam: storage pointer + dtype + shape + element strides
 * (lumen/graph_compiler/python.rs:1130-1157). `ptr` already includes the element offset. */
typedef struct {
    void* ptr;
    int32_t dtype; /* lb_dtype */
    int32_t rank;
    int64_t shape[LB_MAX_RANK];
    int64_t stride[LB_MAX_RANK]; /* in elements */
} lb_tensor;

const char* lb_last_error(void);
/* Library and toolchain description, a static string ("lumen_b200 <version> sm_100a ..."). */
const char* lb_version(void);

/* ---- fused elementwise / reduction / row kernels --------------------------------------------------------------
 * Replaces the LAUNCH hook `fn(name, source, tensors, outputs, n)` (lumen/runtime/kernel/cuda/mod.rs:22-38) and
 * the generator behind it (lumen/codegen/elementwise/cuda/mod.rs:54-333), extended to what the reference only has
 * on Triton: reductions with fused prologue/epilogue (lumen/codegen/reduction/triton.rs) and row kernels
 * (lumen/codegen/row/triton.rs).
 *
 * `body_text` is a fusion body in the graph text format (see lumen_b200/graph.py). The kernel is generated for
 * sm_100a, compiled once per distinct body and cached for the life of the process. */
typedef struct lb_fusion lb_fusion;

/* Compiles (or finds in the cache) the kernel for `body_text`. `*out` stays valid until process exit. */
int lb_fusion_compile(const char* body_text, lb_fusion** out);
/* Whether the generator has a kernel for `body_text` (LB_OK, or the status and message lb_fusion_compile would give)
 * without compiling it: what a fusion pass asks before it grows a group, as the reference's pass asks its
 * `can_fuse` rules (lumen/graph_compiler/passes/fusion). */
int lb_fusion_check(const char* body_text);
/* Number of body inputs / outputs, and the generated CUDA source (for inspection, like lumen's dump_code). */
int lb_fusion_num_inputs(const lb_fusion* f);
int lb_fusion_num_outputs(const lb_fusion* f);
const char* lb_fusion_source(const lb_fusion* f);
/* Bytes of scratch global memory one launch needs (0 for most bodies; column reductions use partial sums). */
size_t lb_fusion_scratch_bytes(const lb_fusion* f);
/* Launches on `stream`. `tensors` = inputs then outputs, each dense row-major of the body's declared type.
 * `scratch` must hold lb_fusion_scratch_bytes() bytes (NULL when that is 0). */
int lb_fusion_launch(const lb_fusion* f, const lb_tensor* tensors, int n_tensors, void* scratch, void* stream);
/* Horizontal launch (the reference's horizontal fusion of same-bodied kernels, lumen/graph_compiler/passes/
 * horizontal.rs:79): `f` was compiled from a module text that starts with the line `option multi` and whose body is
 * elementwise over rows of C elements (shape [2, C]; the row count is a placeholder). `tensors` holds n_groups x (inputs + outputs) dense tensors,
 * group after group; every tensor of a group has the same element count, a multiple of C. ONE launch applies the body
 * to every group (the pointer table travels as a kernel parameter; more than about a hundred groups take further
 * launches). The training step's per-parameter optimizer updates run this way, one launch per gradient bucket. */
int lb_fusion_launch_groups(const lb_fusion* f, const lb_tensor* tensors, int n_groups, void* stream);
/* One-shot form of the LAUNCH hook: compile-or-lookup + launch. Fails if the body needs scratch. */
int lb_launch_fused(const char* body_text, const lb_tensor* tensors, int n_inputs, int n_outputs, void* stream);


/* ---- GEMM ---------------------------------------------------------------------------------------------------
 * Replaces the GEMM hook `fn(a, b, output, config)` (lumen/runtime/kernel/cuda/mod.rs:41-68) and the Ampere
 * mma.sync kernel behind it (lumen/codegen/dot_general/cuda/ampere.py:35-904): `a` is a view [.., M, K], `b` a view
 * [.., K, N] (rank 2, or rank 3 with a leading batch), with ANY unit-stride major each - the reference hands over
 * transposed views the same way (lumen/codegen/dot_general/cuda/mod.rs:722-732). Accumulation is float32; the
 * product is written row-major as float32 or rounded once to the operands' dtype. bfloat16 and float16 operands run on
 * the tcgen05/TMEM/TMA kernels; float32 operands (and layouts TMA cannot address) run on a CUDA-core kernel that
 * accumulates in contracting order exactly like the reference interpreter (no hidden TF32 narrowing). */
/* Epilogues applied after the float32 accumulation, spelled as the primitives they stand for so that results equal
 * the unfused program's: RELU = max(acc, 0) before the output rounding; ADD = round(round(acc) + aux); MASK_POSITIVE
 * = aux > 0 ? round(acc) : 0 (the backward of a relu whose output is `aux`). ADD and MASK_POSITIVE take `aux`, a
 * row-major tensor of the output's shape and dtype (16-bit outputs, tensor-core kernels). They are the counterpart
 * of the reference's dot_general fusions with an elementwise tail (lumen/codegen/fusion/triton.rs:56-74). */
typedef enum { LB_EPILOGUE_NONE = 0, LB_EPILOGUE_RELU = 1, LB_EPILOGUE_ADD = 2, LB_EPILOGUE_MASK_POSITIVE = 3 } lb_epilogue;
typedef struct {
    lb_tensor product; /* [.., M, N], row-major */
    int32_t epilogue;  /* lb_epilogue */
    int32_t reserved;
    lb_tensor aux;     /* operand of LB_EPILOGUE_ADD / LB_EPILOGUE_MASK_POSITIVE; ignored otherwise */
} lb_gemm_out;
typedef struct {
    int32_t kernel; /* 0 = choose, 1 = require a tcgen05 kernel, 2 = force the CUDA-core kernel, 3 = require the
                     * one-CTA tcgen05 kernel (1 picks CTA pairs, tcgen05.mma.cta_group::2, when M > 128) */
    int32_t reserved;
    /* Optional scratch for split-K (the counterpart of the reference's split_k pass + `combine` kernel,
     * lumen/codegen/reduction/triton.rs): GEMMs with few output tiles and a long K (weight gradients) cut K into
     * ranges, write float32 partial tiles here and add them in a fixed order. NULL = never split. */
    void* scratch;
    size_t scratch_bytes;
    /* Tuned choices (0 = the library's own): the number of K ranges - honoured when `scratch` holds that many float32
     * partial tiles - and the rows of output tiles walked together before moving along N. The plan's autotuner
     * (lb_plan_autotune) sets them per step from measurements, as the reference's autotuner picks a kernel's config
     * (lumen/autotune/mod.rs:74-160). */
    int32_t splits;
    int32_t group_m;
} lb_gemm_cfg;
/* Scratch bytes that let lb_gemm split K for this problem (0 when it would not split). */
size_t lb_gemm_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t batch);
int lb_gemm(const lb_tensor* a, const lb_tensor* b, const lb_gemm_out* out, const lb_gemm_cfg* cfg /* nullable */,
            void* stream);

/* ---- flash attention ----------------------------------------------------------------------------------------
 * Replaces the ATTENTION hook `fn(&Forward{operands, dtype, heads_per_kv, causal, scores, grid, heads}, tensors,
 * &Config)` (lumen/codegen/attention/cuda/mod.rs:33-62) and the Ampere FA-2 forward kernel behind it
 * (lumen/codegen/attention/cuda/ampere/forward.py:810-1157). Operands are strided [B, S, N, H] views read in place
 * (the reference records them as strided accesses, lumen/graph_compiler/passes/attention/forward.rs:598-772);
 * key/value heads serve N / Nkv query heads each. Scores, softmax and both products accumulate in float32; the
 * probabilities are rounded to bfloat16 before the value product, as the traced program does
 * (lumen/functional/attention/flash.py:38-45). `lse` (nullable) receives each row's float32 log-sum-exp,
 * dense [B, N, Sq]. */
typedef struct {
    float scale;           /* multiplies the scores before the softmax; must be positive */
    int32_t causal;        /* non-zero: key j is visible to query i iff j <= i + causal_offset */
    int64_t causal_offset; /* Sk - Sq for flash-attn's bottom-right alignment */
} lb_attn_desc;
int lb_attention_fwd(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                     const lb_tensor* o, const lb_tensor* lse /* nullable */, void* stream);
/* Backward of lb_attention_fwd, FlashAttention-2's as the reference traces it
 * (lumen/functional/attention/flash.py:51-85): probabilities recomputed from `lse`; `delta` [B, N, Sq] float32 is
 * caller-provided scratch that receives rowsum(dO * O); dq, dk, dv are bfloat16 views shaped like q, k, v. The
 * reference's CUDA backend never launches its backward kernel (lumen/codegen/attention/README.md:27-28); its
 * Triton backend's deterministic pair (dkdv_kernel, dq_kernel; lumen/codegen/attention/triton/kernel.py:108-264)
 * is the design followed: no atomics, bit-identical from run to run. */
int lb_attention_bwd(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                     const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* delta,
                     const lb_tensor* dq, const lb_tensor* dk, const lb_tensor* dv, void* stream);
/* lb_attention_bwd in the mode the reference's backend runs unless its `deterministic` option is set: ONE kernel
 * that computes dK and dV per key block and adds each key block's dS K into a float32 dQ atomically, in no fixed
 * order (lumen/codegen/attention/triton/mod.rs:176-180,458-466; kernel.py:108-200 with ADD_DQ). `dq_accum` is
 * caller-provided scratch, dense float32 [B, Sq, N, H]; the call zeroes it, accumulates into it and rounds it to `dq`.
 * Five tensor-core products and one set of exponentials per (key tile, query tile) instead of the deterministic
 * pair's seven and two. The single-kernel form covers bfloat16 operands of head dim 64; everything else runs as
 * lb_attention_bwd does (dq_accum unused). dK and dV are bit-identical from run to run; dQ is not. */
int lb_attention_bwd_atomic(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                            const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* delta,
                            const lb_tensor* dq_accum, const lb_tensor* dq, const lb_tensor* dk, const lb_tensor* dv,
                            void* stream);
/* lb_attention_bwd for callers that cannot allocate device memory at call time (code inside a fixed memory pool,
 * inside a region where the allocator is locked, or on a latency budget that rules allocation out). It has no
 * counterpart in the reference. The per-row scratch `delta` lives in a 4 MiB array built into the library (every
 * GPU that loads the library holds it until exit), so the call takes no scratch argument and performs no
 * cudaMalloc/cudaFree. Limits: batch * heads * query length <= 1,048,576 (larger problems are rejected with a
 * message), bfloat16 operands, head dim 64 or 128. All calls share the array: calls whose kernels may overlap on the
 * GPU race on it. The first call on a device looks up the array's device address; make it before any stream
 * capture begins. */
int lb_attention_bwd_static(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                            const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* dq,
                            const lb_tensor* dk, const lb_tensor* dv, void* stream);

/* ---- scatter-add of rows ----------------------------------------------------------------------------------------
 * `out[clamp(ids[t]), :] = x[..] + sum of updates[t, :]`: the `scatter_add` primitive along axis 0 of a [rows, width]
 * operand (lumen/reference/mod.rs:765-808), the gradient of an embedding lookup. float32 or bfloat16 rows, int32 or
 * int64 indices clamped into range. `x` NULL = an operand of zeros. The two forms of the reference's backends
 * (lumen/codegen/scatter_add/README.md:23-39): `deterministic` non-zero sorts the updates by destination row
 * (count, starts, place, sort) and adds each row's updates in update order, rounding to the operand's dtype after every
 * add as the interpreter does - bit-identical to it and from run to run; zero adds with float32 atomics in arrival
 * order and rounds once (the last bits vary when a row is hit more than once). */
size_t lb_scatter_add_scratch_bytes(int64_t rows, int64_t width, int64_t updates, int deterministic);
int lb_scatter_add_rows(const lb_tensor* x /* nullable */, const lb_tensor* ids, const lb_tensor* updates, const lb_tensor* out,
                        void* scratch, size_t scratch_bytes, int deterministic, void* stream);

/* ---- plan ---------------------------------------------------------------------------------------------------
 * Replaces `trait Plan { steps(); run_in(workspace, inputs) }` with `workspace_bytes()/workspace_alignment()`
 * (lumen/plan/mod.rs:102-127,255-262) and its step loop (lumen/plan/run.rs:356-427): an ordered list of prepared
 * steps (generated fused kernels, GEMMs, attention forward/backward, row scatter-adds, copies) over the caller's
 * inputs, outputs and one 256-byte aligned workspace. The plan text is produced by the host-side compiler
 * (lumen_b200/compiler.py); fusion bodies in it are compiled when the plan is created. Running a plan queues its
 * launches on `stream` and returns: no allocation, no synchronisation. `first_step`/`last_step` (last < 0 = all)
 * run a sub-range, which is how collectives issued by the host are placed between steps
 * (lumen/plan/step/triton.rs:122-177). Outputs stay valid until the next run (lumen/plan/README.md:47-48). */
typedef struct lb_plan lb_plan;
int lb_plan_create(const char* plan_text, lb_plan** out);
/* The device target's lowering, `Cuda::lower(module, device) -> Result<Box<dyn Plan>, String>`
 * (lumen/graph_compiler/device.rs:88-112, lumen/codegen/devices/cuda/mod.rs:140-189): `module_text` is a module AFTER
 * the pass pipeline in the graph text format (fusion bodies first, the main graph last); every `fusion` node of the
 * main graph becomes a step (a generated kernel, a GEMM for `dot_general` fusions with no tail or a relu, the attention
 * kernels for `flash_attention` / `flash_attention_backward`), `reshape` / `transpose` / `slice` views (copied where a
 * kernel needs them dense or aligned), concatenations copies into place, constants fills or kernels without operands;
 * every value gets a place and the plan its workspace size. A node there is no kernel for is rejected with a message
 * naming the primitive. This is the same lowering the Python side has (live-range placement, donation, the gradient
 * arena with its buckets and `all_reduce` / `wait` steps, horizontally fused updates); the Python one emits plan text
 * for lb_plan_create.
 * `config` may be NULL (defaults); `device` < 0 keeps the current device. */
typedef struct {
    int32_t deterministic;  /* non-zero (the default): attention backward as the bit-reproducible kernel pair */
    int32_t n_donate;       /* pairs in `donate` */
    const int32_t* donate;  /* (output index, input index) pairs: the output is written into that input's memory, which
                               the caller gives up (the updated weights of a training step over the weights; the
                               reference's donated buffers, lumen/plan/compile.rs:17-46). The caller passes the same
                               pointer for both, or any pointer for the output: it is not written. */
    int64_t bucket_bytes;   /* all-reduced gradients are reduced in buckets of at least this many bytes; 0 = 64 MiB */
    int32_t reserved[2];    /* zero */
} lb_config;
int lb_compile(const char* module_text, int device, const lb_config* config, lb_plan** out);
void lb_plan_destroy(lb_plan* plan);
size_t lb_plan_workspace_bytes(const lb_plan* plan);
size_t lb_plan_workspace_alignment(const lb_plan* plan);
int lb_plan_num_steps(const lb_plan* plan);
/* Kernels of this library that one run of the plan launches (a column reduction and a split-K product count two,
 * attention backward three, a copy of a permuted or sliced view one; block copies, fills and collectives none). */
int lb_plan_kernel_launches(const lb_plan* plan);
/* JSON list of {kind, label} per step, like Plan.steps() (lumen/graph_compiler/python.rs:163-191). */
const char* lb_plan_steps_json(const lb_plan* plan);
/* The plan text the plan was made from (what lb_compile emitted, or lb_plan_create's argument): modules, tensors and
 * steps, for dumps and debugging. Owned by the plan. */
const char* lb_plan_text(const lb_plan* plan);
int lb_plan_run(const lb_plan* plan, void* workspace, void* const* inputs, int n_inputs, void* const* outputs,
                int n_outputs, int first_step, int last_step, void* stream);

/* Binds the communicator that the plan's `all_reduce` steps use (NULL unbinds). A collective is a plan step like any
 * other (lumen/plan/step/triton.rs:122-177): `all_reduce` queues NCCL's all-reduce of a gradient bucket on the plan's
 * side stream once the steps before it have finished, `wait` makes the compute stream wait for that collective's event
 * (lumen/distributed/nccl.rs:279-307,532-565). The host never blocks. lb_plan_num_collectives counts them. */
typedef struct lb_comm lb_comm;
int lb_plan_set_comm(lb_plan* plan, lb_comm* comm);
int lb_plan_num_collectives(const lb_plan* plan);

/* Times the candidate configurations of every tensor-core GEMM step of at least 2^30 multiply-adds on the plan's own
 * buffers and keeps the fastest for later runs (lumen/autotune/mod.rs:74-160, lumen/codegen/dot_general/cuda/mod.rs:603:
 * the same threshold): candidates are the K-split counts the step's scratch can hold around the cost model's choice,
 * the tile raster's group size, and CTA pairs against single CTAs. Before timing, the workspace is filled with noise
 * in [-1, 1) (clocks under zeros differ, lumen/plan/step/cuda.rs:90-128) and the device runs for 0.2 s to reach its
 * sustained clocks; each candidate gets 5 untimed and 10 timed runs. Steps with equal shapes, majors, dtypes and
 * epilogues share a result, within the process and across plans. Call it before the first real run: it overwrites the
 * workspace and the plan's outputs (never its inputs). `report` (nullable) receives a JSON list of
 * {label, m, n, k, candidates, picked: {kernel, splits, group_m}, us, default_us}. Synchronises the stream. */
int lb_plan_autotune(lb_plan* plan, void* workspace, void* const* inputs, int n_inputs, void* const* outputs, int n_outputs,
                     void* stream, char* report, size_t report_bytes);

/* A step range of a plan recorded once as a CUDA graph over fixed workspace/input/output pointers, then replayed
 * with one launch per call: the replay removes the per-launch host cost and the gaps between dependent launches of
 * the step loop (lumen/plan/run.rs:356-427 dispatches step by step; the reference has no recorded form). Recording
 * runs nothing on the device and happens on a private stream; run the range once with lb_plan_run beforehand so that
 * one-time set-up (kernel attributes, module loads) is not part of the recording. The pointers given at capture are
 * the ones every replay uses. lb_graph_launch queues the replay on `stream`. */
typedef struct lb_graph lb_graph;
int lb_plan_capture(const lb_plan* plan, void* workspace, void* const* inputs, int n_inputs, void* const* outputs,
                    int n_outputs, int first_step, int last_step, lb_graph** out);
int lb_graph_launch(const lb_graph* graph, void* stream);
void lb_graph_destroy(lb_graph* graph);

/* ---- device memory, streams, events -----------------------------------------------------------------------------
 * The backend's own runtime layer, so that a host binding this library needs no other CUDA framework: the region
 * allocator (lumen/allocator/region.rs:13-121, lumen/allocator/cuda.rs:59-121) - ONE cudaMalloc per region on first
 * use, then first-fit blocks at 256-byte (or larger power-of-two) alignment, coalesced when freed; running out is an
 * error with the free-space summary, not an abort - and thin owners of streams, events and pinned host memory
 * (lumen/runtime/stream/cuda.rs:119-290). While a recorded graph launches into a region's blocks, put the region on
 * hold: blocks freed meanwhile return only at release (cuda.rs:123-170). */
typedef struct lb_region lb_region;
int lb_set_device(int device);     /* makes `device` current; fails unless it is an sm_100 part */
int lb_device_count(void);
int lb_device_synchronize(void);
int lb_device_memory(size_t* free_bytes, size_t* total_bytes);
int lb_region_create(size_t capacity_bytes, lb_region** out); /* reserves nothing yet; the current device is the region's */
void lb_region_destroy(lb_region* region);
int lb_region_alloc(lb_region* region, size_t bytes, size_t alignment /* 0 = 256 */, void** out);
int lb_region_free(lb_region* region, void* ptr);
int lb_region_hold(lb_region* region);
int lb_region_release(lb_region* region);
int lb_region_stats(lb_region* region, size_t* capacity, size_t* live_bytes, size_t* peak_bytes, size_t* largest_free);
int lb_stream_create(void** out); /* a non-blocking stream */
int lb_stream_destroy(void* stream);
int lb_stream_synchronize(void* stream);
int lb_stream_wait_event(void* stream, void* event);
int lb_event_create(int timing, void** out);
int lb_event_destroy(void* event);
int lb_event_record(void* event, void* stream);
int lb_event_synchronize(void* event);
int lb_event_elapsed_ms(void* start, void* stop, float* ms);
int lb_host_alloc(size_t bytes, void** out); /* page-locked host memory */
int lb_host_free(void* ptr);
int lb_copy_to_device(void* dst, const void* src, size_t bytes, void* stream);
int lb_copy_to_host(void* dst, const void* src, size_t bytes, void* stream);
int lb_copy_on_device(void* dst, const void* src, size_t bytes, void* stream);
int lb_fill_bytes(void* dst, int byte, size_t bytes, void* stream);

/* ---- rendezvous store and communicator --------------------------------------------------------------------------
 * The keyed TCP store of lumen/distributed/store.rs:43-72,100-230 (the master rank's process serves it, every rank is
 * a client): set, get (waits for the key), add (integer counter), wait (for several keys), delete. EVERY wait has a
 * deadline in milliseconds (0 = the store's default) and returns LB_ERR_TIMEOUT when it passes - a peer that never
 * arrives cannot hang the others. `port` 0 lets the master pick one (lb_store_port tells which). */
typedef struct lb_store lb_store;
int lb_store_create(const char* host, int port, int is_master, int timeout_ms, lb_store** out);
void lb_store_destroy(lb_store* store);
int lb_store_port(const lb_store* store);
int lb_store_set(lb_store* store, const char* key, const void* value, size_t n);
int lb_store_get(lb_store* store, const char* key, void* out, size_t capacity, size_t* n, int timeout_ms);
int lb_store_add(lb_store* store, const char* key, int64_t amount, int64_t* result /* nullable */);
int lb_store_wait(lb_store* store, const char* const* keys, int n_keys, int timeout_ms);
int lb_store_delete(lb_store* store, const char* key);
/* The NCCL communicator of a group of `world` ranks on the current device (lumen/distributed/nccl.rs:103-213):
 * libnccl.so.2 is loaded at the first call, rank 0 publishes ncclGetUniqueId through the store, every rank passes a
 * store barrier with a deadline and then calls ncclCommInitRank. The store must outlive the communicator.
 * lb_comm_all_reduce queues ncclAllReduce on `stream` (op: 0 sum, 1 prod, 2 max, 3 min; nccl.rs:387-410).
 * lb_comm_barrier is a host barrier through the store. lb_comm_check reports NCCL's asynchronous error state without
 * blocking. lb_comm_synchronize waits for `stream` for at most `timeout_ms` while polling that state; on an error or at
 * the deadline it ABORTS the communicator and returns LB_ERR_CUDA / LB_ERR_TIMEOUT, so the host never waits on a dead
 * peer forever. */
int lb_comm_create(lb_store* store, int rank, int world, int timeout_ms, lb_comm** out);
void lb_comm_destroy(lb_comm* comm);
int lb_comm_rank(const lb_comm* comm);
int lb_comm_size(const lb_comm* comm);
int lb_comm_all_reduce(lb_comm* comm, const void* send, void* recv, size_t count, int dtype /* lb_dtype */, int op, void* stream);
int lb_comm_broadcast(lb_comm* comm, void* buffer, size_t count, int dtype, int root, void* stream);
int lb_comm_barrier(lb_comm* comm, int timeout_ms);
int lb_comm_check(lb_comm* comm);
int lb_comm_synchronize(lb_comm* comm, void* stream, int timeout_ms);
int lb_comm_abort(lb_comm* comm);
const char* lb_nccl_version(void); /* "2.27.3"; "" when NCCL cannot be loaded */

/* Synchronises the current device, then reads and clears its status words - the library's own and the one
 * lb_attention_bwd_static uses: 0, or LB_ERR_TIMEOUT when a kernel's bounded wait gave up and the kernel wound itself
 * down (its outputs are then undefined). Allocates nothing. The reference has no counterpart (its kernels never
 * wait). */
int lb_device_status(void);
/* Diagnostic, no counterpart in the reference: launches one CTA that waits on a barrier nobody arrives on, for at most
 * `cycles` SM cycles (1 .. 100,000,000), then gives up the way every kernel here does - it raises the status word
 * and returns normally; nothing faults, traps or hangs. `static_word` non-zero raises lb_attention_bwd_static's word
 * instead of the library's. lb_device_status() then returns LB_ERR_TIMEOUT once. */
int lb_debug_wait_timeout(long long cycles, int static_word, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUMEN_B200_H */
