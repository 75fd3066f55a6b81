/* aicf_b200.h - C ABI of the B200 (sm_100a) backend.
 *
 * Plain C: pointers, sizes and integers only. Every function returns an aicf status code
 * (0 Ok, 1 InvalidArgument, 2 NotImplemented, 3 Internal) unless stated otherwise, never throws,
 * and - apart from the helpers in the "device memory" and "plan" sections - neither allocates nor
 * synchronises: a launch only enqueues work on the given stream.
 *
 * Each entry point names the interface of the reference project (jeehun98/ai-compiler-framework,
 * paths relative to its ai-compiler-framework/ directory) that it stands in for.
 */
#ifndef AICF_B200_H_
#define AICF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AICF_B200_ABI_VERSION 1

/* ---- handle types ---------------------------------------------------------------------------
 * Bit-compatible with aicf::cuda::TensorDesc (include/aicf/backends/cuda/registry/tensor_desc.hpp:88-104,
 * sizeof 96) and aicf::cuda::AttrBlob (attr_blob.hpp:13-17, sizeof 16). */
enum { AICF_DTYPE_UNKNOWN = 0, AICF_DTYPE_F32 = 1, AICF_DTYPE_F16 = 2, AICF_DTYPE_BF16 = 3, AICF_DTYPE_I32 = 4 };
enum { AICF_OK = 0, AICF_INVALID_ARGUMENT = 1, AICF_NOT_IMPLEMENTED = 2, AICF_INTERNAL = 3 };

typedef struct aicf_tensor_desc {
  void* data;        /* device pointer, borrowed */
  uint8_t dtype;     /* AICF_DTYPE_* */
  int32_t rank;      /* 0 = scalar, at most 4 */
  int64_t shape[4];  /* elements */
  int64_t stride[4]; /* elements */
  uint8_t contiguous;
  int32_t alignment; /* bytes, 0 = unknown */
  int32_t device;
} aicf_tensor_desc;

typedef struct aicf_attr_blob {
  uint32_t schema_id; /* 0 = op defaults */
  uint32_t bytes;
  const void* data; /* little-endian POD payload */
} aicf_attr_blob;

/* A CUDA stream handle (cudaStream_t) passed as an integer; 0 = the legacy default stream.
 * Reference: the uint64 stream argument of _C.op_call / _C.launch_by_id
 * (src/python_bindings/bindings.cpp:272,295-297). */
typedef uint64_t aicf_stream;

/* ---- library ------------------------------------------------------------------------------- */
int aicf_b200_abi_version(void);
/* Name of a status code. Reference: status_to_string (registry/status.hpp:15-23). */
const char* aicf_b200_status_string(int status);
/* Text of the most recent failure on the calling thread ("" if none). */
const char* aicf_b200_last_error(void);
/* Lower-case op name of an OpKind value, "unknown" if out of range.
 * Reference: opkind_to_name (src/python_bindings/bindings.cpp:196-219). */
const char* aicf_b200_op_name(int op_kind);

/* ---- dispatch ------------------------------------------------------------------------------
 * Replaces aicf::cuda::dispatch_v0 (include/aicf/backends/cuda/registry/dispatch.hpp:12-17;
 * src/backends/cuda/registry/registry.cpp:144-215): first supported variant in priority order. */
int aicf_b200_op_call(int op_kind, const aicf_tensor_desc* inputs, int num_inputs, aicf_tensor_desc* outputs,
                      int num_outputs, const aicf_attr_blob* attr /* may be NULL */, aicf_stream stream);

/* Replaces aicf::cuda::dispatch_by_id_v0 (dispatch.hpp:19-26; registry.cpp:16-64): the variant
 * pinned by its kernel id. Unknown id -> NotImplemented; contract mismatch -> InvalidArgument. */
int aicf_b200_launch_by_id(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                           aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr,
                           aicf_stream stream);

/* The three function pointers of a KernelVariant (kernel_variant.hpp:44-61), addressed by id.
 * launch_ws passes caller-owned scratch straight to KernelVariant::launch. */
int aicf_b200_supported(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                        const aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr); /* 1/0 */
size_t aicf_b200_query_workspace(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                                 const aicf_attr_blob* attr);
int aicf_b200_launch_ws(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                        aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr, void* workspace,
                        size_t workspace_bytes, aicf_stream stream);

/* Scratch arena used by op_call / launch_by_id for variants that need workspace (the reference refuses
 * such variants, registry.cpp:52-56). NULL restores the library-owned arena, which is allocated on
 * first need and never while the target stream is capturing. */
int aicf_b200_set_workspace(void* ptr, size_t bytes);

/* Registry introspection. Reference: KernelRegistry::variants_snapshot / find_by_id
 * (registry.hpp:38-41); ids are those of register_all.cpp:105-291 plus this backend's additions. */
int aicf_b200_kernel_count(int op_kind);
const char* aicf_b200_kernel_id(int op_kind, int index); /* priority order; NULL past the end */
int aicf_b200_num_op_kinds(void);

/* Status word of the tcgen05 GEMM's bounded waits: 0 = no wait ever expired. Synchronises the
 * device. No counterpart in the reference (its kernels have no device-side waits). */
int aicf_b200_gemm_status(int clear);
/* All device-side bounded waits of this library in one word: low 16 bits = the GEMM code above, bit 16 =
 * a row copy of the softmax / softmax-CE prefetch pipeline did not arrive within its budget, bits 17-18 = a
 * cross-GPU wait of dp_adam_step expired (1 waiting for gradients, 2 waiting for completion). 0 = healthy.
 * Synchronises the device. No counterpart in the reference. */
int aicf_b200_wait_status(int clear);
/* Tuning aid of the tcgen05 GEMM: reads the 16-slot timeline that CTA 0 of the last GEMM wrote (globaltimer ns:
 * start, set-up, first TMA, first stage landed, first tile issued, first accumulator ready, first / last tile stored,
 * end, then wait and busy totals per role and the tile count), then switches recording on or off. out16 may be NULL.
 * Synchronises the device. No counterpart in the reference. */
int aicf_b200_gemm_timeline(int enable, uint64_t* out16);
/* The tcgen05 GEMM reads its tuning overrides (environment variables AICF_GEMM_CTA_GROUP, _TILE_N, _SPLITK, _GROUP_M,
 * _C_STREAM, _AB_HINT, _TAIL_HALVES) at the first GEMM of the process, not on every launch. This reads them again: for a
 * test or a tuning sweep that changes a setting inside one process. No counterpart in the reference. */
int aicf_b200_gemm_reload_tuning(void);

/* Column sum [rows, cols] -> [cols] (fp32, row-major, contiguous) for callers that must not allocate
 * device memory: a host that was given a fixed memory budget up front, or code that runs where the
 * CUDA allocator is off limits - for example a KernelVariant::launch body, which by contract may only
 * enqueue work and which the reference's dispatcher always hands a null workspace. No counterpart in
 * the reference.
 * Same kernels and summation order as reduce_sum_keep_lastdim_f32_v0, but the partial sums go to a
 * 512 KiB array built into the library's device image instead of a caller- or library-allocated
 * workspace; cudaMalloc / cudaFree are never called. Shapes whose partial sums need more than
 * AICF_B200_NOALLOC_SCRATCH_BYTES return InvalidArgument (the message names the need).
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before starting any stream capture. All calls on a device share the one array and
 * it keeps whatever the last call left in it (each call rewrites every partial it later reads, so
 * nothing has to be cleared); two calls that overlap on the GPU - different streams without an
 * ordering between them - race on it. */
#define AICF_B200_NOALLOC_SCRATCH_BYTES (512u * 1024u)
int aicf_b200_colsum_f32_noalloc(const float* x, float* out, int64_t rows, int64_t cols, aicf_stream stream);

/* ---- op trace ------------------------------------------------------------------------------
 * Replaces trace_enable / trace_reset / trace_get of the reference binding
 * (src/python_bindings/bindings.cpp:193-231,459-472). Entries are "<opname>" for op_call and
 * "kid:<id> kind:<opname>" for launch_by_id. Enabled by default; kept in a bounded ring (the newest
 * AICF_B200_TRACE_CAPACITY entries). Only the *_traced launch functions record. */
#define AICF_B200_TRACE_CAPACITY 65536
void aicf_b200_trace_enable(int flag);
void aicf_b200_trace_reset(void);
int aicf_b200_trace_count(void);
const char* aicf_b200_trace_get(int index); /* valid until the next trace call on any thread */
int aicf_b200_op_call_traced(int op_kind, const aicf_tensor_desc* inputs, int num_inputs, aicf_tensor_desc* outputs,
                             int num_outputs, const aicf_attr_blob* attr, aicf_stream stream);
int aicf_b200_launch_by_id_traced(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                                  aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr,
                                  aicf_stream stream);

/* ---- process-global CUDA graph ---------------------------------------------------------------
 * Replaces graph_begin / graph_end / graph_launch / graph_reset / graph_stream
 * (src/python_bindings/bindings.cpp:137-187,475-547): one graph at a time, captured on and launched
 * into a dedicated non-blocking stream. graph_begin stores the capture stream in *stream_out. */
int aicf_b200_graph_begin(aicf_stream* stream_out);
int aicf_b200_graph_end(void);    /* InvalidArgument + "graph_end called but not capturing" */
int aicf_b200_graph_launch(void); /* InvalidArgument + "graph_launch called but no captured graph exists" */
int aicf_b200_graph_reset(void);
aicf_stream aicf_b200_graph_stream(void); /* 0 before the first graph_begin */

/* ---- device memory / streams / events (host plumbing for callers without a tensor library) -----
 * The reference borrows all of this from torch (torch.empty, Tensor.copy_, torch.cuda.synchronize);
 * these are thin wrappers over the CUDA runtime. */
int aicf_b200_device_count(void);
int aicf_b200_set_device(int device);
/* Facts about a device that sizing decisions and benchmark reports need: L2 cache bytes, SM count, total global
 * memory bytes (any pointer may be NULL). What a torch user reads from torch.cuda.get_device_properties. */
int aicf_b200_device_info(int device, int64_t* l2_bytes, int* sm_count, int64_t* total_bytes);
/* PCI address of a device as "dddd:bb:dd.f" (NUL-terminated; capacity >= 13). A one-process-per-GPU job uses it to
 * find the host NUMA node the device hangs off (sysfs numa_node of that address) and to keep its pinned staging
 * buffers and copy-issuing threads there. No counterpart in the reference (single device, torch owns host memory). */
int aicf_b200_device_pci_bus_id(int device, char* out, int capacity);
/* Measuring aid: a minimal streaming kernel that reads `reads` (1-4) arrays and writes `writes` (1-3) arrays of
 * bytes_each bytes (16-byte aligned, multiple of 16) with 16-byte evict-first accesses - the bandwidth ceiling of this
 * device for a kernel with that mix of input and output streams (fused Adam: 4 + 3), which a plain copy's rate
 * overstates. packets_in_flight (1, 2 or 4; 0 = 2) is the number of 16-byte packets per array each thread has in
 * flight, blocks_per_sm (1-1024; 0 = 8) the number of 256-thread blocks per SM: the ceiling is the best rate over
 * those choices. No counterpart in the reference. */
int aicf_b200_stream_probe(int reads, int writes, const void* const* inputs, void* const* outputs, size_t bytes_each,
                           int packets_in_flight, int blocks_per_sm, aicf_stream stream);
int aicf_b200_malloc(void** ptr, size_t bytes);
int aicf_b200_free(void* ptr);
int aicf_b200_host_alloc_pinned(void** ptr, size_t bytes);
/* Pinned host memory for buffers the host only WRITES and the device reads (the staging buffer of a step's input batch):
 * write-combined, so device reads of it are not snooped through the CPU caches; host reads of it are very slow. Freed
 * with aicf_b200_host_free_pinned. What a torch user gets nowhere (torch pins cacheable memory only). */
int aicf_b200_host_alloc_staging(void** ptr, size_t bytes);
int aicf_b200_host_free_pinned(void* ptr);
int aicf_b200_memcpy_h2d(void* dst, const void* src, size_t bytes, aicf_stream stream); /* async on `stream` */
int aicf_b200_memcpy_d2h(void* dst, const void* src, size_t bytes, aicf_stream stream);
int aicf_b200_memcpy_d2d(void* dst, const void* src, size_t bytes, aicf_stream stream);
int aicf_b200_memset(void* dst, int value, size_t bytes, aicf_stream stream);
int aicf_b200_stream_create(aicf_stream* out);
int aicf_b200_stream_destroy(aicf_stream s);
int aicf_b200_stream_sync(aicf_stream s);
int aicf_b200_device_sync(void);
int aicf_b200_event_create(uint64_t* out);
int aicf_b200_event_destroy(uint64_t ev);
int aicf_b200_event_record(uint64_t ev, aicf_stream s);
int aicf_b200_event_sync(uint64_t ev);
int aicf_b200_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms);
int aicf_b200_stream_wait_event(aicf_stream s, uint64_t ev);

/* ---- captured execution plan ------------------------------------------------------------------
 * C++ replacement of the reference's Python executor: build_binding_plan / allocate_static_env
 * (python/aicf_fw/core_v2/plan.py:90-137,174-209) and PlannedExecutor.run / capture / replay /
 * reset_graph (python/aicf_fw/core_v2/exec.py:337-497). A plan is built from the lowered-op list
 * (op name, input/output value ids, attr payload, optional kernel id; lower.py:9-21):
 *   values with role INPUT or PARAM live in caller- or plan-owned pointer-stable buffers,
 *   STATIC values are carved from one arena with liveness-based reuse,
 *   kernel variants, attr payloads and workspace slices are resolved once at finalize().
 * run() enqueues every op; capture() records them into a CUDA graph; replay(n) launches the graph
 * n times with no host work in between. */
typedef struct aicf_plan aicf_plan;
enum { AICF_ROLE_INPUT = 0, AICF_ROLE_PARAM = 1, AICF_ROLE_STATIC = 2 };

aicf_plan* aicf_b200_plan_create(const char* name);
void aicf_b200_plan_destroy(aicf_plan* plan);
/* Declares value `vid`. persistent != 0 keeps a STATIC value out of arena reuse (optimizer state,
 * anything read after the step). zero_init != 0 clears it at finalize (opt.step / opt.m / opt.v,
 * plan.py:160-171). */
int aicf_b200_plan_add_value(aicf_plan* plan, int vid, const char* name, int dtype, int rank, const int64_t* shape,
                             int role, int persistent, int zero_init);
/* Appends a lowered op. kernel_id NULL -> the variant is chosen by priority at finalize. */
int aicf_b200_plan_add_op(aicf_plan* plan, const char* op_name, const char* kernel_id, const int* inputs,
                          int num_inputs, const int* outputs, int num_outputs, uint32_t schema_id,
                          const void* attr_bytes, uint32_t attr_len);
/* Makes `vid` an alias of `target_vid` (same buffer). Used to drop copy_saved ops. */
int aicf_b200_plan_alias(aicf_plan* plan, int vid, int target_vid);
/* Binds a value to caller-owned device memory (must outlive the plan and stay at that address). */
int aicf_b200_plan_bind(aicf_plan* plan, int vid, void* device_ptr);
/* Data-parallel exchange over peer memory (dp_adam_step ops; no counterpart in the reference). Values marked
 * peer-visible before finalize (gradients, broadcast working copies, biases) are placed in one pool allocation
 * per plan. After finalize every rank exports its pool as a 64-byte IPC handle (all zero when the plan has no
 * pool), the handles are exchanged by the caller, and open_peers maps the other ranks' pools
 * (handles = world x 64 bytes in rank order; the own entry is ignored). One process per GPU.
 * Attrs of a dp_adam_step op: schema 'DPAD' (0x44415044), payload <fffffIi> lr, beta1, beta2, eps, weight_decay,
 * decoupled, slot (index of the op's flag block, unique per op of a plan, < 60), optionally followed by <ii>
 * flags, fence_slots. flags bit 0 (defer_done): the op does not wait for the other ranks' "my stores into your memory
 * are done" words; the plan must then end the step with a dp_adam_step op carrying fence_slots = n, which waits for
 * those words of slots [0, n) before it completes. flags bit 1 (solo): no other kernel runs beside this op, so it
 * may take two CTAs per SM instead of leaving room for a co-resident GEMM. Without the two optional fields every op
 * waits for itself and leaves that room.
 * After a non-zero aicf_b200_wait_status (bits 17-18) the replicas are no longer known to agree: restore the model
 * and optimizer state from a checkpoint before training on. */
int aicf_b200_plan_set_peer_visible(aicf_plan* plan, int vid);
int aicf_b200_plan_peer_handle(aicf_plan* plan, void* handle64, size_t* pool_bytes);
int aicf_b200_plan_open_peers(aicf_plan* plan, int rank, int world, const void* handles);
/* Same, for callers that already hold device addresses of the other ranks' pools (one process driving several
 * GPUs with peer access enabled, or a test that stands a silent buffer in for a rank that never arrives).
 * bases[k] = address of rank k's pool as seen from this device; bases[rank] is ignored. */
int aicf_b200_plan_open_peers_raw(aicf_plan* plan, int rank, int world, void* const* bases);
size_t aicf_b200_plan_peer_pool_bytes(aicf_plan* plan);
/* Address, as seen from this device, of rank `rank`'s pool once the peers are open (the own rank: the plan's own
 * pool; before open_peers only rank 0 = the own pool answers). NULL otherwise. The first 8 KiB of a pool are the
 * exchange's control block. For tools that measure the peer links with the plan's own mappings. */
void* aicf_b200_plan_peer_pool_base(aicf_plan* plan, int rank);
/* Allocates the arena and every unbound value, resolves variants. No ops may be added afterwards. */
int aicf_b200_plan_finalize(aicf_plan* plan);
void* aicf_b200_plan_value_ptr(aicf_plan* plan, int vid);
size_t aicf_b200_plan_value_bytes(aicf_plan* plan, int vid);
/* Byte offset of a value inside the plan's shared arena, or -1 when the value has a buffer of its own (inputs,
 * parameters, persistent and bound values, values in the peer pool) or is unknown. Values whose live ranges do not
 * overlap may report overlapping ranges: that is the reuse. For dumps of the memory layout. */
int64_t aicf_b200_plan_value_arena_offset(aicf_plan* plan, int vid);
size_t aicf_b200_plan_arena_bytes(aicf_plan* plan);        /* bytes actually allocated for STATIC values */
size_t aicf_b200_plan_arena_bytes_no_reuse(aicf_plan* plan); /* what one buffer per value would need */
int aicf_b200_plan_num_ops(aicf_plan* plan);
const char* aicf_b200_plan_op_kernel_id(aicf_plan* plan, int op_index);
int aicf_b200_plan_run(aicf_plan* plan, aicf_stream stream); /* eager: one launch per op */
int aicf_b200_plan_capture(aicf_plan* plan);                 /* graph on the plan's own stream */
int aicf_b200_plan_replay(aicf_plan* plan, int n);           /* n graph launches, no sync */
/* Same, launched into `stream` instead of the plan's own stream (plans that share parameter buffers are
 * serialised by replaying them into one stream). */
int aicf_b200_plan_replay_on(aicf_plan* plan, int n, aicf_stream stream);
int aicf_b200_plan_reset_graph(aicf_plan* plan);
aicf_stream aicf_b200_plan_stream(aicf_plan* plan);
int aicf_b200_plan_sync(aicf_plan* plan);
int aicf_b200_plan_graph_nodes(aicf_plan* plan); /* all nodes of the captured graph, -1 if none */
int aicf_b200_plan_graph_kernel_nodes(aicf_plan* plan); /* kernel nodes only: launches per replay */
/* Eager step with a CUDA event pair around every op on the plan's stream (all_reduce ops stay on that
 * stream too); after a synchronise, ms_per_op[i] is the device time of op i. For measurement only. */
int aicf_b200_plan_profile(aicf_plan* plan, float* ms_per_op, int capacity);

/* ---- data-parallel gradient exchange -------------------------------------------------------------
 * No counterpart in the reference (single device, bindings.cpp:123). One process per GPU; rank 0
 * creates a 128-byte id, every rank calls dp_init with it. all_reduce ops (OpKind 22) then sum fp32
 * buffers in place over the ranks with NCCL on the launch stream. */
int aicf_b200_dp_unique_id(void* id128);
int aicf_b200_dp_init(int rank, int world_size, const void* id128);
int aicf_b200_dp_finalize(void);
int aicf_b200_dp_world_size(void); /* 1 when not initialised */
int aicf_b200_dp_rank(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* AICF_B200_H_ */
