/* C ABI of libvteb200.so: the CUDA bridge and the decode-attention entry points
 * that stand in for what VTE binds from amdhip64 (vte/bridge/hip_runtime.py:249-317,
 * `_map_hip_functions`) plus direct launchers for the split-KV attention path.
 *
 * Conventions
 *   - every function returns an int status: 0 = success, > 0 = the CUDA (or
 *     NCCL, for vteb_nccl_*) error code, < 0 = a shim-level rejection
 *     (VTEB_ERR_*).  vteb_last_error_string() describes the last failure on the
 *     calling thread.
 *   - pointers are plain addresses; nothing here knows about Python or torch.
 *   - one device per process: vteb_init(device) makes it current and creates
 *     nothing else; streams, events, modules and graphs are opaque void*.
 *   - not thread-safe beyond what the CUDA runtime itself guarantees, like the
 *     wrapper it replaces (single stream, one calling thread).
 */
#ifndef VTEB200_H
#define VTEB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VTEB_ERR_INVALID_ARGUMENT (-1)
#define VTEB_ERR_NOT_INITIALIZED (-2)
#define VTEB_ERR_UNSUPPORTED (-3)
#define VTEB_ERR_DRIVER_ENTRY (-4)   /* a driver entry point could not be resolved */
#define VTEB_ERR_NCCL_UNAVAILABLE (-5)
#define VTEB_ERR_DEVICE_STATUS (-6)  /* a kernel reported a timed-out wait */
#define VTEB_ERR_TOO_LARGE (-7)

/* Device attribute ids for vteb_device_attr(). */
#define VTEB_ATTR_SM_COUNT 0
#define VTEB_ATTR_MAX_THREADS_PER_BLOCK 1
#define VTEB_ATTR_MAX_SMEM_PER_BLOCK 2        /* without opt-in */
#define VTEB_ATTR_MAX_SMEM_PER_BLOCK_OPTIN 3
#define VTEB_ATTR_CC_MAJOR 4
#define VTEB_ATTR_CC_MINOR 5
#define VTEB_ATTR_L2_BYTES 6
#define VTEB_ATTR_CLOCK_KHZ 7

/* Launch flags for vteb_launch(). */
#define VTEB_LAUNCH_PROGRAMMATIC 1  /* programmatic dependent launch: the kernel may start
                                       before its predecessor in the stream has finished and
                                       orders itself with griddepcontrol.wait */

const char* vteb_last_error_string(void);
int vteb_version(void);

/* ---- device -------------------------------------------------------------
 * hipInit / hipGetDeviceCount / hipSetDevice (hip_runtime.py:436-504),
 * hipDeviceGetAttribute (:506-519), hipMemGetInfo (:565-584),
 * hipDeviceSynchronize (:909-929). */
int vteb_device_count(int* count);
int vteb_init(int device_index);
int vteb_current_device(int* device_index);
int vteb_device_attr(int device_index, int attr_id, int* value);
int vteb_device_name(int device_index, char* buf, int buf_len);
int vteb_mem_info(size_t* free_bytes, size_t* total_bytes);
int vteb_device_synchronize(void);

/* ---- memory -------------------------------------------------------------
 * hipMalloc / hipFree / hipMemcpy(kind 1, 2) / hipMemset
 * (hip_runtime.py:586-762).  The *_async forms and pinned host buffers have no
 * counterpart in the reference; the decode-step driver uses them for its
 * staging copies. */
int vteb_malloc(void** dev_ptr, size_t bytes);
int vteb_free(void* dev_ptr);
int vteb_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes);
int vteb_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes);
int vteb_memcpy_d2d(void* dst_dev, const void* src_dev, size_t bytes);
int vteb_memcpy_h2d_async(void* dst_dev, const void* src_host, size_t bytes, void* stream);
int vteb_memcpy_d2h_async(void* dst_host, const void* src_dev, size_t bytes, void* stream);
int vteb_memset(void* dst_dev, int value, size_t bytes);
int vteb_memset_async(void* dst_dev, int value, size_t bytes, void* stream);
int vteb_host_alloc(void** host_ptr, size_t bytes);
int vteb_host_free(void* host_ptr);

/* ---- modules and launches -----------------------------------------------
 * hipModuleLoad / hipModuleGetFunction (hip_runtime.py:793-803) and
 * hipModuleLaunchKernel (:805-907), same parameter order.  `params` is an
 * array of pointers to the argument values.  vteb_func_set_max_dynamic_smem
 * has no HIP analogue in the reference: CUDA needs the opt-in before a launch
 * may ask for more than 48 KB of dynamic shared memory. */
int vteb_module_load(void** module, const char* cubin_path);
int vteb_module_get_function(void** function, void* module, const char* name);
int vteb_module_unload(void* module);
int vteb_func_set_max_dynamic_smem(void* function, int bytes);
/* Preferred shared-memory carve-out of the function, percent of the maximum (CUDA only). */
int vteb_func_set_shared_carveout(void* function, int percent);
int vteb_launch(void* function, unsigned gx, unsigned gy, unsigned gz,
                unsigned bx, unsigned by, unsigned bz,
                unsigned shared_mem_bytes, void* stream, void** params, unsigned flags);

/* ---- streams, events, graphs --------------------------------------------
 * hipStreamCreate (hip_runtime.py:483), hipStreamBeginCapture mode 0 = global /
 * hipStreamEndCapture (:991-1001), hipGraphInstantiate / hipGraphLaunch /
 * hipGraphDestroy / hipGraphExecDestroy (:1003-1038), hipEvent* (:319-340). */
int vteb_stream_create(void** stream);
int vteb_stream_destroy(void* stream);
int vteb_stream_synchronize(void* stream);
int vteb_stream_begin_capture(void* stream, int mode);
int vteb_stream_end_capture(void* stream, void** graph);
int vteb_graph_instantiate(void** graph_exec, void* graph);
int vteb_graph_launch(void* graph_exec, void* stream);
int vteb_graph_destroy(void* graph);
int vteb_graph_exec_destroy(void* graph_exec);
int vteb_graph_node_count(void* graph, size_t* count);
int vteb_event_create(void** event);
int vteb_event_record(void* event, void* stream);
int vteb_event_synchronize(void* event);
int vteb_event_elapsed_ms(float* ms, void* start, void* stop);
int vteb_event_destroy(void* event);

/* ---- NCCL (no counterpart in the reference, which is single-GPU) ---------
 * The library is opened at first use (libnccl.so.2).  The unique id is 128
 * bytes; rank 0 creates it and hands it to the other ranks by any host
 * channel. */
int vteb_nccl_unique_id(void* id128);
int vteb_nccl_comm_init_rank(void** comm, int n_ranks, const void* id128, int rank);
int vteb_nccl_all_gather_f32(void* comm, const void* send, void* recv, size_t count_per_rank, void* stream);
int vteb_nccl_all_reduce_max_f32(void* comm, const void* send, void* recv, size_t count, void* stream);
int vteb_nccl_comm_destroy(void* comm);

/* ---- peer memory between the ranks of one node (no counterpart in the reference) ---
 * cudaIpcGetMemHandle / cudaIpcOpenMemHandle: a rank exports a whole cudaMalloc
 * allocation (64-byte handle, sent through the host rendezvous) and its peers map it;
 * kernels then store into it over NVLink.  Used by the KV-range sharded path to
 * exchange the (o, m, l) states without a collective library. */
int vteb_ipc_get_handle(void* dev_ptr, void* handle64);
int vteb_ipc_open_handle(const void* handle64, void** dev_ptr);
int vteb_ipc_close_handle(void* dev_ptr);

/* ---- split-KV decode attention, direct launchers -------------------------
 * These launch the same kernels the cubin exports, from inside the library.
 *
 * Geometry of the fast path for a head configuration
 * (replaces the grid/block/shared-memory arithmetic of
 * vte/core/split_kv_attention.py:178-217). */
typedef struct vteb_fast_plan {
    int ok;            /* 0: configuration not covered by the fast kernel */
    int hg;            /* KV heads staged together per work item */
    int n_hgroups;     /* head groups per sequence */
    int tile;          /* positions per pipeline stage */
    int nstages;
    int smem_bytes;    /* dynamic shared memory of the split kernel */
    int threads;       /* block size of the split kernel */
    int combine_dsplit;/* CTAs per (sequence, query head) of the combine kernel */
    int combine_smem_bytes; /* per split, up to 256 splits: min(max_chunks, 256) * this */
} vteb_fast_plan;
int vteb_split_kv_plan(int num_q_heads, int num_kv_heads, int head_dim, vteb_fast_plan* plan);
/* Same for the compact CTA shape (6 consumer warps + 2 loader warps of at most 160
 * registers, still one CTA per SM): it leaves register-file room beside it for the CTAs of
 * the combine launch, which shortens a layer whose whole split launch lasts only some
 * microseconds.  `ok` is 0 when a head group needs more than six consumer warps. */
int vteb_split_kv_plan_compact(int num_q_heads, int num_kv_heads, int head_dim, vteb_fast_plan* plan);
/* Encodes the 128-byte tensor map the fast split kernels take for a K or V cache: the cache
 * seen as `n_rows` position rows (all sequences, one after another) of `row_halves` =
 * Hkv * D fp16 values, in boxes of 64 values x `box_rows` rows (the plan's `tile`) with the
 * 128-byte swizzle.  `cache` must be 16-byte aligned, `row_halves` a multiple of 64.  The
 * kernels use it for whole tiles; ragged ends still travel as 16-byte copies.  No reference
 * counterpart: the reference's kernels read the cache with scalar loads
 * (flash_attention_split_kv_partial.hip.template:86-93). */
int vteb_kv_tensor_map(void* out_128_bytes, const void* cache, long long n_rows, int row_halves, int box_rows);
/* Columns per lane of the short-list combine kernel (split counts up to 64): a warp
 * merges 32 * epl columns of one (sequence, head) row. */
int vteb_combine_rows_epl(int rows, int head_dim);

/* One layer's decode attention for a batch: split kernel then combine.
 *   q [batch, Hq, D] fp16; k_cache, v_cache [batch, max_seq, Hkv, D] fp16 with
 *   sequence b at element offset b * kv_batch_stride; kv_offsets int32[batch]
 *   (device), sequence b attends to positions 0..kv_offsets[b];
 *   partial_m, partial_l fp32[batch*Hq*max_chunks], partial_o
 *   fp32[batch*Hq*max_chunks*D] scratch; work int32[4] scratch that must be
 *   zero before the first call (word 0: work-queue ticket, word 1: status);
 *   output [batch, Hq, D], fp32 when out_is_f32 else fp16.
 * Replaces the partial + reduce launches built by
 * SplitKVAttentionDispatcher.build_launches (vte/core/split_kv_attention.py:196-217)
 * and the kernels of flash_attention_split_kv_partial.hip.template:31-120 and
 * flash_attention_split_kv_reduce.hip.template:14-67.
 * flags: bit 0 = use the reference-geometry kernels instead of the fast path;
 *        bit 1 = zero partial_o of empty splits as the reference does;
 *        bit 2 = programmatic dependent launch. */
#define VTEB_ATTN_COMPAT 1
#define VTEB_ATTN_WRITE_EMPTY_O 2
#define VTEB_ATTN_PROGRAMMATIC 4
#define VTEB_ATTN_COMPACT 16   /* compact CTA shape where it applies, see vteb_split_kv_plan_compact */
#define VTEB_ATTN_NO_TENSOR_MAPS 32   /* fetch every tile with 16-byte asynchronous copies (no tensor-map copies) */
#define VTEB_ATTN_SHORT_SPLITS 128 /* hint: no split is longer than 16 positions (short contexts spread over many
                                      splits); the compact kernel for 128-wide heads then lets the warps of a KV head
                                      split the output columns instead of the blocks.  Correct at any length */
#define VTEB_ATTN_BALANCED 64   /* several sequences: every CTA takes an equal share of all cached positions; a
                                   (sequence, KV head group) is cut where shares end, into at most max_chunks
                                   splits (max_chunks >= 2; min_chunk is ignored); no work queue */
int vteb_split_kv_decode(const void* q, const void* k_cache, const void* v_cache,
                         const int* kv_offsets, void* output, int out_is_f32,
                         float* partial_m, float* partial_l, float* partial_o, int* work,
                         int batch, int num_q_heads, int num_kv_heads, int head_dim,
                         float scale, long long kv_batch_stride, int max_chunks,
                         int min_chunk, unsigned flags, int n_ctas, void* stream);

/* Same computation as vteb_split_kv_decode for callers that cannot allocate
 * device memory: code running inside a CUDA stream capture, a host callback or
 * a latency-critical serving loop where cudaMalloc (which may synchronise the
 * device and is forbidden during capture) is off the table, or a plugin host
 * that hands this library tensors but no allocator.  It has no counterpart in
 * the reference.  The split partials and the work-queue words live in a
 * file-scope device array inside the library (VTEB_NOALLOC_SCRATCH_BYTES, held
 * by every GPU that loads the library until the process exits); the caller
 * passes only inputs and the output.
 *   - Limit: batch * Hq * max_chunks * (D + 2) * 4 + 768 bytes must fit the
 *     array; larger requests return VTEB_ERR_TOO_LARGE and launch nothing.
 *   - The first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress) and raises the kernels' shared-memory limit; make
 *     that first call before any stream capture begins.
 *   - Every call uses the same array and finds the previous call's contents in
 *     it: the entry point clears the work-queue word, which must start at zero, and
 *     two calls that overlap on the GPU (different streams, no ordering) race.
 *   - The status word of the kernels' bounded waits lives in the array too and is
 *     left alone by later calls: read (and clear) it with vteb_noalloc_check_status
 *     after synchronising, as vteb_check_status does for caller-provided work words.
 *   - It calls no cudaMalloc, cudaFree or other allocating routine. */
#define VTEB_NOALLOC_SCRATCH_BYTES (16u << 20)
int vteb_split_kv_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                 const int* kv_offsets, void* output, int out_is_f32,
                                 int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                 float scale, long long kv_batch_stride, int max_chunks,
                                 int min_chunk, unsigned flags, int n_ctas, void* stream);

/* vteb_check_status for the work words inside the library's own array: returns
 * VTEB_ERR_DEVICE_STATUS (and clears the word) when a bounded wait of any
 * vteb_split_kv_decode_noalloc call since the last check gave up, 0 otherwise, also
 * when no such call has been made on this device yet.  Synchronises `stream`.  No
 * counterpart in the reference. */
int vteb_noalloc_check_status(void* stream);

/* Writes the current token's K/V rows at position kv_offsets[b]
 * (kv_cache_append.hip.template:13-39; launch built at split_kv_attention.py:186-194). */
int vteb_kv_cache_append(const void* k, const void* v, void* k_cache, void* v_cache,
                         const int* kv_offsets, int batch, int num_kv_heads, int head_dim,
                         long long kv_batch_stride, void* stream);

/* Reads the status word a split kernel leaves in work[1] and clears it.
 * Returns VTEB_ERR_DEVICE_STATUS when a bounded wait gave up. */
int vteb_check_status(int* work, void* stream);

/* Fills n fp16 values with N(0, sigma) from a counter-based generator; a
 * fraction outlier_prob of them is multiplied by outlier_scale.  Benchmark
 * input synthesis only; no counterpart in the reference. */
int vteb_fill_normal_f16(void* dst, size_t n, unsigned long long seed, float sigma,
                         float outlier_prob, float outlier_scale, void* stream);

/* Streams `bytes` of device memory through the SMs with 128-bit loads and
 * writes one checksum word per CTA: the read-bandwidth ceiling probe
 * (method of tools/bench_gemv_q4k_bandwidth.py:81-109). */
int vteb_read_bandwidth_probe(const void* src, size_t bytes, unsigned* sink, int n_ctas, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VTEB200_H */
