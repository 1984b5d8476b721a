/* b200.h — C ABI of the Blackwell (sm_100a) execution backend for arrayjit routines.
 *
 * This is the surface an OCaml `Lowered_backend` implementation binds through ctypes/C
 * stubs.  Each entry point names the reference interface member it serves (paths are
 * relative to the reference project).  Conventions:
 *   - every function returns 0 on success; a negative value is one of B200_E_*, a
 *     positive value is the CUresult / nvrtcResult / ncclResult_t that failed;
 *   - b200_last_error() returns a thread-local message for the last failure on the
 *     calling thread;
 *   - all device work is asynchronous on the device's single stream, like the cuda
 *     backend's (arrayjit/lib/cuda_backend.ml:215-238); host buffers passed to the copy
 *     functions must stay valid until the next b200_await / b200_event_sync;
 *   - there is no CPU fallback: with no usable driver or GPU every compute entry point
 *     fails with B200_E_NO_DEVICE.
 */
#ifndef B200_H
#define B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_E_INVALID (-1)     /* bad argument (Invalid_argument on the OCaml side) */
#define B200_E_NO_DEVICE (-2)   /* driver, NVRTC or GPU unavailable */
#define B200_E_PARSE (-3)       /* malformed b200ir */
#define B200_E_UNSUPPORTED (-4) /* valid IR that this backend cannot run */
#define B200_E_USER (-5)        /* Utils.User_error: bad static index, missing binding, ... */
#define B200_E_DEVICE (-6)      /* a kernel reported a device-side status (bounded wait expired) */
#define B200_E_NO_SPACE (-7)    /* a fixed-capacity entry point was given a larger problem */

typedef struct b200_dev b200_dev;
typedef struct b200_event b200_event;
typedef struct b200_code b200_code;
typedef struct b200_routine b200_routine;
typedef struct b200_comm b200_comm;

const char* b200_last_error(void);
const char* b200_version(void);

/* ---- devices: Backend_device_common.{num_devices, get_device, get_name, static_properties}
 *      (arrayjit/lib/backend_intf.ml:218-266; cuda: arrayjit/lib/cuda_backend.ml:215-238) */
int b200_init(void);
int b200_num_devices(int* out);
int b200_device_open(int ordinal, b200_dev** out);     /* memoised per ordinal */
int b200_device_props(b200_dev* dev, char* json, size_t cap);

/* ---- pools: Slab_alloc.{alloc_pool, free_pool, memset_zero}
 *      (arrayjit/lib/backend_intf.ml:22-37; cuda: arrayjit/lib/cuda_backend.ml:60-94).
 *      Allocating an id that exists frees the old slab first. */
int b200_pool_alloc(b200_dev* dev, int pool_id, size_t bytes, size_t alignment);
int b200_pool_free(b200_dev* dev, int pool_id);
int b200_pool_memset0(b200_dev* dev, int pool_id, size_t offset, size_t bytes);
int b200_pool_address(b200_dev* dev, int pool_id, uint64_t* device_ptr, size_t* bytes);

/* ---- copies: No_buffer_retrieval_or_syncing.{from_host, to_host, device_to_device}
 *      (arrayjit/lib/backend_impl.ml:292-315; cuda: arrayjit/lib/cuda_backend.ml:262-314) */
int b200_h2d(b200_dev* dev, int pool_id, size_t offset, const void* src, size_t bytes);
int b200_d2h(b200_dev* dev, int pool_id, size_t offset, void* dst, size_t bytes);
int b200_d2d(b200_dev* dst_dev, int dst_pool, size_t dst_offset, b200_dev* src_dev, int src_pool,
             size_t src_offset, size_t bytes);
/* `~into_merge_buffer:Copy`: grows the destination's merge slab (reserved pool id 0,
 * arrayjit/lib/backend_intf.ml:131-132) and copies the source node into it. */
int b200_merge_copy(b200_dev* dst_dev, b200_dev* src_dev, int src_pool, size_t src_offset, size_t bytes);
/* page-locked host staging memory for from_host / to_host */
int b200_host_alloc(size_t bytes, void** out);
int b200_host_free(void* p);

/* ---- events and stream: Device.{all_work, is_done, sync, will_wait_for, await, is_idle}
 *      (arrayjit/lib/backend_intf.ml:97-126; cuda: arrayjit/lib/cuda_backend.ml:107-111,256-260) */
int b200_event_record(b200_dev* dev, b200_event** out);
int b200_event_query(b200_event* ev, int* done);
int b200_event_sync(b200_event* ev);
int b200_event_elapsed_ms(b200_event* start, b200_event* stop, float* ms);
int b200_event_free(b200_event* ev);
int b200_stream_wait(b200_dev* dev, b200_event* ev);
int b200_await(b200_dev* dev);
int b200_is_idle(b200_dev* dev, int* idle);
int b200_stream_handle(b200_dev* dev, uint64_t* custream);
/* Extension (the reference has one stream per device, arrayjit/lib/cuda_backend.ml:215-238): with
 * `on`, b200_h2d copies run on a second stream.  A copy waits for everything queued before it.
 * Work queued after it waits for the copy when it may touch the copied pool: b200_launch waits for
 * the copies into the pools its routine binds (and pool 0), b200_d2h / b200_pool_memset0 for the
 * copies into their pool, every other call for all copies.  Uploading the next batch into a second
 * pool before launching the current step therefore overlaps the two. */
int b200_set_async_uploads(b200_dev* dev, int on);

/* ---- routines: Lowered_backend.{compile, link} (arrayjit/lib/backend_impl.ml:334-367;
 *      cuda: arrayjit/lib/cuda_backend.ml:898-928 compile, :983-1066 link and launch).
 *      b200_compile is device independent.  `options` is a space-separated list of
 *      key=value pairs (gemm, attn, coop, fuse, pairs, splitk, tf32, large_models, bounds; each 0|1); NULL for defaults.
 *      gemm: tensor-core contractions; attn: the attention chain (scores, softmax, weights . values,
 *      lib/nn_blocks.ml:222-236) as one kernel; coop: cooperative reductions; fuse: several stages per
 *      launch; pairs: two neighbouring elements per thread with packed 16-bit arithmetic; splitk:
 *      few-tile fp32 accumulations split over K (atomic adds, order not fixed); tf32: contractions of
 *      single-precision operands on the tensor cores as tf32 (10-bit mantissas, fp32 sums; with
 *      tf32=0 they stay on the exact generic kernels); bounds: a range-checked build of the generated
 *      kernels (generic kernels only): an access outside a node is skipped and the next wait returns
 *      B200_E_DEVICE naming the node id and the element. */
int b200_compile(const char* name, const char* b200ir, size_t len, const char* options, b200_code** out);
int b200_code_info(b200_code* code, char* json, size_t cap);
int b200_code_source(b200_code* code, int stage, char* buf, size_t cap, size_t* needed);
int b200_code_free(b200_code* code);

typedef struct {
  int32_t tn_id;   /* tensor node id of the routine */
  int32_t pool_id; /* Backend_intf.buffer_loc: pool + byte offset */
  uint64_t offset;
} b200_binding;

/* Bindings need only be aligned to the node's element size, which is all the reference's
 * allocator promises (plan_pool_segments, arrayjit/lib/backends.ml:22-51; an offset that is not a
 * multiple of the element size is B200_E_INVALID).  Stages whose compiled form wants more (8-byte
 * pairs, 16-byte TMA operand bases) are re-planned for the addresses at hand; b200_routine_info
 * reports the plan that runs. */
int b200_link(b200_dev* dev, b200_code* code, const b200_binding* bindings, int n_bindings,
              b200_routine** out);
int b200_routine_info(b200_routine* r, char* json, size_t cap);   /* like b200_code_info, for the linked plan */
/* Runs the routine once on the device stream.  static_idx has one value per static symbol
 * of the routine, in declaration order; a negative or out-of-range value is B200_E_USER
 * (cuda: arrayjit/lib/cuda_backend.ml:1015-1030). */
int b200_launch(b200_routine* r, const int64_t* static_idx, int n_static);
int b200_routine_use_graph(b200_routine* r, int enable);
int b200_routine_launch_count(b200_routine* r, int64_t* kernels_per_run);
/* Per-stage device timing (CUDA events around every stage of the next runs; disables graph
 * replay while on).  No counterpart in the reference, which has no profiler hooks. */
int b200_routine_profile(b200_routine* r, int enable);
int b200_routine_stage_time(b200_routine* r, int stage, float* total_ms, int* runs);
int b200_routine_free(b200_routine* r);

/* ---- observability: get_used_memory, get_debug_info (arrayjit/lib/cuda_backend.ml:123-126,1114-1118) */
int b200_used_memory(b200_dev* dev, size_t* bytes);
int b200_debug_info(b200_dev* dev, char* json, size_t cap);

/* ---- data parallel exchange.  Replaces the owner-reduce + broadcast of
 *      Parallel.data_parallel's grad_sync (lib/parallel.ml:247-304) by one NCCL allreduce
 *      per contiguous gradient range.  One communicator rank per process and device. */
int b200_comm_unique_id(char* id128);                                      /* 128 bytes */
int b200_comm_init_rank(b200_dev* dev, int n_ranks, int rank, const char* id128, b200_comm** out);
/* One process that holds every shard, as the reference's data_parallel does
 * (lib/parallel.ml:166-208): all communicators at once, and one range per device reduced as one
 * NCCL group (a thread that drives several devices must group its calls). */
int b200_comm_init_all(int n_devices, b200_dev* const* devs, b200_comm** out);
int b200_allreduce_all(int n, b200_comm* const* comms, const int* pool_ids, const size_t* offsets, size_t count,
                       int dtype, int op);
#define B200_SUM 0
#define B200_AVG 1
#define B200_F32 0
#define B200_BF16 1
int b200_allreduce(b200_comm* comm, int pool_id, size_t offset, size_t count, int dtype, int op);
/* Overlap of the exchange with the backward pass.  The ranges (at most a few buckets, e.g. the
 * gradients of the last layers and those of the first) are reduced on the communicator's own
 * stream, each as soon as the routine's last stage that writes into it has been queued, while the
 * remaining stages run; the compute stream waits for all of them at the end of the routine, so the
 * optimizer step that follows sees reduced gradients.  Replaces the gradient-by-gradient
 * owner-reduce that follows the whole backward pass in lib/parallel.ml:292-304.  n = 0 detaches. */
int b200_routine_overlap_allreduce(b200_routine* r, b200_comm* comm, int n, const int* pool_ids,
                                   const size_t* offsets, const size_t* counts, int dtype, int op);
/* With a timeout (> 0 ms) b200_await polls instead of blocking: an asynchronous NCCL error
 * (ncclCommGetAsyncError), or a stream still busy after the timeout (a rank that never arrived),
 * aborts the communicator (ncclCommAbort) and is returned as an error; the device stays usable,
 * the communicator does not.  No counterpart in the reference, whose shards share one process. */
int b200_comm_set_timeout(b200_comm* comm, long long timeout_ms);
int b200_comm_free(b200_comm* comm);

/* ---- allocation-free reduction.  No counterpart in the reference: added for callers that may
 *      not reach the device allocator while they run (inside a stream capture, in a serving
 *      loop that cannot afford cudaMalloc's implicit synchronisation, or under a memory budget
 *      that was handed out up front).  Writes sum(in[0..count)) as one float at the output
 *      location, in stream order on the device's stream, with its scratch in a 4 KiB array that
 *      is part of the library's device image.  count <= 2^26, else B200_E_NO_SPACE; count 0
 *      writes 0.0f.  Both offsets must be multiples of 4, else B200_E_INVALID (checked on the
 *      host: nothing is launched).  A positive return value here is a cudaError_t.  The first
 *      call on a device resolves the array's address: make it before any stream capture.
 *      Calls that overlap on the GPU race on the shared array; stream-ordered calls do not. */
int b200_sum_f32_static(b200_dev* dev, int in_pool, size_t in_offset, size_t count, int out_pool,
                        size_t out_offset);

#ifdef __cplusplus
}
#endif
#endif /* B200_H */
