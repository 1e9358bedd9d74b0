/*
 * kvmig — C ABI of the paged-KV block migration / swap library for B200.
 *
 * Every entry point takes plain pointers, integers and an opaque stream, and
 * returns 0 on success or a negative KVMIG_E* code; the text of the last
 * failure on the calling thread is available from kvmig_last_error().  Nothing
 * is launched when validation fails.  There is no CPU fallback: without a CUDA
 * device every compute entry point returns KVMIG_ECUDA.
 *
 * The functions replace the four native operators that DistServe resolves from
 * SwiftTransformer's libst_pybinding.so (distserve/__init__.py:4-16).  The
 * operator shim in libst_pybinding.so (same directory as this library) binds
 * them under the operator names the reference calls.
 *
 * Pool layout, both stages, K and V separately (distserve/worker.py:107-121):
 *   [num_blocks, layers_local, kv_heads_local, block_size, head_dim], contiguous.
 * Parallel-config vectors use ParallelConfig.to_list() order
 *   [tp_size, tp_rank, pp_size, pp_rank]            (distserve/config.py:57-63).
 */
#ifndef KVMIG_H_
#define KVMIG_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVMIG_ABI_VERSION 2   /* 2: handles carry a per-process number; kvmig_handle_is_local */

#if defined(__GNUC__)
#define KVMIG_API __attribute__((visibility("default")))
#else
#define KVMIG_API
#endif

/* Number of int64 words in an exported pool handle (a plain int list, so it
 * survives pickling between worker processes; distserve/utils.py:73). */
#define KVMIG_HANDLE_WORDS 24

enum {
    KVMIG_OK = 0,
    KVMIG_EINVAL = -1,     /* bad argument: shape, length, id out of range, duplicate target, bad handle words */
    KVMIG_ENOTREG = -2,    /* a context worker needed for this copy was never registered */
    KVMIG_ECUDA = -3,      /* a CUDA runtime call failed (text in kvmig_last_error) */
    KVMIG_EDEVICE = -4,    /* the copy kernel reported a device-side problem (bounded wait ran out) */
    KVMIG_ELIMIT = -5      /* a fixed capacity was exceeded */
};

/* Shape of one pool as the worker allocated it (distserve/worker.py:109-121). */
typedef struct kvmig_pool_shape {
    int64_t num_blocks;
    int64_t num_layers;   /* layers held by this worker   = L / pp_size */
    int64_t num_heads;    /* KV heads held by this worker = H / tp_size */
    int64_t block_size;   /* token slots per block */
    int64_t head_dim;
    int64_t elem_size;    /* bytes per value: 2 for fp16/bf16, 4 for fp32 */
} kvmig_pool_shape;

KVMIG_API int kvmig_abi_version(void);

/* Text of the most recent failure on this thread ("" if none). */
KVMIG_API const char* kvmig_last_error(void);

/*
 * Export a pool so that another worker process on the same node can map it.
 * Replaces torch.ops.block_migration_ops.get_ipc_mem_handle(Tensor) -> int[]
 * (distserve/worker.py:133-134).  `pool` is the device address of element 0;
 * `handle_out` receives KVMIG_HANDLE_WORDS words: the CUDA IPC handle of the
 * enclosing allocation, the pool's byte offset inside it, its shape, and the
 * exporter's pid together with a number the exporting process drew at random
 * when it started (a handle registered by the process that exported it is
 * resolved without CUDA IPC, which cannot open its own handles; the pid alone
 * would not identify that process, because workers in different pid
 * namespaces can carry the same pid).
 */
KVMIG_API int kvmig_get_ipc_mem_handle(const void* pool, const kvmig_pool_shape* shape, int64_t* handle_out);

/*
 * 1 if `handle` was exported by the calling process (pid and per-process
 * number both match), 0 if it came from another process, a negative KVMIG_E*
 * code if the words are not a valid handle.  Needs no device.  (No
 * counterpart in the reference; it tells a host which of the two mapping
 * routes registration will take.)
 */
KVMIG_API int kvmig_handle_is_local(const int64_t* handle, int64_t handle_len);

/*
 * Make one context-stage worker's K and V pools addressable from the calling
 * (decoding-stage) worker.  Replaces
 * torch.ops.block_migration_ops.register_ipc_mem_handle(k_handle, v_handle,
 *   num_layers, num_heads, context_parallel_config, decoding_parallel_config)
 * (distserve/worker.py:239-246).  num_layers / num_heads are the model's
 * global counts; ctx_parallel_config names the exporting worker and
 * dec_parallel_config the caller, both in to_list() order.  Handles of
 * context workers whose layer/head rectangle does not meet the caller's are
 * recorded but not mapped.  Registering the same context rank again replaces
 * the earlier entry.  Mappings live until the process exits: the reference has
 * no unregister call site.
 */
KVMIG_API int kvmig_register_ipc_mem_handle(const int64_t* k_handle, int64_t k_handle_len,
                                  const int64_t* v_handle, int64_t v_handle_len,
                                  int64_t num_layers, int64_t num_heads,
                                  const int64_t* ctx_parallel_config,
                                  const int64_t* dec_parallel_config);

/*
 * Pull blocks from the registered context workers into this worker's pools:
 * for X in {K,V}, every i, every global layer l and KV head h this worker
 * holds,
 *   X_dec[dec_blocks[i], l - l0_dec, h - h0_dec, :, :] =
 *   X_ctx(owner of l,h)[ctx_blocks[i], l - l0_ctx, h - h0_ctx, :, :].
 * Replaces torch.ops.block_migration_ops.migrate_blocks(ctx_pp, ctx_tp,
 *   ctx_blocks, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks,
 *   k_cache, v_cache)                              (distserve/worker.py:256-267;
 * note the pp-then-tp argument order).  The copy kernel is launched on
 * `stream` (a cudaStream_t, NULL = the legacy default stream) and the call
 * returns only after the kernel has finished, because the caller frees the
 * source blocks as soon as it returns
 * (distserve/single_stage_engine.py:524-536).
 */
KVMIG_API int kvmig_migrate_blocks(int64_t ctx_pp_size, int64_t ctx_tp_size,
                         const int64_t* ctx_blocks, int64_t num_ctx_blocks,
                         int64_t dec_pp_size, int64_t dec_tp_size,
                         int64_t dec_pp_rank, int64_t dec_tp_rank,
                         const int64_t* dec_blocks, int64_t num_dec_blocks,
                         void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
                         void* stream);

/*
 * Same copy, not awaited: the kernel is enqueued on `stream` and `*ticket`
 * identifies it.  kvmig_migrate_wait(ticket) blocks until that kernel has
 * finished and returns its status; source blocks must not be reused before.
 * Lets a caller enqueue a request's migration beside an in-flight decode step
 * (the call cadence of distserve/decoding_stage_scheduler.py:247-260 is one
 * awaited request at a time).  At most KVMIG_MAX_INFLIGHT tickets may be
 * outstanding per device; older ones are awaited implicitly.
 *
 * Ordering.  Migrations enqueued on one stream complete in the order they were
 * enqueued, and whatever the caller enqueues on that stream afterwards runs
 * after all of them.  A migration may *begin* before earlier ones have
 * finished, but only when it is independent of every one of them that is still
 * executing: it reads no pool that one of them writes, writes no pool that one
 * of them reads, and where both write the same pools it writes other blocks
 * (or, for kvmig_migrate_layers_async, other layers of the same blocks).  A
 * migration that conflicts with one still executing on ANOTHER stream is
 * ordered after it through that migration's event.  Work of other libraries is
 * ordered by its own completion: a kernel that the caller puts on the stream
 * between two migrations runs after the first has finished, and the second
 * begins after that kernel has finished.  Ordering against work on other
 * streams that is not a migration of this library is the caller's business,
 * as with any stream.
 */
#define KVMIG_MAX_INFLIGHT 8
KVMIG_API int kvmig_migrate_blocks_async(int64_t ctx_pp_size, int64_t ctx_tp_size,
                               const int64_t* ctx_blocks, int64_t num_ctx_blocks,
                               int64_t dec_pp_size, int64_t dec_tp_size,
                               int64_t dec_pp_rank, int64_t dec_tp_rank,
                               const int64_t* dec_blocks, int64_t num_dec_blocks,
                               void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
                               void* stream, uint64_t* ticket);
KVMIG_API int kvmig_migrate_wait(uint64_t ticket);

/*
 * kvmig_migrate_blocks_async restricted to the global layers
 * [layer_begin, layer_end): only the part of this worker's rectangle inside
 * the window is copied (nothing, and no launch, if the window misses the
 * worker's layers).  The reference migrates a request only after its whole
 * prefill has finished (distserve/single_stage_engine.py:393-401); with this
 * call a context stage that signals per-layer completion can have the
 * decoding stage pull each group of layers while prefill is still computing
 * the next ones.  Launches whose windows are disjoint may overlap on the GPU
 * even when they write the same blocks.
 */
KVMIG_API int kvmig_migrate_layers_async(int64_t ctx_pp_size, int64_t ctx_tp_size,
                               const int64_t* ctx_blocks, int64_t num_ctx_blocks,
                               int64_t dec_pp_size, int64_t dec_tp_size,
                               int64_t dec_pp_rank, int64_t dec_tp_rank,
                               const int64_t* dec_blocks, int64_t num_dec_blocks,
                               void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
                               int64_t layer_begin, int64_t layer_end,
                               void* stream, uint64_t* ticket);

/*
 * kvmig_migrate_blocks for hosts that must not allocate.  (No counterpart in
 * the reference: its worker has the one migrate operator.)
 *
 * The ordinary entry point keeps its block tables and status word in memory
 * it obtains from cudaMalloc / cudaHostAlloc on first use.  A decoding worker
 * that has sized its KV pools to take the HBM that was free at start-up
 * (distserve/worker.py:152-192) cannot count on a later allocation
 * succeeding, and an allocation in the middle of a decode loop can stall the
 * device; other embedders simply forbid allocation after start-up.  This
 * variant performs the same copy with the same kernels, arguments and
 * completion rule (it returns when the source blocks have been read), but its
 * scratch is a fixed array compiled into the library (33 KiB of device memory
 * on every GPU that loads it, held until the process exits), and it calls no
 * cudaMalloc, cudaFree, cudaHostAlloc, event creation or other routine that
 * allocates device or pinned memory.  (Ordinary host-heap use remains: the
 * planning step builds a few small vectors per call.)  Every call ends by
 * waiting for its stream.
 *
 * Limits and rules:
 *  - at most KVMIG_STATIC_MAX_BLOCKS block indexes per call; more is refused
 *    with KVMIG_ELIMIT (split the lists, or use kvmig_migrate_blocks);
 *  - at most 8 context workers may contribute to the calling worker's
 *    rectangle (one launch carries 16 strided-copy descriptors, two per
 *    contributing worker); a reshard that needs more is refused with
 *    KVMIG_ELIMIT;
 *  - every context worker it reads must already have been mapped by
 *    kvmig_register_ipc_mem_handle for this decoding rank (mapping a peer pool
 *    is registration's job; this call refuses instead of mapping);
 *  - the first call on each device looks up the array's device address
 *    (with that device current); make that first call before any stream
 *    capture begins;
 *  - all calls on a device share the one array, which keeps the previous
 *    call's contents; each call rewrites every word it will read before it
 *    launches.  Two calls whose kernels overlapped on the GPU would race on
 *    the tables; the entry point therefore serialises its callers and returns
 *    only after its kernel has finished, so calls made through it never
 *    overlap.  Do not copy the pattern into an asynchronous wrapper.
 */
#define KVMIG_STATIC_MAX_BLOCKS 4096
KVMIG_API int kvmig_migrate_blocks_static(int64_t ctx_pp_size, int64_t ctx_tp_size,
                                const int64_t* ctx_blocks, int64_t num_ctx_blocks,
                                int64_t dec_pp_size, int64_t dec_tp_size,
                                int64_t dec_pp_rank, int64_t dec_tp_rank,
                                const int64_t* dec_blocks, int64_t num_dec_blocks,
                                void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
                                void* stream);

/*
 * Copy whole blocks between the GPU pools and the pinned host pools, in list
 * order, on `stream`, without waiting for completion.  Replaces
 * torch.ops.swapping_ops.swap(source_block_ids, target_block_ids, is_swap_in,
 *   k_cache, v_cache, k_swap, v_swap)              (distserve/worker.py:303-311).
 * is_swap_in != 0: host block source[i] -> GPU block target[i]; else GPU block
 * source[i] -> host block target[i].  `shape` describes the GPU pools; the
 * host pools have the same per-block shape and num_cpu_blocks blocks
 * (distserve/worker.py:122-130).
 *
 * The reference worker records the event it later waits on BEFORE it calls
 * this operator (distserve/worker.py:286-287 vs 302-311), so with the
 * unmodified worker neither wait_for_all_swap_in/out nor the per-request wait
 * in step() covers the copies; a deployment on that worker relies on a stream
 * or device synchronize, or sets the option "swap_wait" (environment variable
 * KVMIG_SWAP_WAIT=1 for hosts that cannot call kvmig_set_option), which makes
 * this call return only after its copies have finished.  Off by default: the
 * copies then overlap whatever the caller does next, which is the point of
 * running them on a side stream.
 */
KVMIG_API int kvmig_swap(const int64_t* source_block_ids, int64_t num_source,
               const int64_t* target_block_ids, int64_t num_target,
               int is_swap_in,
               void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
               void* k_swap, void* v_swap, int64_t num_cpu_blocks,
               void* stream);

/*
 * Tuning and introspection (no counterpart in the reference).
 *   options : "kernel" 0 auto | 1 vector loads | 2 bulk-copy pipeline,
 *             "chunk_bytes" size of one work unit = one shared-memory stage
 *             (default 16384), "stages" ring depth per CTA (default 0 =
 *             automatic: 3, and 4 for calls of more than 256 blocks; a
 *             positive value applies to every call),
 *             "ctas_per_sm" (default 0 = as many as keep 96 KiB in flight per
 *             SM: 2 with the defaults),
 *             "inline_tables" 1 = lists of up to 1024 blocks travel in the
 *             kernel parameters instead of a device table (default 1),
 *             "overlap_launches" 1 = a migration whose target blocks are
 *             disjoint from those of the migrations still in flight may start
 *             before they finish (default 1),
 *             "max_ctas" N > 0 = launch at most N CTAs, so that a migration
 *             running beside a decode step leaves the other SMs to it
 *             (default 0 = no cap),
 *             "dynamic_units" 1 = CTAs draw work units from a device counter
 *             instead of a fixed round-robin share (default 1), "unit_batch"
 *             units drawn per visit (default 0 = 2 for long launches, else 1),
 *             "l2_hint" bit 0 / bit 1 = evict-first L2 policy on the bulk
 *             loads / stores (default 0),
 *             "wait_limit_ms" longest the copy kernel waits for one of its
 *             loads before it records the failure and returns, making the
 *             call fail with KVMIG_EDEVICE (default 2000),
 *             "lose_unit_plus1" N > 0 = failure-path exercise: work unit N-1
 *             arms its completion barrier but never issues its load, so that
 *             wait runs out (default 0),
 *             "wait_mode" 1 = kvmig_migrate_wait / kvmig_migrate_blocks poll the
 *             kernel's event from the calling thread instead of calling
 *             cudaEventSynchronize (default 0),
 *             "swap_wait" 1 = kvmig_swap returns only after its copies have
 *             finished (default 0, or the value of KVMIG_SWAP_WAIT in the
 *             environment when the option was never set)
 *   counters: "kernel_launches", "memcpy_calls", "bytes_migrated",
 *             "bytes_swapped", "mapped_peers", "migrate_calls",
 *             "plan_cache_hits" (calls that reused the previous call's
 *             planning), and the host time of the migration entry points by
 *             segment, in nanoseconds summed over calls: "ns_prepare"
 *             (arguments to launch descriptors), "ns_validate" (block ids),
 *             "ns_order" (may the launch overlap its predecessors?),
 *             "ns_launch" (parameters, launch, event), "ns_wait" (waiting for
 *             the kernel in kvmig_migrate_wait / kvmig_migrate_blocks)
 */
KVMIG_API int kvmig_set_option(const char* name, int64_t value);
KVMIG_API int64_t kvmig_get_option(const char* name);
KVMIG_API int64_t kvmig_get_counter(const char* name);

/* Forget every registered context worker of the current device (test use;
 * mapped peer allocations stay mapped and are reused on re-registration). */
KVMIG_API int kvmig_reset_registry(void);

#ifdef __cplusplus
}
#endif
#endif /* KVMIG_H_ */
