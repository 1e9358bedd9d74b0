// Paged-KV block migration and swap for B200 (sm_100a): copy kernels, the
// per-process registry of mapped context-stage pools, and the C ABI declared
// in include/kvmig.h.
//
// The data path is a pure byte move.  A decoding-stage worker pulls, for each
// migrated block, the (layer range x KV-head range) rectangle it owns out of
// the context-stage workers' pools.  Every such rectangle decomposes into
// "segments" (one per contributing context worker and per K/V pool), each a
// 2-D strided copy per block: `rows` runs of `run_bytes` contiguous bytes.
// Runs are cut into chunks; one chunk is the unit of work a CTA takes from a
// static round-robin schedule, so neighbouring CTAs touch neighbouring DRAM
// pages.  Two kernels execute the same schedule:
//   * kv_migrate_bulk : one elected thread per CTA drives a ring of shared
//     memory stages with cp.async.bulk (global -> shared, completion on an
//     mbarrier; shared -> global as a bulk group).  No multicast anywhere.
//   * kv_migrate_vec  : 256 threads, 16-byte (or narrower, for odd shapes)
//     vector loads and stores, four in flight per thread.
// Source and destination block ids come from device-resident int32 tables
// uploaded once per call.
#include "../../include/kvmig.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>
#include <unistd.h>

namespace kvmig {

// ---------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------

constexpr int kMaxSegs = 16;          // segments per launch (more -> several launches)
constexpr int kVecThreads = 256;
constexpr int kVecUnroll = 4;
constexpr unsigned kSpinLimit = 1u << 26;  // hard cap on mbarrier polls, on top of the time limit below

struct __align__(16) Seg {
    const char* src;                  // context pool base + in-block offset of the rectangle
    char* dst;                        // decoding pool base + in-block offset
    unsigned long long src_block_stride, dst_block_stride;
    unsigned long long src_row_stride, dst_row_stride;
    unsigned long long run_bytes;
    unsigned int rows, chunks_per_run, units_per_block, unit_begin;
};

struct MigParams {
    Seg seg[kMaxSegs];
    const int* src_ids;
    const int* dst_ids;
    int* status;                      // [0] code, [1] unit, [2] detail; host-mapped
    unsigned int nseg, n_blocks, units_per_block, total_units, chunk_bytes;
    unsigned int wait_prior;          // 1: order this grid after the previous grid of the stream before touching memory
    unsigned int l2_hint;             // bit 0: loads evict-first in L2, bit 1: stores evict-first in L2
    unsigned int lose_unit_plus1;     // diagnostic: unit (index + 1) whose load is armed but never issued; 0 = none
    unsigned long long wait_limit_ns; // longest wait for one load before the kernel gives up
    unsigned int batch;               // units drawn per visit to the work counter
    int* work;                        // {next unit, finished CTAs}, both zero between launches; NULL = static deal
};

enum DevStatus { kDevOk = 0, kDevLoadTimeout = 1, kDevDrainTimeout = 2 };

struct Unit {
    const char* src;
    char* dst;
    unsigned int bytes;
};

__device__ __forceinline__ Unit decode_unit(const MigParams& p, const int* src_ids, const int* dst_ids, unsigned int u) {
    unsigned int blk = u / p.units_per_block;
    unsigned int r = u - blk * p.units_per_block;
    unsigned int si = 0;
    while (si + 1 < p.nseg && r >= p.seg[si + 1].unit_begin) ++si;
    const Seg& g = p.seg[si];
    r -= g.unit_begin;
    unsigned int row = r / g.chunks_per_run;
    unsigned int c = r - row * g.chunks_per_run;
    unsigned long long off = (unsigned long long)c * p.chunk_bytes;
    unsigned long long rem = g.run_bytes - off;
    Unit out;
    out.bytes = rem < p.chunk_bytes ? (unsigned int)rem : p.chunk_bytes;
    out.src = g.src + (unsigned long long)src_ids[blk] * g.src_block_stride + row * g.src_row_stride + off;
    out.dst = g.dst + (unsigned long long)dst_ids[blk] * g.dst_block_stride + row * g.dst_row_stride + off;
    return out;
}

// ---- vector-load kernel ----------------------------------------------------

template <int VEC> struct VecType;
template <> struct VecType<16> { using T = uint4; };
template <> struct VecType<8> { using T = uint2; };
template <> struct VecType<4> { using T = unsigned int; };
template <> struct VecType<2> { using T = unsigned short; };
template <> struct VecType<1> { using T = unsigned char; };

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename T> __device__ __forceinline__ T ld_stream(const T* p) { return *p; }

template <int VEC>
__global__ void __launch_bounds__(kVecThreads) kv_migrate_vec(const __grid_constant__ MigParams p) {
    using T = typename VecType<VEC>::T;
    for (unsigned int u = blockIdx.x; u < p.total_units; u += gridDim.x) {
        Unit w = decode_unit(p, p.src_ids, p.dst_ids, u);
        const T* s = reinterpret_cast<const T*>(w.src);
        T* d = reinterpret_cast<T*>(w.dst);
        unsigned int n = w.bytes / VEC;
        for (unsigned int base = threadIdx.x; base < n; base += kVecThreads * kVecUnroll) {
            T v[kVecUnroll];
#pragma unroll
            for (int j = 0; j < kVecUnroll; ++j) {
                unsigned int i = base + j * kVecThreads;
                if (i < n) v[j] = ld_stream(s + i);
            }
#pragma unroll
            for (int j = 0; j < kVecUnroll; ++j) {
                unsigned int i = base + j * kVecThreads;
                if (i < n) d[i] = v[j];
            }
        }
    }
}

// ---- bulk-copy (TMA, untiled) pipeline kernel ------------------------------

__device__ __forceinline__ unsigned int smem_u32(const void* p) {
    return (unsigned int)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits for the barrier's phase, but never longer than limit_ns (nor more than kSpinLimit polls);
// false means the load never signalled.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned int parity, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned int it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u && global_ns() - t0 > limit_ns) return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, unsigned int bytes, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, unsigned int bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gsrc, unsigned int bytes, unsigned long long* bar,
                                              unsigned long long pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(pol) : "memory");
}
__device__ __forceinline__ void bulk_s2g_hint(void* gdst, const void* smem_src, unsigned int bytes, unsigned long long pol) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
                 ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes), "l"(pol) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

constexpr int kMaxStages = 16;

// Shared memory: [stages * stage_bytes ring][stages mbarriers][stages dst ptr][stages sizes]
__device__ __forceinline__ void bulk_pipeline(const MigParams& p, const int* src_ids, const int* dst_ids,
                                              unsigned int stages, unsigned int stage_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    if (threadIdx.x != 0) return;
    unsigned char* ring = smem;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (size_t)stages * stage_bytes);
    char** dst_of = reinterpret_cast<char**>(bars + stages);
    unsigned int* bytes_of = reinterpret_cast<unsigned int*>(dst_of + stages);

    // Let the next migration grid of the stream start while this one is still running (its ramp-up
    // then hides this grid's tail).  The host sets wait_prior when the two grids are not independent.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (unsigned int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_proxy();
    if (p.wait_prior) asm volatile("griddepcontrol.wait;" ::: "memory");

    const unsigned long long pol = l2_evict_first_policy();

    // Work distribution.  With a counter pair (work[0] next unit, work[1] finished CTAs) CTAs draw batches of
    // consecutive units on demand, so no CTA is left finishing a fixed share after the others are done; without
    // one, units are dealt round-robin (unit = blockIdx.x + k * gridDim.x).
    int* const work = p.work;
    const unsigned int batch = p.batch ? p.batch : 1u;
    unsigned int batch_next = 0, batch_end = 0, fetched = 0;
    bool exhausted = false;
    auto next_unit = [&]() -> unsigned int {
        if (work) {
            if (batch_next == batch_end) {
                batch_next = (unsigned int)atomicAdd(work, (int)batch);
                batch_end = batch_next + batch;
            }
            return batch_next++;
        }
        return blockIdx.x + (fetched++) * gridDim.x;
    };

    unsigned int issued = 0;
    auto try_issue = [&]() {
        const unsigned int u = next_unit();
        if (u >= p.total_units) {
            exhausted = true;
            return;
        }
        const unsigned int s = issued % stages;
        Unit w = decode_unit(p, src_ids, dst_ids, u);
        dst_of[s] = w.dst;
        bytes_of[s] = w.bytes;
        mbar_expect_tx(&bars[s], w.bytes);
        if (p.lose_unit_plus1 && u + 1u == p.lose_unit_plus1) {
            // Failure-path exercise: the barrier is armed but the load is never issued, so the wait below
            // must run out and report.  Nothing is in flight towards this stage, so leaving is safe.
        } else if (p.l2_hint & 1u) {
            bulk_g2s_hint(ring + (size_t)s * stage_bytes, w.src, w.bytes, &bars[s], pol);
        } else {
            bulk_g2s(ring + (size_t)s * stage_bytes, w.src, w.bytes, &bars[s]);
        }
        ++issued;
    };

    for (unsigned int i = 0; i < stages && !exhausted; ++i) try_issue();

    unsigned int waited = 0;   // loads whose barrier has been observed complete
    bool ok = true;
    for (unsigned int k = 0; k < issued; ++k) {      // `issued` grows while units remain
        const unsigned int s = k % stages;
        if (!mbar_wait_bounded(&bars[s], (k / stages) & 1u, p.wait_limit_ns)) {
            p.status[0] = kDevLoadTimeout;
            p.status[1] = (int)k;
            ok = false;
            break;
        }
        waited = k + 1;
        if (p.l2_hint & 2u) bulk_s2g_hint(dst_of[s], ring + (size_t)s * stage_bytes, bytes_of[s], pol);
        else bulk_s2g(dst_of[s], ring + (size_t)s * stage_bytes, bytes_of[s]);
        bulk_commit();
        // Refill the stage whose store was issued one iteration ago: by now only the
        // newest store group may still be reading shared memory.
        if (k >= 1 && !exhausted) {
            bulk_wait_read<1>();
            try_issue();
        }
    }
    if (!ok) {
        // Give every load already in flight a bounded chance to land before the
        // shared memory it targets is released.
        for (unsigned int k = waited + 1; k < issued; ++k)
            if (!mbar_wait_bounded(&bars[k % stages], (k / stages) & 1u, p.wait_limit_ns)) { p.status[2] = kDevDrainTimeout; break; }
    }
    bulk_wait_all();
    // A grid that was allowed to start before its predecessor finished must not *finish* before it: whatever
    // follows in the stream waits only for this grid, and must thereby have waited for every earlier one.
    if (!p.wait_prior) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (work) {
        // The last CTA to finish rearms the counter pair for the next launch that uses it.
        __threadfence();
        if (atomicAdd(work + 1, 1) == (int)gridDim.x - 1) {
            work[0] = 0;
            work[1] = 0;
            __threadfence();
        }
    }
}

// Block tables in device memory (any number of blocks).
__global__ void __launch_bounds__(32) kv_migrate_bulk(const __grid_constant__ MigParams p,
                                                       unsigned int stages, unsigned int stage_bytes) {
    bulk_pipeline(p, p.src_ids, p.dst_ids, stages, stage_bytes);
}

// Block tables carried in the kernel's own parameter block ([src ids | dst ids], n_blocks each):
// a typical request (<= 256 blocks) then needs no table upload ahead of the launch, which removes a
// copy-engine hop from the latency of every call.
template <int NIDS>
struct MigParamsInline {
    MigParams base;
    int ids[2 * NIDS];
};

template <int NIDS>
__global__ void __launch_bounds__(32) kv_migrate_bulk_inline(const __grid_constant__ MigParamsInline<NIDS> q,
                                                              unsigned int stages, unsigned int stage_bytes) {
    bulk_pipeline(q.base, q.ids, q.ids + q.base.n_blocks, stages, stage_bytes);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CU_TRY(expr)                                                                       \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess)                                                             \
            return fail(KVMIG_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                               \
    } while (0)

constexpr int64_t kMagic = 0x4b564d4947303031LL;  // "KVMIG001"
// handle words
enum {
    HW_MAGIC = 0, HW_IPC = 1 /*..8*/, HW_OFFSET = 9, HW_BYTES = 10, HW_PID = 11, HW_PTR = 12,
    HW_IPC_VALID = 13, HW_NB = 14, HW_NL = 15, HW_NH = 16, HW_BS = 17, HW_HD = 18, HW_ES = 19,
    HW_DEVICE = 20, HW_RESERVED0 = 21, HW_RESERVED1 = 22, HW_CHECK = 23
};

int64_t handle_checksum(const int64_t* w) {
    uint64_t h = 0x9e3779b97f4a7c15ULL;
    for (int i = 0; i < HW_CHECK; ++i) {
        h ^= (uint64_t)w[i] + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
    }
    return (int64_t)h;
}

// Defaults from sweeps on B200: 8 KiB chunks, a 3-stage ring and 4 CTAs per SM (96 KiB in flight per SM,
// 592 CTAs).  With CTAs drawing units on demand and consecutive launches overlapping, same-GPU copies of
// OPT-13B-shaped blocks run at 6.8 TB/s for any setting from 64 to 192 KiB in flight per SM; awaited single
// calls, which pay their own ramp-up and tail, were fastest around 96 KiB.  Anything from 16 KiB in flight per
// SM upward saturates NVLink.
struct Options {
    std::atomic<int64_t> kernel{0}, chunk_bytes{8192}, stages{3}, ctas_per_sm{0}, inline_tables{1}, overlap_launches{1}, max_ctas{0}, l2_hint{0},
        dynamic_units{1}, wait_limit_ms{2000}, lose_unit_plus1{0};
};
Options g_opt;

struct Counters {
    std::atomic<int64_t> kernel_launches{0}, memcpy_calls{0}, bytes_migrated{0}, bytes_swapped{0}, mapped_peers{0};
};
Counters g_cnt;

struct CtxKey {
    int64_t tp, pp, pp_rank, tp_rank;
    bool operator<(const CtxKey& o) const {
        return std::tie(tp, pp, pp_rank, tp_rank) < std::tie(o.tp, o.pp, o.pp_rank, o.tp_rank);
    }
};

struct CtxEntry {
    std::array<int64_t, KVMIG_HANDLE_WORDS> hk, hv;
    int64_t L = 0, H = 0;
    char* k = nullptr;   // mapped pool addresses, valid in this process once `mapped`
    char* v = nullptr;
    bool mapped = false;
};

struct Slot {
    int* h_tab = nullptr;      // pinned
    int* d_tab = nullptr;
    int* status = nullptr;     // pinned + mapped, 4 ints
    int* status_dev = nullptr;
    int* work = nullptr;       // kWorkPairs counter pairs in device memory, zero whenever no launch is using them
    int64_t layer0 = 0, layer1 = INT64_MAX;   // window of global layers the launch in flight writes
    cudaEvent_t done = nullptr;
    int64_t cap = 0;           // ids per table
    uint64_t seq = 0;          // ticket sequence currently (or last) using this slot
    bool busy = false;
    int64_t bytes = 0;
};

struct DeviceState {
    bool inited = false;
    int sm_count = 0;
    int max_smem_optin = 0;
    std::map<CtxKey, CtxEntry> registry;
    std::map<std::array<int64_t, 8>, char*> ipc_bases;   // opened IPC allocations
    Slot slots[KVMIG_MAX_INFLIGHT];
    uint64_t next_seq = 1;
    int sticky_error = 0;
    std::string sticky_text;
    int bulk_smem_set = 0;
    // Per destination pool (keyed by the K pool's address): ticket sequence of the last launch that wrote
    // each block, used to decide whether a new launch may overlap the launches still in flight.
    std::map<const void*, std::vector<uint64_t>> last_writer;
    std::vector<char> seen;   // duplicate-target bitmap, all zero between calls
};

std::mutex g_mu;
std::map<int, DeviceState> g_dev;

int ensure_device(DeviceState** out, int* dev_out) {
    int dev = -1;
    CU_TRY(cudaGetDevice(&dev));
    DeviceState& st = g_dev[dev];
    if (!st.inited) {
        CU_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
        CU_TRY(cudaDeviceGetAttribute(&st.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        st.inited = true;
    }
    *out = &st;
    if (dev_out) *dev_out = dev;
    return 0;
}

int check_shape(const kvmig_pool_shape* s, const char* what) {
    if (!s) return fail(KVMIG_EINVAL, "%s: shape is NULL", what);
    if (s->num_blocks < 0 || s->num_layers <= 0 || s->num_heads <= 0 || s->block_size <= 0 || s->head_dim <= 0 ||
        s->elem_size <= 0)
        return fail(KVMIG_EINVAL, "%s: non-positive dimension in pool shape [%lld,%lld,%lld,%lld,%lld] x %lld B", what,
                    (long long)s->num_blocks, (long long)s->num_layers, (long long)s->num_heads,
                    (long long)s->block_size, (long long)s->head_dim, (long long)s->elem_size);
    if (s->num_blocks > INT32_MAX) return fail(KVMIG_ELIMIT, "%s: more than 2^31-1 blocks", what);
    return 0;
}

inline int64_t block_bytes(const kvmig_pool_shape& s) {
    return s.num_layers * s.num_heads * s.block_size * s.head_dim * s.elem_size;
}

kvmig_pool_shape shape_of_handle(const int64_t* w) {
    kvmig_pool_shape s;
    s.num_blocks = w[HW_NB]; s.num_layers = w[HW_NL]; s.num_heads = w[HW_NH];
    s.block_size = w[HW_BS]; s.head_dim = w[HW_HD]; s.elem_size = w[HW_ES];
    return s;
}

int validate_handle(const int64_t* w, int64_t len, const char* what) {
    if (!w) return fail(KVMIG_EINVAL, "%s handle is NULL", what);
    if (len != KVMIG_HANDLE_WORDS)
        return fail(KVMIG_EINVAL, "%s handle has %lld words, expected %d", what, (long long)len, KVMIG_HANDLE_WORDS);
    if (w[HW_MAGIC] != kMagic) return fail(KVMIG_EINVAL, "%s handle was not produced by get_ipc_mem_handle (bad magic)", what);
    if (w[HW_CHECK] != handle_checksum(w)) return fail(KVMIG_EINVAL, "%s handle is corrupted (checksum mismatch)", what);
    kvmig_pool_shape s = shape_of_handle(w);
    int rc = check_shape(&s, what);
    if (rc) return rc;
    if (w[HW_BYTES] != s.num_blocks * block_bytes(s)) return fail(KVMIG_EINVAL, "%s handle: byte size does not match its shape", what);
    return 0;
}

// Resolve an exported pool to an address usable on the current device.
int map_pool(DeviceState& st, int dev, const int64_t* w, char** out) {
    if (w[HW_PID] == (int64_t)getpid()) {
        // Exported by this very process: CUDA IPC cannot open its own handles.
        char* p = reinterpret_cast<char*>((uintptr_t)w[HW_PTR]);
        cudaPointerAttributes attr;
        CU_TRY(cudaPointerGetAttributes(&attr, p));
        if (attr.type != cudaMemoryTypeDevice)
            return fail(KVMIG_EINVAL, "handle from this process no longer names device memory");
        if (attr.device != dev) {
            int can = 0;
            CU_TRY(cudaDeviceCanAccessPeer(&can, dev, attr.device));
            if (!can) return fail(KVMIG_ECUDA, "device %d cannot access peer device %d", dev, attr.device);
            cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
            else if (e != cudaSuccess) return fail(KVMIG_ECUDA, "cudaDeviceEnablePeerAccess(%d): %s", attr.device, cudaGetErrorString(e));
        }
        *out = p;
        return 0;
    }
    if (!w[HW_IPC_VALID])
        return fail(KVMIG_ECUDA,
                    "the exporting process could not create a CUDA IPC handle for this pool "
                    "(allocations from a virtual-memory / expandable-segments allocator cannot be shared this way)");
    std::array<int64_t, 8> key;
    std::memcpy(key.data(), &w[HW_IPC], 64);
    auto it = st.ipc_bases.find(key);
    char* base = nullptr;
    if (it != st.ipc_bases.end()) {
        base = it->second;
    } else {
        cudaIpcMemHandle_t h;
        static_assert(sizeof(h) == 64, "CUDA IPC handle is 64 bytes");
        std::memcpy(&h, &w[HW_IPC], 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(KVMIG_ECUDA, "cudaIpcOpenMemHandle (exporter pid %lld, device %lld): %s", (long long)w[HW_PID],
                        (long long)w[HW_DEVICE], cudaGetErrorString(e));
        }
        base = static_cast<char*>(p);
        st.ipc_bases[key] = base;
        g_cnt.mapped_peers++;
    }
    *out = base + w[HW_OFFSET];
    return 0;
}

struct SegPlan {
    CtxKey ctx;
    int64_t src_layer_off, dst_layer_off, n_layers, src_head_off, dst_head_off, n_heads;
};

// Which context workers feed decoding worker (t_d, p_d), and with which sub-rectangles.
// Worker (tp, t, pp, p) owns layers [p*L/pp, (p+1)*L/pp) and heads [t*H/tp, (t+1)*H/tp)
// (distserve/config.py:244-257,279-286).
int plan_segments(int64_t L, int64_t H, int64_t ctx_tp, int64_t ctx_pp, int64_t dec_tp, int64_t t_d, int64_t dec_pp,
                  int64_t p_d, std::vector<SegPlan>* out) {
    if (L <= 0 || H <= 0) return fail(KVMIG_EINVAL, "num_layers and num_heads must be positive");
    if (ctx_tp <= 0 || ctx_pp <= 0 || dec_tp <= 0 || dec_pp <= 0) return fail(KVMIG_EINVAL, "parallel sizes must be positive");
    if (L % ctx_pp || L % dec_pp)
        return fail(KVMIG_EINVAL, "num_layers %lld is not divisible by the pipeline-parallel sizes (%lld, %lld)", (long long)L,
                    (long long)ctx_pp, (long long)dec_pp);
    if (H % ctx_tp || H % dec_tp)
        return fail(KVMIG_EINVAL, "num_heads %lld is not divisible by the tensor-parallel sizes (%lld, %lld)", (long long)H,
                    (long long)ctx_tp, (long long)dec_tp);
    if (t_d < 0 || t_d >= dec_tp || p_d < 0 || p_d >= dec_pp) return fail(KVMIG_EINVAL, "decoding rank out of range");
    const int64_t Ld = L / dec_pp, Hd = H / dec_tp, Lc = L / ctx_pp, Hc = H / ctx_tp;
    const int64_t gl0 = p_d * Ld, gl1 = gl0 + Ld, gh0 = t_d * Hd, gh1 = gh0 + Hd;
    out->clear();
    for (int64_t p = gl0 / Lc; p * Lc < gl1; ++p) {
        int64_t la = std::max(gl0, p * Lc), lb = std::min(gl1, (p + 1) * Lc);
        for (int64_t t = gh0 / Hc; t * Hc < gh1; ++t) {
            int64_t ha = std::max(gh0, t * Hc), hb = std::min(gh1, (t + 1) * Hc);
            SegPlan s;
            s.ctx = CtxKey{ctx_tp, ctx_pp, p, t};
            s.src_layer_off = la - p * Lc; s.dst_layer_off = la - gl0; s.n_layers = lb - la;
            s.src_head_off = ha - t * Hc; s.dst_head_off = ha - gh0; s.n_heads = hb - ha;
            out->push_back(s);
        }
    }
    return 0;
}

constexpr int kWorkPairs = 16;

int grow_slot(Slot& sl, int64_t n) {
    if (!sl.done) CU_TRY(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming));
    if (!sl.work) {
        CU_TRY(cudaMalloc((void**)&sl.work, 2 * kWorkPairs * sizeof(int)));
        CU_TRY(cudaMemset(sl.work, 0, 2 * kWorkPairs * sizeof(int)));
    }
    if (!sl.status) {
        CU_TRY(cudaHostAlloc((void**)&sl.status, 4 * sizeof(int), cudaHostAllocMapped));
        CU_TRY(cudaHostGetDevicePointer((void**)&sl.status_dev, sl.status, 0));
    }
    if (n <= sl.cap) return 0;
    int64_t cap = std::max<int64_t>(1024, sl.cap);
    while (cap < n) cap *= 2;
    if (sl.h_tab) { CU_TRY(cudaFreeHost(sl.h_tab)); sl.h_tab = nullptr; }
    if (sl.d_tab) { CU_TRY(cudaFree(sl.d_tab)); sl.d_tab = nullptr; }
    sl.cap = 0;
    CU_TRY(cudaHostAlloc((void**)&sl.h_tab, 2 * cap * sizeof(int), cudaHostAllocDefault));
    CU_TRY(cudaMalloc((void**)&sl.d_tab, 2 * cap * sizeof(int)));
    sl.cap = cap;
    return 0;
}

int retire_slot(DeviceState& st, Slot& sl) {
    if (!sl.busy) return 0;
    cudaError_t e = cudaEventSynchronize(sl.done);
    sl.busy = false;
    if (e != cudaSuccess) return fail(KVMIG_ECUDA, "waiting for the migration kernel: %s", cudaGetErrorString(e));
    if (sl.status[0] != kDevOk)
        return fail(KVMIG_EDEVICE, "migration kernel gave up (code %d) at work unit %d, detail %d", sl.status[0], sl.status[1],
                    sl.status[2]);
    g_cnt.bytes_migrated += sl.bytes;
    return 0;
}

int pick_vec(uintptr_t bits) {
    for (int v = 16; v > 1; v >>= 1)
        if ((bits & (uintptr_t)(v - 1)) == 0) return v;
    return 1;
}

constexpr int kInlineSmall = 256;    // block ids per table that fit the classic 4 KB parameter block
constexpr int kInlineLarge = 1024;   // needs the large (32 KB) parameter block of recent drivers

template <int NIDS>
cudaError_t launch_bulk_inline(const MigParams& p, const int64_t* src, const int64_t* dst, unsigned grid, size_t smem,
                               cudaStream_t stream, int64_t stages, int64_t chunk, bool overlap) {
    static_assert(sizeof(MigParamsInline<kInlineSmall>) <= 4096, "small inline tables must fit 4 KB of parameters");
    MigParamsInline<NIDS> q;
    q.base = p;
    q.base.src_ids = q.base.dst_ids = nullptr;
    const unsigned n = p.n_blocks;
    for (unsigned i = 0; i < n; ++i) {
        q.ids[i] = (int)src[i];
        q.ids[n + i] = (int)dst[i];
    }
    // Programmatic stream serialization: this grid may begin once the previous grid of the stream has
    // executed griddepcontrol.launch_dependents (our own kernels do so at once; any other kernel
    // triggers only by finishing, which leaves ordinary stream order in place).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kv_migrate_bulk_inline<NIDS>, q, (unsigned)stages, (unsigned)chunk);
}

template <int VEC>
cudaError_t launch_vec(const MigParams& p, unsigned grid, cudaStream_t stream) {
    kv_migrate_vec<VEC><<<grid, kVecThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

int enqueue_migration(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                      int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks, int64_t n_dec,
                      void* k_cache, void* v_cache, const kvmig_pool_shape* shape, cudaStream_t stream, uint64_t* ticket,
                      int64_t layer_begin = 0, int64_t layer_end = INT64_MAX) {
    g_err.clear();
    if (ticket) *ticket = 0;
    int rc = check_shape(shape, "migrate_blocks");
    if (rc) return rc;
    if (n_ctx < 0 || n_dec < 0) return fail(KVMIG_EINVAL, "negative list length");
    if (n_ctx != n_dec)
        return fail(KVMIG_EINVAL, "context_block_indexes has %lld entries but decoding_block_indexes has %lld",
                    (long long)n_ctx, (long long)n_dec);
    if (n_ctx > 0 && (!ctx_blocks || !dec_blocks)) return fail(KVMIG_EINVAL, "block index list is NULL");
    if (!k_cache || !v_cache) return fail(KVMIG_EINVAL, "k_cache / v_cache is NULL");

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* stp;
    int dev;
    rc = ensure_device(&stp, &dev);
    if (rc) return rc;
    DeviceState& st = *stp;

    const int64_t L = shape->num_layers * dec_pp, H = shape->num_heads * dec_tp;
    std::vector<SegPlan> plan;
    rc = plan_segments(L, H, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank, &plan);
    if (rc) return rc;
    // Optional window of global layers: keep only the part of each segment that lies inside it.
    if (layer_begin < 0 || layer_end < layer_begin)
        return fail(KVMIG_EINVAL, "layer window [%lld, %lld) is not a range", (long long)layer_begin, (long long)layer_end);
    layer_end = std::min(layer_end, L);
    const bool windowed = layer_begin > 0 || layer_end < L;
    if (windowed) {
        const int64_t first_layer = dec_pp_rank * shape->num_layers;   // global index of this worker's local layer 0
        std::vector<SegPlan> clipped;
        for (SegPlan sp : plan) {
            const int64_t g0 = first_layer + sp.dst_layer_off, g1 = g0 + sp.n_layers;
            const int64_t a = std::max(g0, layer_begin), b = std::min(g1, layer_end);
            if (a >= b) continue;
            sp.src_layer_off += a - g0;
            sp.dst_layer_off += a - g0;
            sp.n_layers = b - a;
            clipped.push_back(sp);
        }
        plan.swap(clipped);
    }

    const int64_t slab = shape->block_size * shape->head_dim * shape->elem_size;
    const int64_t Lc = L / ctx_pp, Hc = H / ctx_tp;
    int64_t src_num_blocks = INT64_MAX;
    std::vector<Seg> segs;
    uintptr_t align_bits = 0;
    int64_t chunk = g_opt.chunk_bytes.load();
    for (const SegPlan& sp : plan) {
        auto it = st.registry.find(sp.ctx);
        if (it == st.registry.end())
            return fail(KVMIG_ENOTREG,
                        "context worker (pp_rank %lld, tp_rank %lld) of a tp=%lld,pp=%lld context stage is not registered "
                        "on this device; call register_ipc_mem_handle first",
                        (long long)sp.ctx.pp_rank, (long long)sp.ctx.tp_rank, (long long)ctx_tp, (long long)ctx_pp);
        CtxEntry& ce = it->second;
        if (ce.L != L || ce.H != H)
            return fail(KVMIG_EINVAL, "registered model shape (%lld layers, %lld heads) differs from this worker's (%lld, %lld)",
                        (long long)ce.L, (long long)ce.H, (long long)L, (long long)H);
        kvmig_pool_shape ss = shape_of_handle(ce.hk.data());
        if (ss.block_size != shape->block_size || ss.head_dim != shape->head_dim || ss.elem_size != shape->elem_size)
            return fail(KVMIG_EINVAL, "context pool block geometry (%lld x %lld x %lld B) differs from the decoding pool's",
                        (long long)ss.block_size, (long long)ss.head_dim, (long long)ss.elem_size);
        if (!ce.mapped) {
            rc = map_pool(st, dev, ce.hk.data(), &ce.k);
            if (rc) return rc;
            rc = map_pool(st, dev, ce.hv.data(), &ce.v);
            if (rc) return rc;
            ce.mapped = true;
        }
        src_num_blocks = std::min(src_num_blocks, std::min(ce.hk[HW_NB], ce.hv[HW_NB]));
        for (int x = 0; x < 2; ++x) {
            Seg g;
            const char* sbase = x == 0 ? ce.k : ce.v;
            char* dbase = static_cast<char*>(x == 0 ? k_cache : v_cache);
            g.src_block_stride = Lc * Hc * slab;
            g.dst_block_stride = shape->num_layers * shape->num_heads * slab;
            g.src_row_stride = Hc * slab;
            g.dst_row_stride = shape->num_heads * slab;
            g.run_bytes = sp.n_heads * slab;
            g.rows = (unsigned)sp.n_layers;
            g.src = sbase + sp.src_layer_off * g.src_row_stride + sp.src_head_off * slab;
            g.dst = dbase + sp.dst_layer_off * g.dst_row_stride + sp.dst_head_off * slab;
            if (g.run_bytes == g.src_row_stride && g.run_bytes == g.dst_row_stride) {
                g.run_bytes *= g.rows;   // whole layers on both sides: rows are adjacent
                g.rows = 1;
            }
            align_bits |= (uintptr_t)g.src | (uintptr_t)g.dst | g.src_block_stride | g.dst_block_stride |
                          g.src_row_stride | g.dst_row_stride | g.run_bytes;
            segs.push_back(g);
        }
    }

    // Validate ids before anything is enqueued.  `seen` is a per-device bitmap kept all-zero between calls.
    std::vector<char>& seen = st.seen;
    if ((int64_t)seen.size() < shape->num_blocks) seen.resize((size_t)shape->num_blocks, 0);
    int64_t checked = 0;
    rc = 0;
    for (; checked < n_ctx && !rc; ++checked) {
        const int64_t i = checked;
        if (ctx_blocks[i] < 0 || ctx_blocks[i] >= src_num_blocks)
            rc = fail(KVMIG_EINVAL, "context_block_indexes[%lld] = %lld is outside the context pool (%lld blocks)", (long long)i,
                      (long long)ctx_blocks[i], (long long)src_num_blocks);
        else if (dec_blocks[i] < 0 || dec_blocks[i] >= shape->num_blocks)
            rc = fail(KVMIG_EINVAL, "decoding_block_indexes[%lld] = %lld is outside the decoding pool (%lld blocks)",
                      (long long)i, (long long)dec_blocks[i], (long long)shape->num_blocks);
        else if (seen[(size_t)dec_blocks[i]])
            rc = fail(KVMIG_EINVAL, "decoding_block_indexes names block %lld twice", (long long)dec_blocks[i]);
        else
            seen[(size_t)dec_blocks[i]] = 1;
    }
    for (int64_t i = 0; i < checked; ++i)
        if (dec_blocks[i] >= 0 && dec_blocks[i] < shape->num_blocks) seen[(size_t)dec_blocks[i]] = 0;
    if (rc) return rc;
    if (n_ctx == 0 || plan.empty()) return 0;   // nothing to move (empty lists, or the window misses this worker)

    // Kernel choice.
    const int vec = pick_vec(align_bits);
    int64_t kernel = g_opt.kernel.load();
    if (kernel == 0) kernel = (vec == 16) ? 2 : 1;
    if (kernel == 2 && vec != 16) return fail(KVMIG_EINVAL, "the bulk-copy kernel needs 16-byte aligned runs; this shape gives %d", vec);
    int64_t stages = std::min<int64_t>(std::max<int64_t>(g_opt.stages.load(), 2), kMaxStages);
    if (chunk < 16 || chunk % 16) return fail(KVMIG_EINVAL, "chunk_bytes must be a positive multiple of 16");
    size_t smem = 0;
    int64_t ctas_per_sm = g_opt.ctas_per_sm.load();
    if (kernel == 2) {
        smem = (size_t)stages * chunk + (size_t)stages * (8 + 8 + 4) + 16;
        if ((int64_t)smem > st.max_smem_optin)
            return fail(KVMIG_ELIMIT, "stages x chunk_bytes = %zu B exceeds the %d B of shared memory a CTA may use", smem,
                        st.max_smem_optin);
        if (ctas_per_sm <= 0) {
            const int64_t ring = stages * chunk, target = 96 * 1024;   // bytes in flight per SM
            ctas_per_sm = std::max<int64_t>(1, std::min<int64_t>(8, (target + ring - 1) / ring));
            ctas_per_sm = std::min<int64_t>(ctas_per_sm, std::max<int64_t>(1, (220 * 1024) / (int64_t)(smem + 1024)));
        }
        if ((int)smem > st.bulk_smem_set) {
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk_inline<kInlineSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk_inline<kInlineLarge>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
            st.bulk_smem_set = (int)smem;
        }
    } else if (ctas_per_sm <= 0) {
        ctas_per_sm = 8;
    }

    // Ticket slot.
    uint64_t seq = st.next_seq++;
    Slot& sl = st.slots[seq % KVMIG_MAX_INFLIGHT];
    rc = retire_slot(st, sl);
    if (rc && !st.sticky_error) { st.sticky_error = rc; st.sticky_text = g_err; }
    // Tables of a typical request ride in the kernel parameters; longer lists go through device memory.
    const bool inline_tables = kernel == 2 && g_opt.inline_tables.load() != 0 && n_ctx <= kInlineLarge;
    rc = grow_slot(sl, inline_tables ? 0 : n_ctx);
    if (rc) return rc;
    sl.status[0] = sl.status[1] = sl.status[2] = sl.status[3] = 0;
    // May this launch overlap the migrations still in flight?  Only if it writes none of their blocks.
    const bool overlap = inline_tables && g_opt.overlap_launches.load() != 0;
    bool depends = !overlap;
    {
        std::vector<uint64_t>& marks = st.last_writer[k_cache];
        if ((int64_t)marks.size() < shape->num_blocks) marks.resize((size_t)shape->num_blocks, 0);
        int running[KVMIG_MAX_INFLIGHT];   // -1 unknown, 0 finished, 1 still running; one query per slot at most
        for (int& r : running) r = -1;
        for (int64_t i = 0; i < n_ctx; ++i) {
            uint64_t& m = marks[(size_t)dec_blocks[i]];
            if (m != 0 && !depends) {
                const int si = (int)(m % KVMIG_MAX_INFLIGHT);
                Slot& other = st.slots[si];
                if (other.seq == m && other.busy && other.layer0 < layer_end && layer_begin < other.layer1) {
                    if (running[si] < 0) running[si] = cudaEventQuery(other.done) == cudaSuccess ? 0 : 1;
                    if (running[si] == 1) depends = true;
                }
            }
            m = seq;
        }
        (void)cudaGetLastError();   // cudaEventQuery reports "not ready" through the error state
    }
    if (!inline_tables) {
        for (int64_t i = 0; i < n_ctx; ++i) {
            sl.h_tab[i] = (int)ctx_blocks[i];
            sl.h_tab[n_ctx + i] = (int)dec_blocks[i];
        }
        CU_TRY(cudaMemcpyAsync(sl.d_tab, sl.h_tab, 2 * n_ctx * sizeof(int), cudaMemcpyHostToDevice, stream));
        g_cnt.memcpy_calls++;
    }

    int64_t bytes_per_block = 0;
    int launch_index = 0;
    for (size_t s0 = 0; s0 < segs.size(); s0 += kMaxSegs) {
        MigParams p;
        std::memset(&p, 0, sizeof p);
        p.nseg = (unsigned)std::min<size_t>(kMaxSegs, segs.size() - s0);
        unsigned upb = 0;
        for (unsigned s = 0; s < p.nseg; ++s) {
            Seg g = segs[s0 + s];
            g.chunks_per_run = (unsigned)((g.run_bytes + chunk - 1) / chunk);
            g.units_per_block = g.rows * g.chunks_per_run;
            g.unit_begin = upb;
            upb += g.units_per_block;
            p.seg[s] = g;
            bytes_per_block += (int64_t)g.run_bytes * g.rows;
        }
        p.src_ids = sl.d_tab;
        p.dst_ids = sl.d_tab + n_ctx;
        p.status = sl.status_dev;
        p.n_blocks = (unsigned)n_ctx;
        p.units_per_block = upb;
        p.chunk_bytes = (unsigned)chunk;
        p.wait_prior = depends ? 1u : 0u;
        p.l2_hint = (unsigned)g_opt.l2_hint.load();
        p.wait_limit_ns = (unsigned long long)std::max<int64_t>(1, g_opt.wait_limit_ms.load()) * 1000000ULL;
        p.lose_unit_plus1 = (unsigned)g_opt.lose_unit_plus1.load();
        // total_units is 32-bit: walk the block list in slices if a launch would overflow.
        const int64_t max_blocks = std::max<int64_t>(1, (int64_t)0x7fffffff / upb);
        for (int64_t b0 = 0; b0 < n_ctx; b0 += max_blocks) {
            int64_t nb = std::min(max_blocks, n_ctx - b0);
            p.src_ids = sl.d_tab + b0;
            p.dst_ids = sl.d_tab + n_ctx + b0;
            p.n_blocks = (unsigned)nb;
            p.total_units = (unsigned)(nb * upb);
            unsigned grid = (unsigned)std::min<int64_t>(p.total_units, (int64_t)st.sm_count * ctas_per_sm);
            // A cap on the grid leaves whole SMs to a decode step running beside the migration.
            if (const int64_t cap = g_opt.max_ctas.load(); cap > 0) grid = (unsigned)std::min<int64_t>(grid, cap);
            // Each launch of this call gets its own counter pair (launches of one call may overlap).
            p.work = nullptr;
            p.batch = 1;
            // (A short launch keeps the fixed deal: the counter's latency would be most of its run time.)
            if (kernel == 2 && g_opt.dynamic_units.load() != 0 && launch_index < kWorkPairs && p.total_units >= 4u * grid) {
                p.work = sl.work + 2 * launch_index;
                p.batch = p.total_units >= 32u * grid ? 4u : (p.total_units >= 8u * grid ? 2u : 1u);
            }
            ++launch_index;
            cudaError_t e;
            if (inline_tables) {
                e = n_ctx <= kInlineSmall
                        ? launch_bulk_inline<kInlineSmall>(p, ctx_blocks + b0, dec_blocks + b0, grid, smem, stream, stages, chunk,
                                                           overlap)
                        : launch_bulk_inline<kInlineLarge>(p, ctx_blocks + b0, dec_blocks + b0, grid, smem, stream, stages,
                                                           chunk, overlap);
            } else if (kernel == 2) {
                kv_migrate_bulk<<<grid, 32, smem, stream>>>(p, (unsigned)stages, (unsigned)chunk);
                e = cudaGetLastError();
            } else {
                switch (vec) {
                    case 16: e = launch_vec<16>(p, grid, stream); break;
                    case 8: e = launch_vec<8>(p, grid, stream); break;
                    case 4: e = launch_vec<4>(p, grid, stream); break;
                    case 2: e = launch_vec<2>(p, grid, stream); break;
                    default: e = launch_vec<1>(p, grid, stream); break;
                }
            }
            if (e != cudaSuccess) return fail(KVMIG_ECUDA, "launching the migration kernel: %s", cudaGetErrorString(e));
            g_cnt.kernel_launches++;
        }
    }
    CU_TRY(cudaEventRecord(sl.done, stream));
    sl.busy = true;
    sl.seq = seq;
    sl.layer0 = layer_begin;
    sl.layer1 = layer_end;
    sl.bytes = bytes_per_block * n_ctx;
    if (ticket) *ticket = ((uint64_t)(unsigned)dev << 48) | seq;
    return 0;
}

int wait_ticket(uint64_t ticket) {
    g_err.clear();
    if (ticket == 0) return 0;
    int dev = (int)(ticket >> 48);
    uint64_t seq = ticket & ((1ULL << 48) - 1);
    std::unique_lock<std::mutex> lock(g_mu);
    auto it = g_dev.find(dev);
    if (it == g_dev.end()) return fail(KVMIG_EINVAL, "unknown ticket");
    DeviceState& st = it->second;      // std::map nodes stay put, so the reference survives unlocking
    if (seq >= st.next_seq) return fail(KVMIG_EINVAL, "unknown ticket");
    Slot& sl = st.slots[seq % KVMIG_MAX_INFLIGHT];
    int rc = 0;
    if (sl.seq == seq && sl.busy) {
        // Wait for the kernel without holding the lock, so other threads can keep enqueuing; the event
        // stays valid (events are created once per slot and never destroyed).
        cudaEvent_t done = sl.done;
        lock.unlock();
        cudaError_t e = cudaEventSynchronize(done);
        lock.lock();
        if (e != cudaSuccess) rc = fail(KVMIG_ECUDA, "waiting for the migration kernel: %s", cudaGetErrorString(e));
        if (!rc && sl.seq == seq) rc = retire_slot(st, sl);   // returns at once: the event has completed
    }
    if (!rc && st.sticky_error) {
        rc = st.sticky_error;
        g_err = st.sticky_text;
        st.sticky_error = 0;
    }
    return rc;
}


// ---------------------------------------------------------------------------
// Allocation-free variant of the migration entry point
// ---------------------------------------------------------------------------
//
// kvmig_migrate_blocks needs a little device scratch besides the pools: the two
// int32 block tables and a status word.  It gets them from cudaMalloc /
// cudaHostAlloc on first use.  Some hosts must not allocate once serving has
// started: a decoding worker sizes its KV pools from whatever HBM is free
// (distserve/worker.py:152-192), so a later cudaMalloc may fail or stall the
// device in the middle of a decode loop, and some embedders forbid allocation
// after start-up altogether.  For them the scratch below is part of the loaded
// module: every GPU that loads this library holds these 33 KiB until exit.
//
// In host code `g_static_scratch` is only a stand-in symbol, not a device
// address; the address is looked up once per device with cudaGetSymbolAddress
// (with that device current) and that pointer is what the kernels receive.
constexpr int kStaticStatusWords = 64;                        // 256 B, keeps the tables 256-byte aligned
static __device__ __align__(256) int g_static_scratch[kStaticStatusWords + 2 * KVMIG_STATIC_MAX_BLOCKS];

constexpr int kStaticMaxDevices = 64;
int* g_static_ptr[kStaticMaxDevices];                         // device address of the array, per device ordinal
int g_static_stage[kStaticStatusWords + 2 * KVMIG_STATIC_MAX_BLOCKS];   // host staging image, guarded by g_mu

int static_scratch_for_current_device(int dev, int** out) {
    if (dev < 0 || dev >= kStaticMaxDevices) return fail(KVMIG_ELIMIT, "device ordinal %d is beyond %d", dev, kStaticMaxDevices);
    if (!g_static_ptr[dev]) {
        int* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(KVMIG_ECUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return 0;
}

int migrate_static(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp, int64_t dec_tp,
                   int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks, int64_t n_dec, void* k_cache,
                   void* v_cache, const kvmig_pool_shape* shape, cudaStream_t stream) {
    g_err.clear();
    int rc = check_shape(shape, "migrate_blocks_static");
    if (rc) return rc;
    if (n_ctx < 0 || n_dec < 0) return fail(KVMIG_EINVAL, "negative list length");
    if (n_ctx != n_dec)
        return fail(KVMIG_EINVAL, "context_block_indexes has %lld entries but decoding_block_indexes has %lld",
                    (long long)n_ctx, (long long)n_dec);
    if (n_ctx > KVMIG_STATIC_MAX_BLOCKS)
        return fail(KVMIG_ELIMIT,
                    "%lld blocks in one call exceed the %d the built-in scratch holds; split the lists or use "
                    "kvmig_migrate_blocks",
                    (long long)n_ctx, KVMIG_STATIC_MAX_BLOCKS);
    if (n_ctx > 0 && (!ctx_blocks || !dec_blocks)) return fail(KVMIG_EINVAL, "block index list is NULL");
    if (!k_cache || !v_cache) return fail(KVMIG_EINVAL, "k_cache / v_cache is NULL");

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* stp;
    int dev;
    rc = ensure_device(&stp, &dev);
    if (rc) return rc;
    DeviceState& st = *stp;
    int* scratch = nullptr;
    rc = static_scratch_for_current_device(dev, &scratch);
    if (rc) return rc;

    const int64_t L = shape->num_layers * dec_pp, H = shape->num_heads * dec_tp;
    std::vector<SegPlan> plan;
    rc = plan_segments(L, H, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank, &plan);
    if (rc) return rc;
    if (plan.size() * 2 > (size_t)kMaxSegs)
        return fail(KVMIG_ELIMIT, "this reshard needs %zu segments; the allocation-free entry point takes %d", plan.size() * 2,
                    kMaxSegs);
    const int64_t slab = shape->block_size * shape->head_dim * shape->elem_size;
    const int64_t Lc = L / ctx_pp, Hc = H / ctx_tp;
    const int64_t chunk = g_opt.chunk_bytes.load();
    MigParams p;
    std::memset(&p, 0, sizeof p);
    int64_t src_num_blocks = INT64_MAX, bytes_per_block = 0;
    uintptr_t align_bits = 0;
    unsigned upb = 0;
    for (const SegPlan& sp : plan) {
        auto it = st.registry.find(sp.ctx);
        if (it == st.registry.end())
            return fail(KVMIG_ENOTREG, "context worker (pp_rank %lld, tp_rank %lld) is not registered on this device",
                        (long long)sp.ctx.pp_rank, (long long)sp.ctx.tp_rank);
        const CtxEntry& ce = it->second;
        if (!ce.mapped)   // mapping a peer pool reserves address space; that belongs to registration, not to this call
            return fail(KVMIG_ENOTREG,
                        "context worker (pp_rank %lld, tp_rank %lld) was registered for another decoding rank and is not "
                        "mapped; register it with this worker's parallel config first",
                        (long long)sp.ctx.pp_rank, (long long)sp.ctx.tp_rank);
        if (ce.L != L || ce.H != H) return fail(KVMIG_EINVAL, "registered model shape differs from this worker's");
        kvmig_pool_shape ss = shape_of_handle(ce.hk.data());
        if (ss.block_size != shape->block_size || ss.head_dim != shape->head_dim || ss.elem_size != shape->elem_size)
            return fail(KVMIG_EINVAL, "context pool block geometry differs from the decoding pool's");
        src_num_blocks = std::min(src_num_blocks, std::min(ce.hk[HW_NB], ce.hv[HW_NB]));
        for (int x = 0; x < 2; ++x) {
            Seg g;
            g.src_block_stride = Lc * Hc * slab;
            g.dst_block_stride = shape->num_layers * shape->num_heads * slab;
            g.src_row_stride = Hc * slab;
            g.dst_row_stride = shape->num_heads * slab;
            g.run_bytes = sp.n_heads * slab;
            g.rows = (unsigned)sp.n_layers;
            g.src = (x == 0 ? ce.k : ce.v) + sp.src_layer_off * g.src_row_stride + sp.src_head_off * slab;
            g.dst = static_cast<char*>(x == 0 ? k_cache : v_cache) + sp.dst_layer_off * g.dst_row_stride + sp.dst_head_off * slab;
            if (g.run_bytes == g.src_row_stride && g.run_bytes == g.dst_row_stride) {
                g.run_bytes *= g.rows;
                g.rows = 1;
            }
            align_bits |= (uintptr_t)g.src | (uintptr_t)g.dst | g.src_block_stride | g.dst_block_stride | g.src_row_stride |
                          g.dst_row_stride | g.run_bytes;
            g.chunks_per_run = (unsigned)((g.run_bytes + chunk - 1) / chunk);
            g.units_per_block = g.rows * g.chunks_per_run;
            g.unit_begin = upb;
            upb += g.units_per_block;
            bytes_per_block += (int64_t)g.run_bytes * g.rows;
            p.seg[p.nseg++] = g;
        }
    }
    for (int64_t i = 0; i < n_ctx; ++i) {
        if (ctx_blocks[i] < 0 || ctx_blocks[i] >= src_num_blocks)
            return fail(KVMIG_EINVAL, "context_block_indexes[%lld] = %lld is outside the context pool (%lld blocks)", (long long)i,
                        (long long)ctx_blocks[i], (long long)src_num_blocks);
        if (dec_blocks[i] < 0 || dec_blocks[i] >= shape->num_blocks)
            return fail(KVMIG_EINVAL, "decoding_block_indexes[%lld] = %lld is outside the decoding pool (%lld blocks)",
                        (long long)i, (long long)dec_blocks[i], (long long)shape->num_blocks);
        for (int64_t j = 0; j < i; ++j)   // n <= 4096: a quadratic scan needs no memory
            if (dec_blocks[j] == dec_blocks[i])
                return fail(KVMIG_EINVAL, "decoding_block_indexes names block %lld twice", (long long)dec_blocks[i]);
    }
    if (n_ctx == 0) return 0;
    if ((int64_t)upb * n_ctx > 0x7fffffff) return fail(KVMIG_ELIMIT, "too many work units for one launch; lower the block count");

    const int vec = pick_vec(align_bits);
    int64_t kernel = g_opt.kernel.load();
    if (kernel == 0) kernel = (vec == 16) ? 2 : 1;
    if (kernel == 2 && vec != 16) return fail(KVMIG_EINVAL, "the bulk-copy kernel needs 16-byte aligned runs; this shape gives %d", vec);
    const int64_t stages = std::min<int64_t>(std::max<int64_t>(g_opt.stages.load(), 2), kMaxStages);
    size_t smem = 0;
    int64_t ctas_per_sm = g_opt.ctas_per_sm.load();
    if (kernel == 2) {
        smem = (size_t)stages * chunk + (size_t)stages * (8 + 8 + 4) + 16;
        if ((int64_t)smem > st.max_smem_optin) return fail(KVMIG_ELIMIT, "stages x chunk_bytes exceeds the shared memory a CTA may use");
        if (ctas_per_sm <= 0) {
            const int64_t ring = stages * chunk, target = 96 * 1024;
            ctas_per_sm = std::max<int64_t>(1, std::min<int64_t>(8, (target + ring - 1) / ring));
            ctas_per_sm = std::min<int64_t>(ctas_per_sm, std::max<int64_t>(1, (220 * 1024) / (int64_t)(smem + 1024)));
        }
        if ((int)smem > st.bulk_smem_set) {
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            st.bulk_smem_set = (int)smem;
        }
    } else if (ctas_per_sm <= 0) {
        ctas_per_sm = 8;
    }

    // One upload carries the cleared status words and both tables: the array keeps whatever the last
    // call left in it, so everything this launch reads is rewritten first.
    const size_t words = (size_t)kStaticStatusWords + 2 * (size_t)n_ctx;
    std::memset(g_static_stage, 0, kStaticStatusWords * sizeof(int));
    for (int64_t i = 0; i < n_ctx; ++i) {
        g_static_stage[kStaticStatusWords + i] = (int)ctx_blocks[i];
        g_static_stage[kStaticStatusWords + n_ctx + i] = (int)dec_blocks[i];
    }
    CU_TRY(cudaMemcpyAsync(scratch, g_static_stage, words * sizeof(int), cudaMemcpyHostToDevice, stream));
    g_cnt.memcpy_calls++;
    p.src_ids = scratch + kStaticStatusWords;
    p.dst_ids = scratch + kStaticStatusWords + n_ctx;
    p.status = scratch;
    p.n_blocks = (unsigned)n_ctx;
    p.units_per_block = upb;
    p.wait_limit_ns = (unsigned long long)std::max<int64_t>(1, g_opt.wait_limit_ms.load()) * 1000000ULL;
    p.chunk_bytes = (unsigned)chunk;
    p.total_units = (unsigned)(n_ctx * upb);
    const unsigned grid = (unsigned)std::min<int64_t>(p.total_units, (int64_t)st.sm_count * ctas_per_sm);
    cudaError_t e;
    if (kernel == 2) {
        kv_migrate_bulk<<<grid, 32, smem, stream>>>(p, (unsigned)stages, (unsigned)chunk);
        e = cudaGetLastError();
    } else {
        switch (vec) {
            case 16: e = launch_vec<16>(p, grid, stream); break;
            case 8: e = launch_vec<8>(p, grid, stream); break;
            case 4: e = launch_vec<4>(p, grid, stream); break;
            case 2: e = launch_vec<2>(p, grid, stream); break;
            default: e = launch_vec<1>(p, grid, stream); break;
        }
    }
    if (e != cudaSuccess) return fail(KVMIG_ECUDA, "launching the migration kernel: %s", cudaGetErrorString(e));
    g_cnt.kernel_launches++;
    int status[4] = {0, 0, 0, 0};
    CU_TRY(cudaMemcpyAsync(status, scratch, sizeof status, cudaMemcpyDeviceToHost, stream));
    CU_TRY(cudaStreamSynchronize(stream));   // sources are read and the staging image is free again
    if (status[0] != kDevOk)
        return fail(KVMIG_EDEVICE, "migration kernel gave up (code %d) at work unit %d, detail %d", status[0], status[1], status[2]);
    g_cnt.bytes_migrated += bytes_per_block * n_ctx;
    return 0;
}

}  // namespace kvmig

using namespace kvmig;

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------

extern "C" {

int kvmig_abi_version(void) { return KVMIG_ABI_VERSION; }

const char* kvmig_last_error(void) { return g_err.c_str(); }

int kvmig_get_ipc_mem_handle(const void* pool, const kvmig_pool_shape* shape, int64_t* w) {
    g_err.clear();
    if (!pool || !w) return fail(KVMIG_EINVAL, "get_ipc_mem_handle: NULL argument");
    int rc = check_shape(shape, "get_ipc_mem_handle");
    if (rc) return rc;
    cudaPointerAttributes attr;
    CU_TRY(cudaPointerGetAttributes(&attr, pool));
    if (attr.type != cudaMemoryTypeDevice) return fail(KVMIG_EINVAL, "get_ipc_mem_handle: the pool is not CUDA device memory");

    // Allocators sub-allocate: the IPC handle names the enclosing allocation,
    // so the pool's offset inside it travels with the handle.
    typedef int (*GetRangeFn)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CU_TRY(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return fail(KVMIG_ECUDA, "cuMemGetAddressRange is unavailable");
    unsigned long long base = 0;
    size_t span = 0;
    int drc = reinterpret_cast<GetRangeFn>(fn)(&base, &span, (unsigned long long)(uintptr_t)pool);
    if (drc != 0) return fail(KVMIG_ECUDA, "cuMemGetAddressRange failed with driver error %d", drc);
    const int64_t bytes = shape->num_blocks * block_bytes(*shape);
    const int64_t offset = (int64_t)((uintptr_t)pool - (uintptr_t)base);
    if (offset + bytes > (int64_t)span) return fail(KVMIG_EINVAL, "get_ipc_mem_handle: the shape exceeds the allocation that holds the pool");

    std::memset(w, 0, sizeof(int64_t) * KVMIG_HANDLE_WORDS);
    cudaIpcMemHandle_t h;
    int prev = -1;
    CU_TRY(cudaGetDevice(&prev));
    if (prev != attr.device) CU_TRY(cudaSetDevice(attr.device));
    cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base));
    if (prev != attr.device) CU_TRY(cudaSetDevice(prev));
    if (e == cudaSuccess) {
        std::memcpy(&w[HW_IPC], &h, 64);
        w[HW_IPC_VALID] = 1;
    } else {
        (void)cudaGetLastError();   // same-process use still works; a remote open reports the problem
        w[HW_IPC_VALID] = 0;
    }
    w[HW_MAGIC] = kMagic;
    w[HW_OFFSET] = offset;
    w[HW_BYTES] = bytes;
    w[HW_PID] = (int64_t)getpid();
    w[HW_PTR] = (int64_t)(uintptr_t)pool;
    w[HW_NB] = shape->num_blocks; w[HW_NL] = shape->num_layers; w[HW_NH] = shape->num_heads;
    w[HW_BS] = shape->block_size; w[HW_HD] = shape->head_dim; w[HW_ES] = shape->elem_size;
    w[HW_DEVICE] = attr.device;
    w[HW_CHECK] = handle_checksum(w);
    return 0;
}

int kvmig_register_ipc_mem_handle(const int64_t* k_handle, int64_t k_len, const int64_t* v_handle, int64_t v_len,
                                  int64_t num_layers, int64_t num_heads, const int64_t* ctx_pc, const int64_t* dec_pc) {
    g_err.clear();
    int rc = validate_handle(k_handle, k_len, "k_cache");
    if (rc) return rc;
    rc = validate_handle(v_handle, v_len, "v_cache");
    if (rc) return rc;
    if (!ctx_pc || !dec_pc) return fail(KVMIG_EINVAL, "parallel config is NULL");
    const int64_t ctx_tp = ctx_pc[0], ctx_t = ctx_pc[1], ctx_pp = ctx_pc[2], ctx_p = ctx_pc[3];
    const int64_t dec_tp = dec_pc[0], dec_t = dec_pc[1], dec_pp = dec_pc[2], dec_p = dec_pc[3];
    if (ctx_tp <= 0 || ctx_pp <= 0 || ctx_t < 0 || ctx_t >= ctx_tp || ctx_p < 0 || ctx_p >= ctx_pp)
        return fail(KVMIG_EINVAL, "context parallel config [%lld,%lld,%lld,%lld] is not [tp_size,tp_rank,pp_size,pp_rank]",
                    (long long)ctx_tp, (long long)ctx_t, (long long)ctx_pp, (long long)ctx_p);
    std::vector<SegPlan> plan;
    rc = plan_segments(num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_t, dec_pp, dec_p, &plan);
    if (rc) return rc;
    kvmig_pool_shape sk = shape_of_handle(k_handle), sv = shape_of_handle(v_handle);
    if (std::memcmp(&sk.num_layers, &sv.num_layers, sizeof(int64_t) * 5) != 0)
        return fail(KVMIG_EINVAL, "K and V pool handles describe different block shapes");
    if (sk.num_layers != num_layers / ctx_pp || sk.num_heads != num_heads / ctx_tp)
        return fail(KVMIG_EINVAL,
                    "exported pool holds %lld layers x %lld heads, but a tp=%lld,pp=%lld worker of a %lld-layer %lld-head model "
                    "holds %lld x %lld",
                    (long long)sk.num_layers, (long long)sk.num_heads, (long long)ctx_tp, (long long)ctx_pp,
                    (long long)num_layers, (long long)num_heads, (long long)(num_layers / ctx_pp), (long long)(num_heads / ctx_tp));

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* stp;
    int dev;
    rc = ensure_device(&stp, &dev);
    if (rc) return rc;
    CtxEntry ce;
    std::memcpy(ce.hk.data(), k_handle, sizeof(int64_t) * KVMIG_HANDLE_WORDS);
    std::memcpy(ce.hv.data(), v_handle, sizeof(int64_t) * KVMIG_HANDLE_WORDS);
    ce.L = num_layers;
    ce.H = num_heads;
    CtxKey key{ctx_tp, ctx_pp, ctx_p, ctx_t};
    bool needed = false;
    for (const SegPlan& sp : plan)
        if (!(sp.ctx < key) && !(key < sp.ctx)) needed = true;
    auto prev = stp->registry.find(key);
    if (prev != stp->registry.end() && prev->second.mapped && prev->second.hk == ce.hk && prev->second.hv == ce.hv) {
        // The same pools registered again (by another decoding rank of this process): keep the mapping.
        ce.k = prev->second.k;
        ce.v = prev->second.v;
        ce.mapped = true;
    } else if (needed) {
        rc = map_pool(*stp, dev, ce.hk.data(), &ce.k);
        if (rc) return rc;
        rc = map_pool(*stp, dev, ce.hv.data(), &ce.v);
        if (rc) return rc;
        ce.mapped = true;
    }
    stp->registry[key] = ce;
    return 0;
}

int kvmig_migrate_blocks_async(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                               int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks,
                               int64_t n_dec, void* k_cache, void* v_cache, const kvmig_pool_shape* shape, void* stream,
                               uint64_t* ticket) {
    if (!ticket) return fail(KVMIG_EINVAL, "ticket is NULL");
    return enqueue_migration(ctx_pp, ctx_tp, ctx_blocks, n_ctx, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks, n_dec,
                             k_cache, v_cache, shape, static_cast<cudaStream_t>(stream), ticket);
}

int kvmig_migrate_layers_async(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                               int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks,
                               int64_t n_dec, void* k_cache, void* v_cache, const kvmig_pool_shape* shape,
                               int64_t layer_begin, int64_t layer_end, void* stream, uint64_t* ticket) {
    if (!ticket) return fail(KVMIG_EINVAL, "ticket is NULL");
    return enqueue_migration(ctx_pp, ctx_tp, ctx_blocks, n_ctx, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks, n_dec,
                             k_cache, v_cache, shape, static_cast<cudaStream_t>(stream), ticket, layer_begin, layer_end);
}

int kvmig_migrate_wait(uint64_t ticket) { return wait_ticket(ticket); }

int kvmig_migrate_blocks(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                         int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks, int64_t n_dec,
                         void* k_cache, void* v_cache, const kvmig_pool_shape* shape, void* stream) {
    uint64_t ticket = 0;
    int rc = enqueue_migration(ctx_pp, ctx_tp, ctx_blocks, n_ctx, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks, n_dec,
                               k_cache, v_cache, shape, static_cast<cudaStream_t>(stream), &ticket);
    if (rc) return rc;
    return wait_ticket(ticket);
}

int kvmig_migrate_blocks_static(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                                int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks,
                                int64_t n_dec, void* k_cache, void* v_cache, const kvmig_pool_shape* shape, void* stream) {
    return migrate_static(ctx_pp, ctx_tp, ctx_blocks, n_ctx, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks, n_dec,
                          k_cache, v_cache, shape, static_cast<cudaStream_t>(stream));
}

int kvmig_swap(const int64_t* src_ids, int64_t n_src, const int64_t* dst_ids, int64_t n_dst, int is_swap_in, void* k_cache,
               void* v_cache, const kvmig_pool_shape* shape, void* k_swap, void* v_swap, int64_t num_cpu_blocks, void* stream_) {
    g_err.clear();
    int rc = check_shape(shape, "swap");
    if (rc) return rc;
    if (n_src < 0 || n_dst < 0) return fail(KVMIG_EINVAL, "negative list length");
    if (n_src != n_dst)
        return fail(KVMIG_EINVAL, "source_block_ids has %lld entries but target_block_ids has %lld", (long long)n_src, (long long)n_dst);
    if (n_src > 0 && (!src_ids || !dst_ids)) return fail(KVMIG_EINVAL, "block id list is NULL");
    if (!k_cache || !v_cache || !k_swap || !v_swap) return fail(KVMIG_EINVAL, "a pool pointer is NULL");
    if (num_cpu_blocks < 0) return fail(KVMIG_EINVAL, "num_cpu_blocks is negative");
    const int64_t src_limit = is_swap_in ? num_cpu_blocks : shape->num_blocks;
    const int64_t dst_limit = is_swap_in ? shape->num_blocks : num_cpu_blocks;
    for (int64_t i = 0; i < n_src; ++i) {
        if (src_ids[i] < 0 || src_ids[i] >= src_limit)
            return fail(KVMIG_EINVAL, "source_block_ids[%lld] = %lld is outside the %s pool (%lld blocks)", (long long)i,
                        (long long)src_ids[i], is_swap_in ? "host" : "GPU", (long long)src_limit);
        if (dst_ids[i] < 0 || dst_ids[i] >= dst_limit)
            return fail(KVMIG_EINVAL, "target_block_ids[%lld] = %lld is outside the %s pool (%lld blocks)", (long long)i,
                        (long long)dst_ids[i], is_swap_in ? "GPU" : "host", (long long)dst_limit);
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t bb = block_bytes(*shape);
    const cudaMemcpyKind kind = is_swap_in ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
    char* src_pool[2] = {static_cast<char*>(is_swap_in ? k_swap : k_cache), static_cast<char*>(is_swap_in ? v_swap : v_cache)};
    char* dst_pool[2] = {static_cast<char*>(is_swap_in ? k_cache : k_swap), static_cast<char*>(is_swap_in ? v_cache : v_swap)};
    // Consecutive ids on both sides are one contiguous span: issue one copy for the whole run.
    for (int64_t i = 0; i < n_src;) {
        int64_t j = i + 1;
        while (j < n_src && src_ids[j] == src_ids[j - 1] + 1 && dst_ids[j] == dst_ids[j - 1] + 1) ++j;
        for (int x = 0; x < 2; ++x) {
            CU_TRY(cudaMemcpyAsync(dst_pool[x] + dst_ids[i] * bb, src_pool[x] + src_ids[i] * bb, (size_t)((j - i) * bb), kind,
                                   stream));
            g_cnt.memcpy_calls++;
        }
        g_cnt.bytes_swapped += 2 * (j - i) * bb;
        i = j;
    }
    return 0;
}

static std::atomic<int64_t>* option_slot(const char* name) {
    if (!name) return nullptr;
    if (!std::strcmp(name, "kernel")) return &g_opt.kernel;
    if (!std::strcmp(name, "chunk_bytes")) return &g_opt.chunk_bytes;
    if (!std::strcmp(name, "stages")) return &g_opt.stages;
    if (!std::strcmp(name, "ctas_per_sm")) return &g_opt.ctas_per_sm;
    if (!std::strcmp(name, "inline_tables")) return &g_opt.inline_tables;
    if (!std::strcmp(name, "overlap_launches")) return &g_opt.overlap_launches;
    if (!std::strcmp(name, "max_ctas")) return &g_opt.max_ctas;
    if (!std::strcmp(name, "l2_hint")) return &g_opt.l2_hint;
    if (!std::strcmp(name, "dynamic_units")) return &g_opt.dynamic_units;
    if (!std::strcmp(name, "wait_limit_ms")) return &g_opt.wait_limit_ms;
    if (!std::strcmp(name, "lose_unit_plus1")) return &g_opt.lose_unit_plus1;
    return nullptr;
}

int kvmig_set_option(const char* name, int64_t value) {
    g_err.clear();
    std::atomic<int64_t>* s = option_slot(name);
    if (!s) return fail(KVMIG_EINVAL, "unknown option '%s'", name ? name : "(null)");
    if (value < 0) return fail(KVMIG_EINVAL, "option '%s' cannot be negative", name);
    if (s == &g_opt.kernel && value > 2) return fail(KVMIG_EINVAL, "kernel must be 0 (auto), 1 (vector) or 2 (bulk)");
    if (s == &g_opt.chunk_bytes && (value < 16 || value % 16 || value > (1 << 20)))
        return fail(KVMIG_EINVAL, "chunk_bytes must be a multiple of 16 in [16, 1 MiB]");
    s->store(value);
    return 0;
}

int64_t kvmig_get_option(const char* name) {
    std::atomic<int64_t>* s = option_slot(name);
    return s ? s->load() : -1;
}

int64_t kvmig_get_counter(const char* name) {
    if (!name) return -1;
    if (!std::strcmp(name, "kernel_launches")) return g_cnt.kernel_launches.load();
    if (!std::strcmp(name, "memcpy_calls")) return g_cnt.memcpy_calls.load();
    if (!std::strcmp(name, "bytes_migrated")) return g_cnt.bytes_migrated.load();
    if (!std::strcmp(name, "bytes_swapped")) return g_cnt.bytes_swapped.load();
    if (!std::strcmp(name, "mapped_peers")) return g_cnt.mapped_peers.load();
    return -1;
}

int kvmig_reset_registry(void) {
    g_err.clear();
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st;
    int rc = ensure_device(&st, nullptr);
    if (rc) return rc;
    st->registry.clear();
    return 0;
}

}  // extern "C"
