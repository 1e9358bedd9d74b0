// Paged-KV block migration and swap for B200 (sm_100a): the per-process registry of mapped
// context-stage pools, launch planning, and the C ABI declared in include/kvmig.h.  The kernels
// live in kvmig_kernels.cuh.
//
// The data path is a pure byte move.  A decoding-stage worker pulls, for each migrated block, the
// (layer range x KV-head range) rectangle it owns out of the context-stage workers' pools.  The
// host side
//   * keeps, per device, the registered context workers and their mapped pool addresses
//     (CUDA IPC for other processes, the raw address for pools of this process);
//   * turns a call into segments (contributing context worker x K/V pool), validates the block
//     lists, picks the kernel (bulk-copy pipeline when every run is 16-byte aligned, vector loads
//     otherwise) and its grid;
//   * hands out tickets backed by an event, a status word in mapped pinned memory and a pair of
//     work counters per launch; block tables of up to 1024 blocks ride in the kernel parameters,
//     longer ones go through a device table;
//   * lets a migration start before earlier ones have finished when its target blocks are
//     disjoint from theirs (programmatic dependent launch), and orders it after them otherwise.
#include "../../include/kvmig.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <string>
#include <tuple>
#include <vector>
#include <unistd.h>

#include "kvmig_kernels.cuh"

namespace kvmig {

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
    HW_DEVICE = 20, HW_NONCE = 21, HW_RESERVED1 = 22, HW_CHECK = 23
};

int64_t handle_checksum(const int64_t* w) {
    uint64_t h = 0x9e3779b97f4a7c15ULL;
    for (int i = 0; i < HW_CHECK; ++i) {
        h ^= (uint64_t)w[i] + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
    }
    return (int64_t)h;
}

// Defaults from sweeps on B200: 16 KiB chunks, a 3-stage ring and 2 CTAs per SM (96 KiB in flight per SM,
// 296 CTAs), CTAs drawing two consecutive units (32 KiB) per visit to the work counter.  With consecutive
// launches overlapping, same-GPU copies of OPT-13B-shaped blocks run at 6.8-6.9 TB/s for any setting from 64 to
// 192 KiB in flight per SM; awaited single calls, which pay their own ramp-up and tail, were fastest around
// 96 KiB.  Anything from 16 KiB in flight per SM upward saturates NVLink.  Calls that carry several requests
// (more than 256 blocks) run long enough to gain about 1 % from a fourth stage, so "stages" 0 means 3 or 4.
struct Options {
    std::atomic<int64_t> kernel{0}, chunk_bytes{16384}, stages{0}, ctas_per_sm{0}, inline_tables{1}, overlap_launches{1}, max_ctas{0}, l2_hint{0},
        dynamic_units{1}, wait_limit_ms{2000}, lose_unit_plus1{0}, unit_batch{0}, swap_wait{-1}, wait_mode{0};
};
Options g_opt;
std::atomic<uint64_t> g_option_gen{1};   // bumped by every kvmig_set_option

struct Counters {
    std::atomic<int64_t> kernel_launches{0}, memcpy_calls{0}, bytes_migrated{0}, bytes_swapped{0}, mapped_peers{0};
    // Host time of the migration entry points, by segment (nanoseconds, summed over calls): turning the arguments
    // into launch descriptors, checking the block ids, deciding whether the launch may overlap its predecessors,
    // filling the parameters and launching, and waiting for the kernel.
    std::atomic<int64_t> migrate_calls{0}, plan_cache_hits{0}, ns_prepare{0}, ns_validate{0}, ns_order{0}, ns_launch{0}, ns_wait{0};
};
Counters g_cnt;

inline int64_t now_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// A number drawn once per process.  It travels in every exported handle next to the pid: a handle is treated
// as "exported by this very process" only if both match, because two workers in different pid namespaces
// (containers) can carry the same pid.
int64_t process_nonce() {
    static const int64_t nonce = [] {
        std::random_device rd;
        uint64_t v = ((uint64_t)rd() << 32) ^ (uint64_t)rd() ^ ((uint64_t)now_ns() << 1) ^ ((uint64_t)getpid() << 40);
        v &= 0x7fffffffffffffffULL;
        return (int64_t)(v ? v : 1);
    }();
    return nonce;
}

inline bool exported_by_this_process(const int64_t* w);

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

struct Range {
    const char* p = nullptr;
    size_t n = 0;
    bool meets(const Range& o) const { return n && o.n && p < o.p + o.n && o.p < p + n; }
};

constexpr int kMaxReadRanges = 64;

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
    // What the launch in flight touches, for the ordering decision of later launches: the stream it runs on,
    // the two pools it writes and the context pools it reads (reads_all: too many to list, assume everything).
    cudaStream_t stream = nullptr;
    Range writes[2];
    Range reads[kMaxReadRanges];
    int n_reads = 0;
    bool reads_all = false;
};

struct Assembly {
    std::vector<Seg> segs;             // two per contributing context worker: K pool, V pool
    uintptr_t align_bits = 0;          // OR of every address, stride and run length
    int64_t src_num_blocks = INT64_MAX;
    std::vector<Range> reads;          // the context pools those segments read
};

struct LaunchShape {
    int64_t kernel = 0;        // 1 vector loads, 2 bulk-copy pipeline
    int vec = 16;              // widest vector every address and length allows
    int64_t stages = 0, chunk = 0, ctas_per_sm = 0;
    size_t smem = 0;
    int64_t stages_long = 0;   // ring depth and shared memory for calls of more than kInlineSmall blocks
    size_t smem_long = 0;

    // The shape to launch a call of n blocks with.
    LaunchShape for_blocks(int64_t n, int64_t long_from) const {
        LaunchShape out = *this;
        if (n > long_from && stages_long > 0) {
            out.stages = stages_long;
            out.smem = smem_long;
        }
        return out;
    }
};

// Everything about a call that does not depend on its block lists.  A worker migrates request after request
// with the same stage layouts, pools and options, so the result of planning is kept and reused until one of
// them changes.
struct Prepared {
    bool valid = false;
    int64_t key[10] = {};
    kvmig_pool_shape shape = {};
    const void* k = nullptr;
    const void* v = nullptr;
    uint64_t registry_gen = 0, option_gen = 0;
    bool nothing_to_move = false;      // the layer window misses this worker
    Assembly as;
    LaunchShape ls;
};

struct DeviceState {
    bool inited = false;
    int sm_count = 0;
    int max_smem_optin = 0;
    std::map<CtxKey, CtxEntry> registry;
    uint64_t registry_gen = 1;           // bumped whenever the registry changes
    std::map<std::array<int64_t, 8>, char*> ipc_bases;   // opened IPC allocations
    Slot slots[KVMIG_MAX_INFLIGHT];
    uint64_t next_seq = 1;
    int sticky_error = 0;
    std::string sticky_text;
    int bulk_smem_set = 0;
    // Per destination pool (keyed by the K pool's address): ticket sequence of the last launch that wrote
    // each block, used to decide whether a new launch may overlap the launches still in flight.
    std::map<const void*, std::vector<uint64_t>> last_writer;
    const void* marks_pool = nullptr;            // the pool looked up last, and its marks
    std::vector<uint64_t>* marks = nullptr;
    std::vector<char> seen;   // duplicate-target bitmap, all zero between calls
    Prepared prepared;        // planning result of the previous ticketed call
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

inline bool exported_by_this_process(const int64_t* w) {
    return w[HW_PID] == (int64_t)getpid() && w[HW_NONCE] == process_nonce();
}

// Resolve an exported pool to an address usable on the current device.
int map_pool(DeviceState& st, int dev, const int64_t* w, char** out) {
    if (exported_by_this_process(w)) {
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

// KV heads a worker of a tp-way stage holds: H/tp — or the single head of a multi-query model, which every
// tensor-parallel rank holds in full (distserve/config.py:233-237 returns 1 whatever the parallel config).
inline int64_t local_heads(int64_t H, int64_t tp) { return H == 1 ? 1 : H / tp; }

// Which context workers feed decoding worker (t_d, p_d), and with which sub-rectangles.
// Worker (tp, t, pp, p) owns layers [p*L/pp, (p+1)*L/pp) and heads [t*H/tp, (t+1)*H/tp)
// (distserve/config.py:244-257,279-286).  With a single KV head every rank holds head 0; decoding rank t_d then
// reads it from context rank floor(t_d * ctx_tp / dec_tp), which spreads the readers over the replicas.
int plan_segments(int64_t L, int64_t H, int64_t ctx_tp, int64_t ctx_pp, int64_t dec_tp, int64_t t_d, int64_t dec_pp,
                  int64_t p_d, std::vector<SegPlan>* out) {
    if (L <= 0 || H <= 0) return fail(KVMIG_EINVAL, "num_layers and num_heads must be positive");
    if (ctx_tp <= 0 || ctx_pp <= 0 || dec_tp <= 0 || dec_pp <= 0) return fail(KVMIG_EINVAL, "parallel sizes must be positive");
    if (L % ctx_pp || L % dec_pp)
        return fail(KVMIG_EINVAL, "num_layers %lld is not divisible by the pipeline-parallel sizes (%lld, %lld)", (long long)L,
                    (long long)ctx_pp, (long long)dec_pp);
    const bool replicated = H == 1;
    if (!replicated && (H % ctx_tp || H % dec_tp))
        return fail(KVMIG_EINVAL, "num_heads %lld is not divisible by the tensor-parallel sizes (%lld, %lld)", (long long)H,
                    (long long)ctx_tp, (long long)dec_tp);
    if (t_d < 0 || t_d >= dec_tp || p_d < 0 || p_d >= dec_pp) return fail(KVMIG_EINVAL, "decoding rank out of range");
    const int64_t Ld = L / dec_pp, Hd = local_heads(H, dec_tp), Lc = L / ctx_pp, Hc = local_heads(H, ctx_tp);
    const int64_t gl0 = p_d * Ld, gl1 = gl0 + Ld, gh0 = replicated ? 0 : t_d * Hd, gh1 = gh0 + Hd;
    out->clear();
    for (int64_t p = gl0 / Lc; p * Lc < gl1; ++p) {
        int64_t la = std::max(gl0, p * Lc), lb = std::min(gl1, (p + 1) * Lc);
        if (replicated) {
            SegPlan s;
            s.ctx = CtxKey{ctx_tp, ctx_pp, p, t_d * ctx_tp / dec_tp};
            s.src_layer_off = la - p * Lc; s.dst_layer_off = la - gl0; s.n_layers = lb - la;
            s.src_head_off = 0; s.dst_head_off = 0; s.n_heads = 1;
            out->push_back(s);
            continue;
        }
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

// The model's global KV-head count, which the migrate call does not carry: heads held locally x dec_tp — unless
// the registered context stage says the model has a single KV head, which every rank then holds.
int64_t global_heads(const DeviceState& st, const kvmig_pool_shape* shape, int64_t ctx_tp, int64_t ctx_pp, int64_t dec_tp) {
    if (shape->num_heads == 1 && dec_tp > 1)
        for (const auto& kv : st.registry)
            if (kv.first.tp == ctx_tp && kv.first.pp == ctx_pp) return kv.second.H == 1 ? 1 : shape->num_heads * dec_tp;
    return shape->num_heads * dec_tp;
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

// ---- pieces shared by every migration entry point ---------------------------------------------

int check_lists(const char* what, const kvmig_pool_shape* shape, const int64_t* ctx_blocks, int64_t n_ctx,
                const int64_t* dec_blocks, int64_t n_dec, const void* k_cache, const void* v_cache) {
    int rc = check_shape(shape, what);
    if (rc) return rc;
    if (n_ctx < 0 || n_dec < 0) return fail(KVMIG_EINVAL, "negative list length");
    if (n_ctx != n_dec)
        return fail(KVMIG_EINVAL, "context_block_indexes has %lld entries but decoding_block_indexes has %lld",
                    (long long)n_ctx, (long long)n_dec);
    if (n_ctx > 0 && (!ctx_blocks || !dec_blocks)) return fail(KVMIG_EINVAL, "block index list is NULL");
    if (!k_cache || !v_cache) return fail(KVMIG_EINVAL, "k_cache / v_cache is NULL");
    return 0;
}

// Keep only the part of each planned overlap that lies inside the window of global layers.
void clip_to_layers(std::vector<SegPlan>* plan, int64_t first_layer, int64_t layer_begin, int64_t layer_end) {
    std::vector<SegPlan> clipped;
    for (SegPlan sp : *plan) {
        const int64_t g0 = first_layer + sp.dst_layer_off, g1 = g0 + sp.n_layers;
        const int64_t a = std::max(g0, layer_begin), b = std::min(g1, layer_end);
        if (a >= b) continue;
        sp.src_layer_off += a - g0;
        sp.dst_layer_off += a - g0;
        sp.n_layers = b - a;
        clipped.push_back(sp);
    }
    plan->swap(clipped);
}


// Turn the planned overlaps into strided-copy descriptors over the registered (mapped) context pools.
// With map_missing a registered-but-unmapped pool is mapped now; without, that is an error (mapping
// reserves address space, which the allocation-free entry point must not do).
int assemble_segments(DeviceState& st, int dev, const std::vector<SegPlan>& plan, int64_t L, int64_t H, int64_t ctx_tp,
                      int64_t ctx_pp, const kvmig_pool_shape* shape, void* k_cache, void* v_cache, bool map_missing,
                      Assembly* out) {
    const int64_t slab = shape->block_size * shape->head_dim * shape->elem_size;
    const int64_t Lc = L / ctx_pp, Hc = local_heads(H, ctx_tp);
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
            if (!map_missing)
                return fail(KVMIG_ENOTREG,
                            "context worker (pp_rank %lld, tp_rank %lld) was registered for another decoding rank and is not "
                            "mapped; register it with this worker's parallel config first",
                            (long long)sp.ctx.pp_rank, (long long)sp.ctx.tp_rank);
            int rc = map_pool(st, dev, ce.hk.data(), &ce.k);
            if (rc) return rc;
            rc = map_pool(st, dev, ce.hv.data(), &ce.v);
            if (rc) return rc;
            ce.mapped = true;
        }
        out->src_num_blocks = std::min(out->src_num_blocks, std::min(ce.hk[HW_NB], ce.hv[HW_NB]));
        out->reads.push_back(Range{ce.k, (size_t)ce.hk[HW_BYTES]});
        out->reads.push_back(Range{ce.v, (size_t)ce.hv[HW_BYTES]});
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
            out->align_bits |= (uintptr_t)g.src | (uintptr_t)g.dst | g.src_block_stride | g.dst_block_stride |
                               g.src_row_stride | g.dst_row_stride | g.run_bytes;
            out->segs.push_back(g);
        }
    }
    return 0;
}

// Ids in range on both sides, no target named twice.  `st.seen` is a bitmap kept all-zero between calls.
int validate_ids(DeviceState& st, const int64_t* ctx_blocks, const int64_t* dec_blocks, int64_t n, int64_t src_num_blocks,
                 int64_t dst_num_blocks) {
    std::vector<char>& seen = st.seen;
    if ((int64_t)seen.size() < dst_num_blocks) seen.resize((size_t)dst_num_blocks, 0);
    int64_t checked = 0;
    int rc = 0;
    for (; checked < n && !rc; ++checked) {
        const int64_t i = checked;
        if (ctx_blocks[i] < 0 || ctx_blocks[i] >= src_num_blocks)
            rc = fail(KVMIG_EINVAL, "context_block_indexes[%lld] = %lld is outside the context pool (%lld blocks)", (long long)i,
                      (long long)ctx_blocks[i], (long long)src_num_blocks);
        else if (dec_blocks[i] < 0 || dec_blocks[i] >= dst_num_blocks)
            rc = fail(KVMIG_EINVAL, "decoding_block_indexes[%lld] = %lld is outside the decoding pool (%lld blocks)",
                      (long long)i, (long long)dec_blocks[i], (long long)dst_num_blocks);
        else if (seen[(size_t)dec_blocks[i]])
            rc = fail(KVMIG_EINVAL, "decoding_block_indexes names block %lld twice", (long long)dec_blocks[i]);
        else
            seen[(size_t)dec_blocks[i]] = 1;
    }
    for (int64_t i = 0; i < checked; ++i)
        if (dec_blocks[i] >= 0 && dec_blocks[i] < dst_num_blocks) seen[(size_t)dec_blocks[i]] = 0;
    return rc;
}


// Kernel, ring geometry and CTAs per SM from the options and the alignment of this call.
int shape_launch(DeviceState& st, uintptr_t align_bits, LaunchShape* ls) {
    ls->vec = pick_vec(align_bits);
    ls->kernel = g_opt.kernel.load();
    if (ls->kernel == 0) ls->kernel = (ls->vec == 16) ? 2 : 1;
    if (ls->kernel == 2 && ls->vec != 16)
        return fail(KVMIG_EINVAL, "the bulk-copy kernel needs 16-byte aligned runs; this shape gives %d", ls->vec);
    // "stages" 0 = automatic: 3, and one more for calls of more than kInlineSmall blocks (several requests in one
    // launch), which run long enough to gain from a third more bytes in flight; a positive value is used for every call.
    const int64_t asked = g_opt.stages.load();
    ls->stages = asked > 0 ? std::min<int64_t>(std::max<int64_t>(asked, 2), kMaxStages) : 3;
    ls->stages_long = asked > 0 ? ls->stages : 4;
    ls->chunk = g_opt.chunk_bytes.load();
    if (ls->chunk < 16 || ls->chunk % 16) return fail(KVMIG_EINVAL, "chunk_bytes must be a positive multiple of 16");
    ls->ctas_per_sm = g_opt.ctas_per_sm.load();
    if (ls->kernel == 2) {
        ls->smem = (size_t)ls->stages * ls->chunk + (size_t)ls->stages * (8 + 8 + 4 + 4) + 16;
        ls->smem_long = (size_t)ls->stages_long * ls->chunk + (size_t)ls->stages_long * (8 + 8 + 4 + 4) + 16;
        if ((int64_t)ls->smem > st.max_smem_optin)
            return fail(KVMIG_ELIMIT, "stages x chunk_bytes = %zu B exceeds the %d B of shared memory a CTA may use", ls->smem,
                        st.max_smem_optin);
        if ((int64_t)ls->smem_long > st.max_smem_optin) {   // the extra stage does not fit: long calls keep the base ring
            ls->stages_long = ls->stages;
            ls->smem_long = ls->smem;
        }
        if (ls->ctas_per_sm <= 0) {
            const int64_t ring = ls->stages * ls->chunk, target = 96 * 1024;   // bytes in flight per SM
            ls->ctas_per_sm = std::max<int64_t>(1, std::min<int64_t>(8, (target + ring - 1) / ring));
            ls->ctas_per_sm = std::min<int64_t>(ls->ctas_per_sm, std::max<int64_t>(1, (220 * 1024) / (int64_t)(ls->smem + 1024)));
        }
        if ((int)std::max(ls->smem, ls->smem_long) > st.bulk_smem_set) {
            const int bytes = (int)std::max(ls->smem, ls->smem_long);
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk_inline<kInlineSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
            CU_TRY(cudaFuncSetAttribute(kv_migrate_bulk_inline<kInlineLarge>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
            st.bulk_smem_set = bytes;
        }
    } else if (ls->ctas_per_sm <= 0) {
        ls->ctas_per_sm = 8;
    }
    return 0;
}

// Fill the descriptors of one launch (at most kMaxSegs segments); returns the work units per block.
unsigned fill_launch(MigParams* p, const Seg* segs, unsigned nseg, const LaunchShape& ls, int* status, int64_t* bytes_per_block) {
    std::memset(p, 0, sizeof *p);
    p->nseg = nseg;
    unsigned upb = 0;
    for (unsigned s = 0; s < nseg; ++s) {
        Seg g = segs[s];
        g.chunks_per_run = (unsigned)((g.run_bytes + ls.chunk - 1) / ls.chunk);
        g.units_per_block = g.rows * g.chunks_per_run;
        g.unit_begin = upb;
        upb += g.units_per_block;
        p->seg[s] = g;
        *bytes_per_block += (int64_t)g.run_bytes * g.rows;
    }
    p->status = status;
    p->units_per_block = upb;
    p->chunk_bytes = (unsigned)ls.chunk;
    p->batch = 1;
    p->l2_hint = (unsigned)g_opt.l2_hint.load();
    p->wait_limit_ns = (unsigned long long)std::max<int64_t>(1, g_opt.wait_limit_ms.load()) * 1000000ULL;
    p->lose_unit_plus1 = (unsigned)g_opt.lose_unit_plus1.load();
    return upb;
}

unsigned grid_for(const DeviceState& st, const LaunchShape& ls, unsigned total_units) {
    unsigned grid = (unsigned)std::min<int64_t>(total_units, (int64_t)st.sm_count * ls.ctas_per_sm);
    // A cap on the grid leaves whole SMs to a decode step running beside the migration.
    if (const int64_t cap = g_opt.max_ctas.load(); cap > 0) grid = (unsigned)std::min<int64_t>(grid, cap);
    return grid;
}

template <int NIDS>
cudaError_t launch_bulk_inline(const MigParams& p, const int64_t* src, const int64_t* dst, unsigned grid, const LaunchShape& ls,
                               cudaStream_t stream, bool overlap) {
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
    cfg.dynamicSmemBytes = ls.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kv_migrate_bulk_inline<NIDS>, q, (unsigned)ls.stages, (unsigned)ls.chunk);
}

template <int VEC>
cudaError_t launch_vec(const MigParams& p, unsigned grid, cudaStream_t stream) {
    kv_migrate_vec<VEC><<<grid, kVecThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

// Launch with the block tables in device memory (p.src_ids / p.dst_ids), ordinary stream order.
cudaError_t launch_device_tables(const MigParams& p, unsigned grid, const LaunchShape& ls, cudaStream_t stream) {
    if (ls.kernel == 2) {
        kv_migrate_bulk<<<grid, 32, ls.smem, stream>>>(p, (unsigned)ls.stages, (unsigned)ls.chunk);
        return cudaGetLastError();
    }
    switch (ls.vec) {
        case 16: return launch_vec<16>(p, grid, stream);
        case 8: return launch_vec<8>(p, grid, stream);
        case 4: return launch_vec<4>(p, grid, stream);
        case 2: return launch_vec<2>(p, grid, stream);
        default: return launch_vec<1>(p, grid, stream);
    }
}

// ---- the ticketed entry point (awaited and asynchronous calls, optional layer window) ----------

// Is the launch that occupies `sl` still executing?  `cache` holds one answer per slot for the current call
// (-1 not asked yet), so that a slot's event is queried at most once.
bool slot_running(DeviceState& st, int si, int* cache) {
    if (cache[si] < 0) {
        cache[si] = cudaEventQuery(st.slots[si].done) == cudaSuccess ? 0 : 1;
        (void)cudaGetLastError();   // "not ready" is reported through the error state
    }
    return cache[si] == 1;
}

int enqueue_migration(int64_t ctx_pp, int64_t ctx_tp, const int64_t* ctx_blocks, int64_t n_ctx, int64_t dec_pp,
                      int64_t dec_tp, int64_t dec_pp_rank, int64_t dec_tp_rank, const int64_t* dec_blocks, int64_t n_dec,
                      void* k_cache, void* v_cache, const kvmig_pool_shape* shape, cudaStream_t stream, uint64_t* ticket,
                      int64_t layer_begin = 0, int64_t layer_end = INT64_MAX) {
    const int64_t t_begin = now_ns();
    g_err.clear();
    if (ticket) *ticket = 0;
    int rc = check_lists("migrate_blocks", shape, ctx_blocks, n_ctx, dec_blocks, n_dec, k_cache, v_cache);
    if (rc) return rc;

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* stp;
    int dev;
    rc = ensure_device(&stp, &dev);
    if (rc) return rc;
    DeviceState& st = *stp;
    g_cnt.migrate_calls++;

    // Planning, segment assembly and kernel geometry depend only on the layouts, the pools, the registry and the
    // options: reuse the previous call's when none of them changed.
    Prepared& pr = st.prepared;
    const int64_t key[10] = {ctx_pp, ctx_tp, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, layer_begin, layer_end, 0, 0};
    const uint64_t option_gen = g_option_gen.load();
    if (pr.valid && std::memcmp(pr.key, key, sizeof key) == 0 && std::memcmp(&pr.shape, shape, sizeof *shape) == 0 &&
        pr.k == k_cache && pr.v == v_cache && pr.registry_gen == st.registry_gen && pr.option_gen == option_gen) {
        g_cnt.plan_cache_hits++;
    } else {
        pr.valid = false;
        const int64_t L = shape->num_layers * dec_pp, H = global_heads(st, shape, ctx_tp, ctx_pp, dec_tp);
        std::vector<SegPlan> plan;
        rc = plan_segments(L, H, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank, &plan);
        if (rc) return rc;
        if (layer_begin < 0 || layer_end < layer_begin)
            return fail(KVMIG_EINVAL, "layer window [%lld, %lld) is not a range", (long long)layer_begin, (long long)layer_end);
        const int64_t window_end = std::min(layer_end, L);
        if (layer_begin > 0 || window_end < L) clip_to_layers(&plan, dec_pp_rank * shape->num_layers, layer_begin, window_end);
        pr.as = Assembly();
        rc = assemble_segments(st, dev, plan, L, H, ctx_tp, ctx_pp, shape, k_cache, v_cache, /*map_missing=*/true, &pr.as);
        if (rc) return rc;
        pr.nothing_to_move = plan.empty();
        pr.ls = LaunchShape();
        if (!pr.nothing_to_move) {
            rc = shape_launch(st, pr.as.align_bits, &pr.ls);
            if (rc) return rc;
        }
        std::memcpy(pr.key, key, sizeof key);
        pr.shape = *shape;
        pr.k = k_cache;
        pr.v = v_cache;
        pr.registry_gen = st.registry_gen;
        pr.option_gen = option_gen;
        pr.valid = true;
    }
    const Assembly& as = pr.as;
    const LaunchShape ls = pr.ls.for_blocks(n_ctx, kInlineSmall);
    const int64_t t_prepared = now_ns();
    g_cnt.ns_prepare += t_prepared - t_begin;

    rc = validate_ids(st, ctx_blocks, dec_blocks, n_ctx, as.src_num_blocks, shape->num_blocks);
    const int64_t t_validated = now_ns();
    g_cnt.ns_validate += t_validated - t_prepared;
    if (rc) return rc;
    if (n_ctx == 0 || pr.nothing_to_move) return 0;   // nothing to move (empty lists, or the window misses this worker)

    // Ticket slot.
    uint64_t seq = st.next_seq++;
    Slot& sl = st.slots[seq % KVMIG_MAX_INFLIGHT];
    rc = retire_slot(st, sl);
    if (rc && !st.sticky_error) { st.sticky_error = rc; st.sticky_text = g_err; }
    // Tables of a typical request ride in the kernel parameters; longer lists go through device memory.
    const bool inline_tables = ls.kernel == 2 && g_opt.inline_tables.load() != 0 && n_ctx <= kInlineLarge;
    rc = grow_slot(sl, inline_tables ? 0 : n_ctx);
    if (rc) return rc;
    sl.status[0] = sl.status[1] = sl.status[2] = sl.status[3] = 0;

    // ---- ordering against the migrations still in flight ------------------------------------------------
    // A launch may begin before earlier ones have finished (programmatic dependent launch) only if it is
    // independent of every one of them that is still executing:
    //   * it reads no pool that one of them writes and writes no pool that one of them reads;
    //   * where it writes a pool one of them writes, it writes other blocks, or other layers of the same blocks.
    // Otherwise the grid waits for its predecessor in the stream before it touches memory (grids complete in
    // stream order, so that covers every earlier launch on the stream), and a conflicting launch on another
    // stream is waited for through its event.
    const int64_t window_end = std::min<int64_t>(layer_end, shape->num_layers * dec_pp);
    const bool overlap = inline_tables && g_opt.overlap_launches.load() != 0;
    bool depends = !overlap;
    bool cross_stream_wait = false;
    int running[KVMIG_MAX_INFLIGHT];
    for (int& r : running) r = -1;
    bool event_awaited[KVMIG_MAX_INFLIGHT] = {};   // slots whose event this stream has already been told to wait for
    const Range my_writes[2] = {Range{static_cast<const char*>(k_cache), (size_t)(shape->num_blocks * block_bytes(*shape))},
                                Range{static_cast<const char*>(v_cache), (size_t)(shape->num_blocks * block_bytes(*shape))}};
    auto must_follow = [&](int si) -> int {
        // The launch in slot si conflicts with this one: order this one after it.
        Slot& other = st.slots[si];
        if (!slot_running(st, si, running)) return 0;
        depends = true;
        if (other.stream != stream && !event_awaited[si]) {
            CU_TRY(cudaStreamWaitEvent(stream, other.done, 0));
            event_awaited[si] = true;
            cross_stream_wait = true;
        }
        return 0;
    };
    bool newest_known = false, other_streams = false;
    uint64_t newest_seq = 0;
    int newest_slot = -1;
    for (int si = 0; si < KVMIG_MAX_INFLIGHT; ++si) {
        Slot& other = st.slots[si];
        if (!other.busy || &other == &sl) continue;
        if (other.stream != stream) other_streams = true;
        if (other.stream == stream && other.seq > newest_seq) { newest_seq = other.seq; newest_slot = si; newest_known = true; }
        bool conflict = false;
        for (int x = 0; x < 2 && !conflict; ++x) {
            // same destination pools: decided per block and layer window below
            if (other.writes[x].p == my_writes[x].p && other.writes[x].n == my_writes[x].n) continue;
            for (int y = 0; y < 2 && !conflict; ++y) conflict = other.writes[x].meets(my_writes[y]);
        }
        if (!conflict && other.reads_all) conflict = true;
        for (int r = 0; r < other.n_reads && !conflict; ++r)
            conflict = other.reads[r].meets(my_writes[0]) || other.reads[r].meets(my_writes[1]);
        for (size_t r = 0; r < as.reads.size() && !conflict; ++r)
            conflict = as.reads[r].meets(other.writes[0]) || as.reads[r].meets(other.writes[1]);
        if (conflict && (rc = must_follow(si))) return rc;
    }
    {
        if (st.marks_pool != k_cache || !st.marks) {
            st.marks = &st.last_writer[k_cache];
            st.marks_pool = k_cache;
        }
        std::vector<uint64_t>& marks = *st.marks;
        if ((int64_t)marks.size() < shape->num_blocks) marks.resize((size_t)shape->num_blocks, 0);
        bool hidden_writers = false;   // a block's mark names a launch on other layers: an older writer may hide behind it
        for (int64_t i = 0; i < n_ctx; ++i) {
            uint64_t& m = marks[(size_t)dec_blocks[i]];
            if (m != 0 && (!depends || other_streams)) {
                const int si = (int)(m % KVMIG_MAX_INFLIGHT);
                Slot& other = st.slots[si];
                if (other.seq == m && other.busy) {
                    if (other.layer0 < window_end && layer_begin < other.layer1) {
                        if ((rc = must_follow(si))) return rc;
                    } else {
                        hidden_writers = true;
                    }
                }
            }
            m = seq;
        }
        if (hidden_writers && (!depends || other_streams)) {
            // Marks keep one launch per block.  Behind a launch on other layers there may be an older one on
            // these layers that is still running: look at every launch into this pool whose window meets ours.
            for (int si = 0; si < KVMIG_MAX_INFLIGHT; ++si) {
                Slot& other = st.slots[si];
                if (!other.busy || &other == &sl || other.writes[0].p != my_writes[0].p) continue;
                if (other.layer0 < window_end && layer_begin < other.layer1 && (rc = must_follow(si))) return rc;
            }
        }
    }
    // Starting early is only meaningful behind a migration of this library that is still executing.  Behind
    // anything else (a producer that filled the source pool, a decode step) the grid waits for its predecessor
    // before it touches memory, which is what makes that kernel's writes visible to it.
    if (!depends && (!newest_known || !slot_running(st, newest_slot, running))) depends = true;
    const bool launch_overlapped = overlap && !cross_stream_wait;
    const int64_t t_ordered = now_ns();
    g_cnt.ns_order += t_ordered - t_validated;

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
    for (size_t s0 = 0; s0 < as.segs.size(); s0 += kMaxSegs) {
        MigParams p;
        const unsigned nseg = (unsigned)std::min<size_t>(kMaxSegs, as.segs.size() - s0);
        const unsigned upb = fill_launch(&p, as.segs.data() + s0, nseg, ls, sl.status_dev, &bytes_per_block);
        p.wait_prior = depends ? 1u : 0u;
        // total_units is 32-bit: walk the block list in slices if a launch would overflow.
        const int64_t max_blocks = std::max<int64_t>(1, (int64_t)0x7fffffff / upb);
        for (int64_t b0 = 0; b0 < n_ctx; b0 += max_blocks) {
            const int64_t nb = std::min(max_blocks, n_ctx - b0);
            p.src_ids = inline_tables ? nullptr : sl.d_tab + b0;
            p.dst_ids = inline_tables ? nullptr : sl.d_tab + n_ctx + b0;
            p.n_blocks = (unsigned)nb;
            p.total_units = (unsigned)(nb * upb);
            const unsigned grid = grid_for(st, ls, p.total_units);
            // Each launch of this call gets its own counter pair (launches of one call may overlap).  A short
            // launch keeps the fixed deal: the counter's latency would be most of its run time.
            p.work = nullptr;
            p.batch = 1;
            if (ls.kernel == 2 && g_opt.dynamic_units.load() != 0 && launch_index < kWorkPairs && p.total_units >= 4u * grid) {
                p.work = sl.work + 2 * launch_index;
                p.batch = p.total_units >= 8u * grid ? 2u : 1u;
                if (const int64_t fixed = g_opt.unit_batch.load(); fixed > 0) p.batch = (unsigned)fixed;
            }
            ++launch_index;
            cudaError_t e;
            if (inline_tables)
                e = nb <= kInlineSmall
                        ? launch_bulk_inline<kInlineSmall>(p, ctx_blocks + b0, dec_blocks + b0, grid, ls, stream, launch_overlapped)
                        : launch_bulk_inline<kInlineLarge>(p, ctx_blocks + b0, dec_blocks + b0, grid, ls, stream, launch_overlapped);
            else
                e = launch_device_tables(p, grid, ls, stream);
            if (e != cudaSuccess) return fail(KVMIG_ECUDA, "launching the migration kernel: %s", cudaGetErrorString(e));
            g_cnt.kernel_launches++;
        }
    }
    CU_TRY(cudaEventRecord(sl.done, stream));
    sl.busy = true;
    sl.seq = seq;
    sl.layer0 = layer_begin;
    sl.layer1 = window_end;
    sl.bytes = bytes_per_block * n_ctx;
    sl.stream = stream;
    sl.writes[0] = my_writes[0];
    sl.writes[1] = my_writes[1];
    sl.reads_all = as.reads.size() > (size_t)kMaxReadRanges;
    sl.n_reads = sl.reads_all ? 0 : (int)as.reads.size();
    for (int r = 0; r < sl.n_reads; ++r) sl.reads[r] = as.reads[r];
    if (ticket) *ticket = ((uint64_t)(unsigned)dev << 48) | seq;
    g_cnt.ns_launch += now_ns() - t_ordered;
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
        const int64_t t0 = now_ns();
        cudaError_t e;
        if (g_opt.wait_mode.load() == 1) {
            // Busy-poll the event from this thread instead of leaving the kind of wait to the device's scheduling flag.
            while ((e = cudaEventQuery(done)) == cudaErrorNotReady) {}
            if (e != cudaSuccess) (void)cudaGetLastError();
        } else {
            e = cudaEventSynchronize(done);
        }
        g_cnt.ns_wait += now_ns() - t0;
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
    int rc = check_lists("migrate_blocks_static", shape, ctx_blocks, n_ctx, dec_blocks, n_dec, k_cache, v_cache);
    if (rc) return rc;
    if (n_ctx > KVMIG_STATIC_MAX_BLOCKS)
        return fail(KVMIG_ELIMIT,
                    "%lld blocks in one call exceed the %d the built-in scratch holds; split the lists or use "
                    "kvmig_migrate_blocks",
                    (long long)n_ctx, KVMIG_STATIC_MAX_BLOCKS);

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* stp;
    int dev;
    rc = ensure_device(&stp, &dev);
    if (rc) return rc;
    DeviceState& st = *stp;
    int* scratch = nullptr;
    rc = static_scratch_for_current_device(dev, &scratch);
    if (rc) return rc;

    const int64_t L = shape->num_layers * dec_pp, H = global_heads(st, shape, ctx_tp, ctx_pp, dec_tp);
    std::vector<SegPlan> plan;
    rc = plan_segments(L, H, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank, &plan);
    if (rc) return rc;
    if (plan.size() * 2 > (size_t)kMaxSegs)
        return fail(KVMIG_ELIMIT, "this reshard needs %zu segments; the allocation-free entry point takes %d", plan.size() * 2,
                    kMaxSegs);
    Assembly as;
    rc = assemble_segments(st, dev, plan, L, H, ctx_tp, ctx_pp, shape, k_cache, v_cache, /*map_missing=*/false, &as);
    if (rc) return rc;
    rc = validate_ids(st, ctx_blocks, dec_blocks, n_ctx, as.src_num_blocks, shape->num_blocks);
    if (rc) return rc;
    if (n_ctx == 0) return 0;
    LaunchShape base;
    rc = shape_launch(st, as.align_bits, &base);
    if (rc) return rc;
    const LaunchShape ls = base.for_blocks(n_ctx, kInlineSmall);

    MigParams p;
    int64_t bytes_per_block = 0;
    const unsigned upb = fill_launch(&p, as.segs.data(), (unsigned)as.segs.size(), ls, scratch, &bytes_per_block);
    if ((int64_t)upb * n_ctx > 0x7fffffff) return fail(KVMIG_ELIMIT, "too many work units for one launch; lower the block count");

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
    p.n_blocks = (unsigned)n_ctx;
    p.total_units = (unsigned)(n_ctx * upb);
    cudaError_t e = launch_device_tables(p, grid_for(st, ls, p.total_units), ls, stream);
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
    w[HW_NONCE] = process_nonce();
    w[HW_PTR] = (int64_t)(uintptr_t)pool;
    w[HW_NB] = shape->num_blocks; w[HW_NL] = shape->num_layers; w[HW_NH] = shape->num_heads;
    w[HW_BS] = shape->block_size; w[HW_HD] = shape->head_dim; w[HW_ES] = shape->elem_size;
    w[HW_DEVICE] = attr.device;
    w[HW_CHECK] = handle_checksum(w);
    return 0;
}

int kvmig_handle_is_local(const int64_t* handle, int64_t len) {
    g_err.clear();
    int rc = validate_handle(handle, len, "pool");
    if (rc) return rc;
    return exported_by_this_process(handle) ? 1 : 0;
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
    if (sk.num_layers != num_layers / ctx_pp || sk.num_heads != local_heads(num_heads, ctx_tp))
        return fail(KVMIG_EINVAL,
                    "exported pool holds %lld layers x %lld heads, but a tp=%lld,pp=%lld worker of a %lld-layer %lld-head model "
                    "holds %lld x %lld",
                    (long long)sk.num_layers, (long long)sk.num_heads, (long long)ctx_tp, (long long)ctx_pp,
                    (long long)num_layers, (long long)num_heads, (long long)(num_layers / ctx_pp),
                    (long long)local_heads(num_heads, ctx_tp));

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
    stp->registry_gen++;
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
    // "swap_wait": -1 until first use, then taken from the environment unless the option was set explicitly.
    int64_t swap_wait = g_opt.swap_wait.load();
    if (swap_wait < 0) {
        const char* env = std::getenv("KVMIG_SWAP_WAIT");
        swap_wait = (env && env[0] && env[0] != '0') ? 1 : 0;
        g_opt.swap_wait.store(swap_wait);
    }
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
    if (swap_wait && n_src > 0) CU_TRY(cudaStreamSynchronize(stream));
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
    if (!std::strcmp(name, "unit_batch")) return &g_opt.unit_batch;
    if (!std::strcmp(name, "lose_unit_plus1")) return &g_opt.lose_unit_plus1;
    if (!std::strcmp(name, "swap_wait")) return &g_opt.swap_wait;
    if (!std::strcmp(name, "wait_mode")) return &g_opt.wait_mode;
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
    g_option_gen++;
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
    if (!std::strcmp(name, "migrate_calls")) return g_cnt.migrate_calls.load();
    if (!std::strcmp(name, "plan_cache_hits")) return g_cnt.plan_cache_hits.load();
    if (!std::strcmp(name, "ns_prepare")) return g_cnt.ns_prepare.load();
    if (!std::strcmp(name, "ns_validate")) return g_cnt.ns_validate.load();
    if (!std::strcmp(name, "ns_order")) return g_cnt.ns_order.load();
    if (!std::strcmp(name, "ns_launch")) return g_cnt.ns_launch.load();
    if (!std::strcmp(name, "ns_wait")) return g_cnt.ns_wait.load();
    return -1;
}

int kvmig_reset_registry(void) {
    g_err.clear();
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st;
    int rc = ensure_device(&st, nullptr);
    if (rc) return rc;
    st->registry.clear();
    st->registry_gen++;
    return 0;
}

}  // extern "C"
