// Device code of the paged-KV block migration: work-unit descriptors, the vector-load kernel and the
// bulk-copy (cp.async.bulk + mbarrier) pipeline kernel.  Included by kvmig.cu only.
//
// A migration call decomposes into "segments" (one per contributing context worker and per K/V pool),
// each a 2-D strided copy per block: `rows` runs of `run_bytes` contiguous bytes.  Runs are cut into
// chunks; one chunk is the unit of work.  Units are numbered block-major, so units with neighbouring
// numbers touch neighbouring addresses.
#pragma once

#include <cuda_runtime.h>

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

// Shared memory: [stages * stage_bytes ring][stages mbarriers][stages dst ptr][stages sizes][stages unit numbers]
__device__ __forceinline__ void bulk_pipeline(const MigParams& p, const int* src_ids, const int* dst_ids,
                                              unsigned int stages, unsigned int stage_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    if (threadIdx.x != 0) return;
    unsigned char* ring = smem;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (size_t)stages * stage_bytes);
    char** dst_of = reinterpret_cast<char**>(bars + stages);
    unsigned int* bytes_of = reinterpret_cast<unsigned int*>(dst_of + stages);
    unsigned int* unit_of = bytes_of + stages;

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
        unit_of[s] = u;
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
            p.status[1] = (int)unit_of[s];   // the work unit (launch-wide number) whose load never signalled
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

}  // namespace kvmig
