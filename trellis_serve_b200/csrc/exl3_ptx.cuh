// Thin wrappers over the sm_90+/sm_100 PTX used by the kernels: mbarrier, 1-D bulk async copy (TMA engine,
// no multicast), warp-level MMA, named barriers.  Every wait is bounded: it returns false after a fixed number
// of polls instead of spinning forever, and the caller records the failure in the device error word.
#pragma once
#include <cstdint>

namespace exl3 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

// A waiting warp is suspended by the hardware for up to this many nanoseconds per poll instead of burning issue slots.
constexpr uint32_t MBAR_SUSPEND_NS = 20000;

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity), "r"(MBAR_SUSPEND_NS)
        : "memory");
    return ok != 0;
}

// Bounded wait: about a second of polling at most, then gives up.
constexpr uint32_t MBAR_MAX_POLLS = 1u << 16;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < MBAR_MAX_POLLS; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Bounded wait for a thread that is in no hurry (a copy producer far ahead of its consumers): sleeps between polls
// so that it does not take issue slots from the warps doing the work.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < MBAR_MAX_POLLS; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(256);
    }
    return false;
}

// ---- thread-block clusters: a barrier of the other CTA of a pair, and the cluster-wide barrier
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// All threads of every CTA of the cluster (convergent warps).
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta)
{
    asm volatile("{\n .reg .b32 ra;\n mapa.shared::cluster.u32 ra, %0, %1;\n mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n}" ::"r"(
                     smem_addr(bar)),
                 "r"(cta)
                 : "memory");
}

// Bounded wait on a barrier of this CTA that threads of the other CTA arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < MBAR_MAX_POLLS; i++) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(smem_addr(bar)), "r"(parity), "r"(MBAR_SUSPEND_NS)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// Shared-memory counter update with acquire-release semantics inside the CTA.
__device__ __forceinline__ int atom_add_acq_rel_cta_shared(int* addr, int v)
{
    int old;
    asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_addr(addr)), "r"(v) : "memory");
    return old;
}

// Single 64-bit accesses at system scope: the unit of the tagged-word exchange between GPUs (value + call number
// arrive together, so the receiver needs no fence and no separate flag).
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p)
{
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Two adjacent tagged words in one 16-byte access (each 8-byte half is what has to arrive whole): a warp then writes
// full 128-byte lines over NVLink instead of half-filled ones.
__device__ __forceinline__ void st_relaxed_sys_v2u64(unsigned long long* p, unsigned long long a, unsigned long long b)
{
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_relaxed_sys_v2u64(const unsigned long long* p, unsigned long long& a, unsigned long long& b)
{
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// global -> shared bulk copy through the TMA engine; completion is counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start before
// the kernel ahead of it in the stream has finished.  `grid_dependency_wait` blocks until that kernel has completed
// and its writes are visible; `grid_launch_dependents` lets the next kernel in the stream start its own prologue.
// 1-D bulk copy shared -> global (16-byte aligned on both sides, size a multiple of 16), tracked by the issuing thread's
// bulk groups: commit, then wait until the source may be overwritten (.read) or until the copies have completed.
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

}  // namespace ptx
}  // namespace exl3
