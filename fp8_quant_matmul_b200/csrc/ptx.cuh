// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA tiled loads (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld)
// and the fences between the generic, async and tensor-core proxies.
// Everything here is device-only and has no state.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace fp8bs {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier ----------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// try_wait with a suspend-time hint (nanoseconds): the hardware parks the thread until the phase completes or
// the time runs out, instead of returning at once; a parked poller issues no instructions, which leaves the
// issue slots of its scheduler to the warps that share it.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// ---------------------------------------------------------------- TMA ---------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}
// 2-D tiled load global -> shared of this CTA; completion is counted in bytes on `bar`.
// c0 is the innermost (contiguous) coordinate; c0 * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int c0, int c1,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// 2-D tiled store shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05 -----------
// Allocate `ncols` TMEM columns (power of two, 32..512); the base address is written to
// the shared-memory word at `slot`.  Whole warp, converged.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], fp8 (e4m3/e5m2) operands, one CTA.
__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive (count 1) on `bar` once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar)
                 : "memory");
}
// ---------------------------------------------------------------- clusters ----------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes from the shared memory of any CTA of the cluster (address from mapa).
__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t cluster_addr)
{
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}
// Arrive on an mbarrier that may live in another CTA of the cluster (shared::cluster address).
// Default semantics on purpose: a cluster-scope release costs several hundred cycles per arrive, and the
// TMEM hand-offs this is used for are ordered by tcgen05.fence::before_thread_sync / after_thread_sync.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load issued by either CTA of a pair; the byte count is reported to `bar`, which may be the
// peer CTA's barrier (shared::cluster address).  No multicast: the data lands in this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int c0, int c1,
                                                 uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
        : "memory");
}
// cta_group::2 forms: TMEM is allocated in both CTAs of the pair at the same column address; the MMA
// is issued by the leader CTA and reads A rows / B columns from both CTAs' shared memory.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Once the pair's MMAs issued so far are done, arrive on the barrier at this shared-memory offset in every CTA named in
// `cta_mask` (bit r = CTA rank r of the cluster): one instruction instead of one commit per CTA.  A commit, not a copy:
// no data is multicast.
__device__ __forceinline__ void mma_commit_pair_all(uint32_t bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}

// ---------------------------------------------------------------- dependent launch --
// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may start
// while the kernel before it in the stream is still finishing.  grid_dependency_wait() blocks until that earlier
// kernel has completed and its memory is visible; everything before it must not touch global memory.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets the next kernel in the stream (if it was launched as a programmatic dependent) begin its own prologue.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- registers ---------
template <int N>
__device__ __forceinline__ void setmaxnreg_inc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// ---------------------------------------------------------------- promotion ---------
// acc[0..15] += sc * cur[OFF .. OFF+31] (two columns per instruction), cur being a 64-column buffer.
template <int OFF>
__device__ __forceinline__ void fma32_from64(unsigned long long (&acc)[16], const uint32_t (&cur)[64], unsigned long long sc2)
{
    asm volatile(
        "{\n\t.reg .b64 t;\n\t"
        "mov.b64 t, {%16, %17};\n\tfma.rn.f32x2 %0, t, %48, %0;\n\t"
        "mov.b64 t, {%18, %19};\n\tfma.rn.f32x2 %1, t, %48, %1;\n\t"
        "mov.b64 t, {%20, %21};\n\tfma.rn.f32x2 %2, t, %48, %2;\n\t"
        "mov.b64 t, {%22, %23};\n\tfma.rn.f32x2 %3, t, %48, %3;\n\t"
        "mov.b64 t, {%24, %25};\n\tfma.rn.f32x2 %4, t, %48, %4;\n\t"
        "mov.b64 t, {%26, %27};\n\tfma.rn.f32x2 %5, t, %48, %5;\n\t"
        "mov.b64 t, {%28, %29};\n\tfma.rn.f32x2 %6, t, %48, %6;\n\t"
        "mov.b64 t, {%30, %31};\n\tfma.rn.f32x2 %7, t, %48, %7;\n\t"
        "mov.b64 t, {%32, %33};\n\tfma.rn.f32x2 %8, t, %48, %8;\n\t"
        "mov.b64 t, {%34, %35};\n\tfma.rn.f32x2 %9, t, %48, %9;\n\t"
        "mov.b64 t, {%36, %37};\n\tfma.rn.f32x2 %10, t, %48, %10;\n\t"
        "mov.b64 t, {%38, %39};\n\tfma.rn.f32x2 %11, t, %48, %11;\n\t"
        "mov.b64 t, {%40, %41};\n\tfma.rn.f32x2 %12, t, %48, %12;\n\t"
        "mov.b64 t, {%42, %43};\n\tfma.rn.f32x2 %13, t, %48, %13;\n\t"
        "mov.b64 t, {%44, %45};\n\tfma.rn.f32x2 %14, t, %48, %14;\n\t"
        "mov.b64 t, {%46, %47};\n\tfma.rn.f32x2 %15, t, %48, %15;\n\t"
        "}"
        : "+l"(acc[0]), "+l"(acc[1]), "+l"(acc[2]), "+l"(acc[3]), "+l"(acc[4]), "+l"(acc[5]), "+l"(acc[6]), "+l"(acc[7]), "+l"(acc[8]), "+l"(acc[9]), "+l"(acc[10]), "+l"(acc[11]), "+l"(acc[12]), "+l"(acc[13]), "+l"(acc[14]), "+l"(acc[15])
        : "r"(cur[OFF + 0]), "r"(cur[OFF + 1]), "r"(cur[OFF + 2]), "r"(cur[OFF + 3]), "r"(cur[OFF + 4]), "r"(cur[OFF + 5]), "r"(cur[OFF + 6]), "r"(cur[OFF + 7]), "r"(cur[OFF + 8]), "r"(cur[OFF + 9]), "r"(cur[OFF + 10]), "r"(cur[OFF + 11]), "r"(cur[OFF + 12]), "r"(cur[OFF + 13]), "r"(cur[OFF + 14]), "r"(cur[OFF + 15]), "r"(cur[OFF + 16]), "r"(cur[OFF + 17]), "r"(cur[OFF + 18]), "r"(cur[OFF + 19]), "r"(cur[OFF + 20]), "r"(cur[OFF + 21]), "r"(cur[OFF + 22]), "r"(cur[OFF + 23]), "r"(cur[OFF + 24]), "r"(cur[OFF + 25]), "r"(cur[OFF + 26]), "r"(cur[OFF + 27]), "r"(cur[OFF + 28]), "r"(cur[OFF + 29]), "r"(cur[OFF + 30]), "r"(cur[OFF + 31]), "l"(sc2));
}

// 64 columns from TMEM, complete on return (load and wait in one statement).
__device__ __forceinline__ void tmem_ld_x64_sync(uint32_t taddr, uint32_t (&v)[64])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr)
        : "memory");
}

// Two 64-column loads from different TMEM addresses in flight together, both complete on return.
__device__ __forceinline__ void tmem_ld_2x64_sync(uint32_t taddr_a, uint32_t taddr_b, uint32_t (&a)[64], uint32_t (&b)[64])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%128];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95, %96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%129];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]), "=r"(a[32]), "=r"(a[33]), "=r"(a[34]), "=r"(a[35]), "=r"(a[36]), "=r"(a[37]), "=r"(a[38]), "=r"(a[39]), "=r"(a[40]), "=r"(a[41]), "=r"(a[42]), "=r"(a[43]), "=r"(a[44]), "=r"(a[45]), "=r"(a[46]), "=r"(a[47]), "=r"(a[48]), "=r"(a[49]), "=r"(a[50]), "=r"(a[51]), "=r"(a[52]), "=r"(a[53]), "=r"(a[54]), "=r"(a[55]), "=r"(a[56]), "=r"(a[57]), "=r"(a[58]), "=r"(a[59]), "=r"(a[60]), "=r"(a[61]), "=r"(a[62]), "=r"(a[63]), "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31]), "=r"(b[32]), "=r"(b[33]), "=r"(b[34]), "=r"(b[35]), "=r"(b[36]), "=r"(b[37]), "=r"(b[38]), "=r"(b[39]), "=r"(b[40]), "=r"(b[41]), "=r"(b[42]), "=r"(b[43]), "=r"(b[44]), "=r"(b[45]), "=r"(b[46]), "=r"(b[47]), "=r"(b[48]), "=r"(b[49]), "=r"(b[50]), "=r"(b[51]), "=r"(b[52]), "=r"(b[53]), "=r"(b[54]), "=r"(b[55]), "=r"(b[56]), "=r"(b[57]), "=r"(b[58]), "=r"(b[59]), "=r"(b[60]), "=r"(b[61]), "=r"(b[62]), "=r"(b[63])
        : "r"(taddr_a), "r"(taddr_b)
        : "memory");
}

// ---------------------------------------------------------------- descriptors -------
// Shared-memory matrix descriptor for an MN-major 8-bit operand held as rows of 128 bytes
// (128 consecutive m or n) per k, 128-byte swizzled -- exactly what a TMA box
// {128 bytes, rows} with CU_TENSOR_MAP_SWIZZLE_128B writes.  One swizzle atom is
// 8 k-rows x 128 B = 1024 B; `sbo` is the byte distance between consecutive 8-row groups
// along K, `lbo` the byte distance between consecutive 128-wide slabs along M/N.
//   bits [0,14)  start address >> 4      bits [16,30) lbo >> 4     bits [32,46) sbo >> 4
//   bits [46,48) descriptor version (1 on sm_100)      bits [61,64) swizzle (2 = 128 B)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo,
                                                         uint32_t sbo)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor for kind::f8f6f4: e4m3 x e4m3 -> fp32, both operands MN-major.
//   [4,6) D format (1 = f32)  [7,10) A format (0 = e4m3)  [10,13) B format (0 = e4m3)
//   [15] A is MN-major  [16] B is MN-major  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_e4m3_mnmajor(int m, int n)
{
    return (1u << 4) | (0u << 7) | (0u << 10) | (1u << 15) | (1u << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace ptx
}  // namespace fp8bs
