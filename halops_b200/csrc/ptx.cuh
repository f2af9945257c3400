// Inline-PTX wrappers for the sm_100a features the GEMM uses: mbarriers with
// bounded waits, TMA (tiled tensor copies and flat bulk copies), tensor memory
// management, the tcgen05 copy / MMA / load instructions and their fences.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hq {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier --------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the
// cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
    asm volatile(
        "{\n\t"
        ".reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t"
        "}" ::"r"(bar),
        "r"(cta)
        : "memory");
}

// Registers `bytes` expected bytes and one arrival on a barrier given by its
// shared::cluster address (it may belong to the other CTA of the pair).
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t bar_cluster, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                     bar_cluster),
                 "r"(bytes)
                 : "memory");
}
// One arrival on a barrier given by its shared::cluster address.
// try_wait that also acquires what another CTA of the cluster released before its
// (remote) arrive, e.g. stores into this CTA's shared memory.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// 16 bytes to an address of the cluster's shared-memory window (another CTA's shared memory).
__device__ __forceinline__ void st_cluster_v4(uint32_t addr_cluster, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr_cluster), "f"(a), "f"(b), "f"(c),
                 "f"(d)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster_addr(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster)
                 : "memory");
}

// Arrival that orders no memory accesses: for signals whose payload is in tensor memory
// (the reads or writes have completed, see tcgen05.wait) and not in shared or global memory.
// Measured on a 2-CTA cluster, back to back: 195 cycles per remote arrival against 517 for
// the releasing form.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster)
                 : "memory");
}

// ---- cluster -------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Full barrier over all threads of all CTAs of the cluster (every warp must call it converged).
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- proxies / fences --------------------------------------------------------

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- TMA ---------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 4 bytes global -> shared, asynchronous (non-bulk); completion is tracked per thread
// with cp_async_arrive_noinc.
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// Arrives on `bar` (as one of its expected arrivals) once every cp.async this thread
// has issued so far has landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// 2-D tile, global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Same, issued by either CTA of a pair: the data lands in this CTA's shared
// memory, the bytes are counted on the barrier at `bar` (an address that may
// name the other CTA of the pair).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y,
                                                 uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Flat copy of `bytes` (multiple of 16, both addresses 16-byte aligned).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// 2-D tile, shared -> global; rows / columns outside the tensor are dropped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
            reinterpret_cast<uint64_t>(m)),
        "r"(src), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tensor memory -------------------------------------------------------------

template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                     "r"(cols)
                     : "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                     "r"(cols)
                     : "memory");
    }
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                     : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                     : "memory");
    }
}

// 32 rows x 16 bytes of shared memory (one quarter of a 512-byte SfAtom row
// set) -> 4 tensor-memory columns, replicated into all four 32-lane quadrants.
template <int kCtaGroup>
__device__ __forceinline__ void tc_copy_sf(uint32_t taddr, uint64_t sdesc) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
                     : "memory");
    } else {
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
                     : "memory");
    }
}

// Block-scaled MMA, both operands from shared memory, accumulator and scale
// factors in tensor memory.  kKind: 0 = mxf8f6f4 (1 scale / 32), 1 = mxf4nvf4
// with 4 scales per K=64 (NVFP4), 2 = mxf4nvf4 with 2 scales per K=64 (MXFP4),
// 3 = mxf8f6f4 again (e4m3 x e2m1; the formats are in the instruction descriptor).
template <int kCtaGroup, int kKind>
__device__ __forceinline__ void tc_mma_block_scaled(uint32_t d, uint64_t adesc, uint64_t bdesc,
                                                    uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                    uint32_t accumulate) {
#define HQ_MMA_ASM(QUAL)                                                                   \
    asm volatile(                                                                          \
        "{\n\t"                                                                            \
        ".reg .pred p;\n\t"                                                                \
        "setp.ne.b32 p, %4, 0;\n\t"                                                        \
        "tcgen05.mma" QUAL " [%0], %1, %2, %3, [%5], [%6], p;\n\t"                         \
        "}" ::"r"(d),                                                                      \
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)            \
        : "memory")
    if constexpr (kCtaGroup == 1) {
        if constexpr (kKind == 0 || kKind == 3) {
            HQ_MMA_ASM(".cta_group::1.kind::mxf8f6f4.block_scale");
        } else if constexpr (kKind == 1) {
            HQ_MMA_ASM(".cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X");
        } else {
            HQ_MMA_ASM(".cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X");
        }
    } else {
        if constexpr (kKind == 0 || kKind == 3) {
            HQ_MMA_ASM(".cta_group::2.kind::mxf8f6f4.block_scale");
        } else if constexpr (kKind == 1) {
            HQ_MMA_ASM(".cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X");
        } else {
            HQ_MMA_ASM(".cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::2X");
        }
    }
#undef HQ_MMA_ASM
}

// Makes `bar` complete once every tcgen05 operation this thread issued so far
// has finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// Pair form: `bar` is a shared::cluster address, so it may name a barrier of
// either CTA of the pair (see mapa_cluster).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// shared::cluster address of this CTA's shared-memory address `addr` in CTA
// `cta` of the cluster.
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane
// (quadrant base + t), registers 0..31 the columns.
__device__ __forceinline__ void tc_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Registers -> tensor memory: thread i of the warp writes r[0..3] to columns
// [col, col + 4) of lane (taddr.lane + i).  A warp may only touch the 32 lanes
// of its own quarter (warp index % 4).
__device__ __forceinline__ void tc_store_32x32_x4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2,
                                                  uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r0),
                 "r"(r1), "r"(r2), "r"(r3)
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                             uint32_t& r3) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// ---- descriptors ------------------------------------------------------------------

// Shared-memory matrix descriptor: start address, leading / stride byte
// offsets (all in 16-byte units), descriptor version 1 (sm_100), swizzle mode
// in bits 61..63 (0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
    return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) |
           (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(layout) << 61);
}

}  // namespace ptx
}  // namespace hq
