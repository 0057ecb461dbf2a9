// Thin device-side wrappers over the sm_100a instructions the tensor-core
// kernels use: mbarrier (with bounded waits), TMA tile loads, tcgen05 TMEM
// allocation, UMMA issue/commit and TMEM loads, plus the shared-memory tile
// layout and the matrix / instruction descriptors that go with it.
//
// Shared-memory operand tiles use the 128-byte-swizzled canonical layout: a
// tile is a stack of "panels", each `rows` x 128 bytes, row pitch 128 B, with the
// 16-byte chunk index XORed with (row & 7).  A panel holds 32 fp32 (or 64
// 16-bit) elements of the contiguous dimension.  The same physical tile can be
// consumed K-major (rows = M/N index, contiguous = K) or MN-major (rows = K
// index, contiguous = M/N) by setting the major bit of the instruction
// descriptor and swapping the roles of the two strides in the matrix descriptor.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace rwkv7 {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- shared-memory tile layout ------------------------------------------------

// Byte offset of fp32 element (row, col) in a tile of `rows` rows; col < 32 * panels.
// The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t tile_off_f32(int rows, int row, int col) {
    const uint32_t off = (uint32_t)(col >> 5) * (uint32_t)rows * 128u + (uint32_t)row * 128u +
                         (uint32_t)(col & 31) * 4u;
    return off ^ (((uint32_t)row & 7u) << 4);
}

// ---- descriptors ----------------------------------------------------------------

// Matrix descriptor for a 128B-swizzled tile.  `lbo` / `sbo` in bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    d |= (uint64_t)2 << 61;  // 128-byte swizzle
    return d;
}

// K-major operand: rows = M (or N) index, 8-row groups 1024 B apart; one MMA
// K-step (32 bytes) advances the start address by 32 B inside a panel.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int rows, int kstep_f32) {
    const uint32_t panel = (uint32_t)(kstep_f32 >> 2), within = (uint32_t)(kstep_f32 & 3);
    return make_smem_desc(tile_addr + panel * (uint32_t)rows * 128u + within * 32u, 16u, 1024u);
}

// MN-major operand over the same physical tile: rows = K index; 32-element
// blocks of the M/N index are one panel (`rows` * 128 B) apart, 8-row K groups
// 1024 B apart; one K-step of 8 fp32 rows advances the start by 1024 B.
// `mn_block0` selects the first 32-element block (panel) of the M/N range.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int rows, int kstep_f32,
                                                 int mn_block0 = 0) {
    return make_smem_desc(tile_addr + (uint32_t)mn_block0 * (uint32_t)rows * 128u +
                              (uint32_t)kstep_f32 * 1024u,
                          (uint32_t)rows * 128u, 1024u);
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };

// Instruction descriptor: fp32 accumulate, dense, no negation.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, int M, int N, bool a_mn, bool b_mn) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- mbarrier -------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `max_polls` polls (each poll itself blocks for a
// hardware-defined short time) and returns false; callers then leave the kernel
// in an orderly way and report a timeout instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t max_polls = 2000000u) {
    for (uint32_t i = 0; i < max_polls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Same bound, but polling with the non-suspending test_wait: lower wake-up latency
// for short waits (an MMA group in flight) at the price of busy issue slots.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t *bar, uint32_t parity, uint32_t max_polls = 20000000u) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < max_polls; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// ---- thread-block clusters: distributed shared memory -------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void st_cluster_u4(uint32_t addr, uint4 v) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
// Asynchronous 16-byte store into another CTA's shared memory that reports its bytes to an
// mbarrier of that CTA when it lands: the sender neither waits nor fences.
__device__ __forceinline__ void st_async_cluster_u4(uint32_t addr, uint4 v, uint32_t remote_bar_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(remote_bar_addr)
                 : "memory");
}
// Bulk copy from this CTA's shared memory into another CTA's (addresses and size multiples of 16
// bytes); the bytes are reported to an mbarrier of the destination CTA as they land.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t remote_dst, const void *local_src, uint32_t bytes,
                                                 uint32_t remote_bar_addr) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(remote_dst), "r"(smem_u32(local_src)), "r"(bytes), "r"(remote_bar_addr)
                 : "memory");
}
// Arrive on an mbarrier of another CTA of the cluster; orders this thread's earlier (remote) writes before it.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr) : "memory");
}
// Bounded wait on a local mbarrier that CTAs of the cluster arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, uint32_t max_polls = 2000000u) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < max_polls; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA ------------------------------------------------------------------------

// 2-D tile load global -> shared, completion counted in bytes on `bar`.  No
// cluster multicast.  x is the innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// 2-D tile store shared -> global as part of the calling thread's current bulk group.  x (innermost,
// elements) times the element size must be a multiple of 16 bytes; coordinates must not be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *smem_src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of the calling thread's bulk groups are still reading their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until at most N of the calling thread's bulk groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05 --------------------------------------------------------------------

// Warp-wide.  Writes the TMEM base address to *smem_dst.  ncols: power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], issued by one thread.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is a TMEM region (128 lanes, 8 fp32
// columns per K-step), e.g. the accumulator of an earlier MMA of the same thread.
// MMAs issued by one thread execute in order, so no wait is needed in between.
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Makes `bar` complete (one arrival) when all MMAs issued so far by this thread are done.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// Each thread of a warp reads 32 consecutive columns of its own TMEM lane
// (lane = 32 * (warp % 4) + lane id; taddr carries that lane base in bits 31:16).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// Same with 16 consecutive columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// fp32 -> tf32 with round-to-nearest, ties away from zero (what cvt.rna.tf32.f32
// computes for finite values).  The tensor core ignores the low 13 mantissa bits,
// so adding half a tf32 ulp to the magnitude is all the rounding needs; as one
// integer add it runs at full rate, whereas the cvt instruction shares the
// quarter-rate transcendental pipe with exp and rcp.  Only finite operands reach it.
__device__ __forceinline__ float round_tf32(float x) {
    return __uint_as_float(__float_as_uint(x) + 0x1000u);
}

}  // namespace sm100
}  // namespace rwkv7
