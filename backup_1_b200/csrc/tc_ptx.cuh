/* Inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path: mbarriers, TMA
 * (cp.async.bulk.tensor), tensor memory (tcgen05.alloc/ld), tcgen05.mma and its descriptors.
 * Shared by the GEMM kernel and the tensor-peak probe. */
#ifndef DECXB_TC_PTX_CUH_
#define DECXB_TC_PTX_CUH_

#include <cuda.h>
#include <stdint.h>

namespace tcptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}

__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank)
{
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

/* Arrive on a barrier given by a shared::cluster address (own CTA or the peer). */
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}

/* Plain 2-D tiled TMA load into this CTA's shared memory, completion on this CTA's barrier. */
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

/* Same load inside a CTA pair: data lands in the issuing CTA's shared memory, the
 * transaction bytes are counted on the barrier at `bar_cluster_addr` (the leader CTA's). */
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}

/* 4-D tiled loads (channel, x, y, image) for the implicit-GEMM convolution: the box is
 * 32 channels x BX pixels x BY rows of one image, out-of-range pixels read as zero. */
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int x, int y, int n)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar), "r"(c), "r"(x), "r"(y), "r"(n) : "memory");
}

__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c, int x, int y, int n)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c), "r"(x), "r"(y), "r"(n) : "memory");
}

/* Tiled TMA store of a 32 x 32 fp32 box from this CTA's shared memory (bulk async-group). */
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
/* The same box as a slice of a 4-D tensor (channel, x, y, image): 32 channels of bx_s x by_s pixels. */
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c, int x, int y, int n)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :: "l"(map), "r"(src), "r"(c), "r"(x), "r"(y), "r"(n) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
/* every bulk store of this thread has finished READING shared memory (the staging buffer may be rewritten) */
template <int PENDING>
__device__ __forceinline__ void tma_store_wait_read()
{
    if (PENDING == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    else              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
/* every bulk store of this thread is complete */
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
/* generic-proxy writes to shared memory become visible to the async proxy (TMA) */
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

/* Brings a tensor map into the copy engine's descriptor cache ahead of its first use. */
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
    if (CTAS == 1) asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_dst), "r"(ncols) : "memory");
    else           asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_dst), "r"(ncols) : "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_relinquish()
{
    if (CTAS == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else           asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
    else           asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}

/* D(tmem) (+)= A(smem desc) * B(smem desc), issued by one thread.
 * COLL names what happens to the tensor core's collector buffer for the A operand:
 * 0 = default (A is read from shared memory, the buffer is not kept), 1 = fill (A is read from
 * shared memory and kept in the buffer), 2 = lastuse (A is taken from the buffer, which must
 * have been filled by the preceding MMA with the same A tile, and released). */
#define DECXB_UMMA_TF32_ASM(GROUP, COLLQ)                                                          \
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                  \
                 "tcgen05.mma.cta_group::" GROUP ".kind::tf32" COLLQ " [%0], %1, %2, %3, p;\n\t}"    \
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory")
template <int CTAS, int COLL = 0>
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    if (CTAS == 1) {
        if (COLL == 1)      DECXB_UMMA_TF32_ASM("1", ".collector::a::fill");
        else if (COLL == 2) DECXB_UMMA_TF32_ASM("1", ".collector::a::lastuse");
        else                DECXB_UMMA_TF32_ASM("1", "");
    } else {
        if (COLL == 1)      DECXB_UMMA_TF32_ASM("2", ".collector::a::fill");
        else if (COLL == 2) DECXB_UMMA_TF32_ASM("2", ".collector::a::lastuse");
        else                DECXB_UMMA_TF32_ASM("2", "");
    }
}

template <int CTAS>
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    if (CTAS == 1) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}

/* Make the barrier observe completion of every tcgen05.mma this thread issued so far.
 * In a CTA pair the arrival is delivered to the same barrier offset in both CTAs. */
template <int CTAS>
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    if (CTAS == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
    } else {
        const uint16_t mask = 3;
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     :: "r"(bar), "h"(mask) : "memory");
    }
}

/* 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread. */
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v)
{
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

/* Shared-memory matrix descriptor for a K-contiguous tile whose rows are 128 bytes,
 * written by TMA with the 128-byte swizzle: 8-row groups lie 1024 bytes apart (stride
 * byte offset), the leading byte offset is unused for swizzled K-major layouts (set to 1),
 * descriptor version 1 (Blackwell), layout type 2 (128-byte swizzle). */
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

/* The same for a K-contiguous tile whose rows are 64 bytes (32 bf16 values), written by TMA with the
 * 64-byte swizzle: 8-row groups lie 512 bytes apart, layout type 4 (64-byte swizzle). */
__device__ __forceinline__ uint64_t make_smem_desc_sw64(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;
    return d;
}

/* Instruction descriptor: D fp32 (bits 4-5 = 1), A and B TF32 (bits 7-9, 10-12 = 2), both
 * K-major (bits 15, 16 = 0), N>>3 at bits 17-22, M>>4 at bits 24-28. */
/* Same with fp16 operands (format code 0 at bits 7-9 and 10-12), fp32 accumulator. */
__host__ __device__ constexpr uint32_t make_idesc_f16(int umma_m, int umma_n)
{
    return (1u << 4) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}

/* bf16 operands (format code 1), fp32 accumulator; issued with kind::f16 like fp16. */
__host__ __device__ constexpr uint32_t make_idesc_bf16(int umma_m, int umma_n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t make_idesc(int umma_m, int umma_n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}

}  // namespace tcptx

#endif
