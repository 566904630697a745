// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the contraction kernels use:
// mbarrier, TMA tiled loads (cp.async.bulk.tensor, one CTA per load), tcgen05 MMA with TMEM
// accumulators, tcgen05.ld/st, and the shared-memory / instruction descriptors of tcgen05.mma.
//
// Every wait is bounded: mbar_wait() gives up after kWaitLimitNs and reports false so the caller can
// raise a status word and leave the kernel in an orderly way instead of spinning forever.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace cgpt {
namespace sm100 {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ std::uint32_t smem_u32(const void* p) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(std::uint64_t* bar, std::uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(std::uint64_t* bar, std::uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(std::uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(std::uint64_t* bar, std::uint32_t parity) {
    std::uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity to complete. Returns false after kWaitLimitNs.
__device__ __forceinline__ bool mbar_wait(std::uint64_t* bar, std::uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = globaltimer_ns();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 1023u) == 0 && globaltimer_ns() - start > kWaitLimitNs) return false;
    }
    return true;
}

// ----------------------------------------------------------------------------------------------- TMA
// 2D tiled load global -> shared of this CTA; completion is signalled on `bar` as transaction bytes.
// x is the innermost coordinate (must make x * element size a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, std::uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, std::uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, std::uint64_t* bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// Untiled bulk copy global -> shared of this CTA: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, std::uint32_t bytes, std::uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<std::uint64_t>(tmap)) : "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (tcgen05.mma / TMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(std::uint32_t* smem_result, std::uint32_t columns) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(std::uint32_t taddr, std::uint32_t columns) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(std::uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16/bf16 inputs, fp32 accumulate. One thread issues.
__device__ __forceinline__ void mma_f16_ss(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                           std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M rows = lanes, K packed 16-bit pairs in columns) is read from TMEM.
__device__ __forceinline__ void mma_f16_ts(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint64_t b_desc,
                                           std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ------------------------------------------------------------------------ CTA pairs (cta_group::2)
// Two CTAs of a cluster of 2 (ranks 0 and 1, on the two SMs of one TPC) run ONE tcgen05.mma per K step: M = 256 rows
// (128 per CTA, each CTA's own A tile and TMEM accumulator), N up to 256 with each CTA holding HALF of the B tile in
// its own shared memory. The leader (rank 0) issues the MMA for both; barriers are addressed across the pair through
// shared::cluster addresses (mapa). Per FLOP each SM then reads and fills two thirds of the shared-memory bytes a
// single-CTA 128 x 256 tile needs. No load is multicast: every CTA issues the TMA loads of the bytes it keeps.
__device__ __forceinline__ std::uint32_t cluster_ctarank() {
    std::uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in the CTA of rank `rank`
__device__ __forceinline__ std::uint32_t mapa_shared(std::uint32_t local_addr, std::uint32_t rank) {
    std::uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Every thread of both CTAs. Not the .aligned form: the lanes of a warp reach it at different times (lane 0 of the
// producer and MMA warps runs a loop the other lanes skip).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(std::uint32_t cluster_addr) {   // arrive on a barrier of either CTA
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into THIS CTA's shared memory whose completion bytes are counted on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, std::uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(std::uint32_t* smem_result, std::uint32_t columns) {  // one warp of EACH CTA
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(std::uint32_t taddr, std::uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair; issued by one thread of the leader CTA.
__device__ __forceinline__ void mma_f16_ss_pair(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                                std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The barrier (of either CTA, shared::cluster address) gets one arrival once every pair MMA issued so far has completed.
__device__ __forceinline__ void tc_commit_pair(std::uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Shared-memory operand descriptor, 128-byte swizzle. The tile must start on a 1024-byte boundary
// (descriptors for later K steps may add to the start address inside the tile).
//   K-major  tile [rows][64 x 16-bit]: rows 128 B apart, 8-row groups `sbo` = 1024 B apart; lbo unused.
//   MN-major tile [k][64 x 16-bit]: k rows 128 B apart, 8-row k groups `sbo` = 1024 B apart, 64-element
//            blocks along M/N `lbo` bytes apart.
__device__ __forceinline__ std::uint64_t smem_desc_sw128(std::uint32_t saddr, std::uint32_t lbo_bytes, std::uint32_t sbo_bytes) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<std::uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<std::uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;  // descriptor version of sm_100
    d |= 2ull << 61;  // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulator, A/B both fp16 (fmt 0) or both bf16 (fmt 1).
// a_mn / b_mn = 1 when that operand's tile is MN-major ("transposed").
__host__ __device__ constexpr std::uint32_t idesc_f16(int fmt, int a_mn, int b_mn, int m, int n) {
    return (1u << 4) | (static_cast<std::uint32_t>(fmt) << 7) | (static_cast<std::uint32_t>(fmt) << 10) |
           (static_cast<std::uint32_t>(a_mn) << 15) | (static_cast<std::uint32_t>(b_mn) << 16) |
           (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives lane (lane field of taddr + i),
// columns [col, col+32). A warp may only touch the lane quarter 32*(warp_id % 4). The load and its
// tcgen05.wait::ld are one asm statement so the compiler cannot schedule a use of the registers
// between them.
__device__ __forceinline__ void tmem_ld_32x32(std::uint32_t taddr, std::uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// Two independent 32-column loads in flight, then one wait.
__device__ __forceinline__ void tmem_ld_32x32_x2(std::uint32_t taddr0, std::uint32_t (&a)[32], std::uint32_t taddr1,
                                                 std::uint32_t (&b)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
          "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]),
          "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]),
          "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
          "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]),
          "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]),
          "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]),
          "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
        : "r"(taddr0), "r"(taddr1)
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(std::uint32_t taddr, const std::uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr)
        : "memory");
}
// 32 lanes x 16 columns: thread i of the warp writes its 16 registers to lane (lane field + i), columns [col, col+16).
__device__ __forceinline__ void tmem_st_32x16(std::uint32_t taddr, const std::uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace sm100

// -------------------------------------------------------------------------------- host: tensor maps
// Encodes a 2D (or higher) row-major tensor map with 128-byte swizzle; out-of-bounds elements read
// as zero. dims/strides are innermost first; strides_bytes has rank-1 entries (the innermost stride is
// the element size). Returns a CGPT status.
int make_tensor_map(CUtensorMap* map, int dtype, const void* base, int rank, const std::uint64_t* dims,
                    const std::uint64_t* strides_bytes, const std::uint32_t* box);

}  // namespace cgpt
