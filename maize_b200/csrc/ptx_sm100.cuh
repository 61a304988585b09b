// Inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarrier,
// TMA tiled loads (every CTA issues its own), tcgen05 MMA / TMEM, cluster and grid-dependency control.
//
// These take the place of the instruction emitters the reference drives through
// LLVM: cp.async + commit/wait groups (crates/maize_core/src/intrinsics/cuda/cp_async.rs:54-65),
// ldmatrix (intrinsics/cuda/ldsm.rs:48-73), mma.sync (crates/maize_tile/src/mma/sm80.rs:136-160)
// and the special-register readers (intrinsics/cuda/sreg.rs:15-159).
#pragma once
#include <cuda.h>  // CUtensorMap (type only; no driver symbol is linked)
#include <cuda_bf16.h>
#include <cstdint>

namespace maize {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ long long sm_clock64()
{
    long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier --

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

// Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One probe of the phase with parity `parity`; may suspend for a hardware-defined
// short time, never blocks indefinitely.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Same with cluster-scope acquire: pairs with remote arrivals / remote TMA bytes.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
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

// --------------------------------------------------------------------- TMA --

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory; completion bytes go to `bar`.
// x is the innermost (contiguous) coordinate in elements and must keep x * 2 bytes
// a multiple of 16; callers only pass multiples of 64.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *map, uint32_t bar, int32_t x,
                                            int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Same with an L2 eviction-priority hint (createpolicy value).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap *map, uint32_t bar, int32_t x,
                                                 int32_t y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// CTA-pair form of the tiled load: the data lands in THIS CTA's shared memory, the
// completion bytes are signalled on `bar_cluster_addr`, a shared::cluster address
// that may name the barrier of either CTA of the pair (every CTA issues its own
// loads; none is shared between CTAs).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t smem_dst, const CUtensorMap *map,
                                                      uint32_t bar_cluster_addr, int32_t x, int32_t y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// 2-D tiled store shared memory -> global (the box of the tensor map, swizzled as the map says); elements outside
// the tensor are not written.  x * 2 bytes must be a multiple of 16 and no coordinate negative.  Completion is
// tracked by bulk groups of the issuing thread.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}

// Same with an L2 eviction-priority hint (createpolicy value) for the lines written.
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap *map, uint32_t smem_src, int32_t x, int32_t y,
                                                  uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smem_src), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Until at most N of this thread's bulk groups are still READING their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Until at most N of this thread's bulk groups are still pending at all (their writes are then performed).
template <int N>
__device__ __forceinline__ void bulk_wait_group()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders this thread's earlier generic-proxy writes to shared memory before later async-proxy (TMA) reads of it.
__device__ __forceinline__ void fence_proxy_async_shared()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Arrive (release, cluster scope) on a barrier named by a shared::cluster address.
__device__ __forceinline__ void mbar_arrive_cluster_addr(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t value)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(value) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t policy_evict_normal()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ----------------------------------------------------------------- tcgen05 --

__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Whole warp.  Writes the TMEM base address of `ncols` columns (power of two >= 32)
// to the shared word at `smem_slot`.
__device__ __forceinline__ void tmem_alloc_1cta(uint32_t smem_slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_1cta()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_1cta(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tmem_alloc_2cta(uint32_t smem_slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_2cta()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 operand tile whose rows are
// 64 elements = 128 bytes, written by TMA with the 128-byte swizzle:
//   bits  0-13  start address >> 4
//   bits 16-29  leading-dimension byte offset >> 4 (unused for swizzled K-major: 1)
//   bits 32-45  stride-dimension byte offset >> 4  (8 rows x 128 B = 1024 B)
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  layout type (2 = 128-byte swizzle)
// The tile base must be 1024-byte aligned; a K step of 16 elements inside the
// 64-wide swizzle atom advances the start address by 32 bytes (+2 in the field).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Shared-memory matrix descriptor for an MN-major bf16 operand (the matrix is stored with its M or N index
// contiguous, e.g. B given as K x N row-major).  The tile is a row of chunks; a chunk is 64 MN-elements
// (128 bytes) wide and holds the tile's K rows one after the other, as a TMA box {64 elements, K rows} with
// the 128-byte swizzle writes it:
//   leading-dimension byte offset  = distance between consecutive 64-element chunks along MN (`chunk_bytes`)
//   stride-dimension byte offset   = distance between consecutive groups of 8 K rows = 8 x 128 B = 1024 B
// A K step of 16 elements is two such groups: the start address advances by 2048 bytes.
__device__ __forceinline__ uint64_t make_smem_desc_sw128_mn(uint32_t smem_addr, uint32_t chunk_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((chunk_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), fp32 D:
//   bits 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format (1 = bf16),
//   bit 15/16 A/B major (0 = K), bits 17-22 N >> 3, bits 24-28 M >> 4.
__host__ __device__ constexpr uint32_t make_instr_desc_bf16(uint32_t mma_m, uint32_t mma_n, bool b_mn_major = false)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((mma_n >> 3) << 17) |
           ((mma_m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, one CTA.  Issued by ONE thread.
__device__ __forceinline__ void mma_bf16_1cta(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Same over a CTA pair (issued by one thread of the even CTA of the pair).
__device__ __forceinline__ void mma_bf16_2cta(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive once on `bar` when every tcgen05.mma this thread issued so far is done.
__device__ __forceinline__ void mma_commit_1cta(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// CTA-pair form: `bar` is a shared::cluster address (use mapa for the peer's barrier).
__device__ __forceinline__ void mma_commit_2cta(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar_cluster_addr)
                 : "memory");
}

// CTA-pair commit that arrives on the barrier at the same offset in every CTA named by
// `cta_mask` (bit i = CTA rank i of the cluster) with one instruction.  This is a barrier
// signal, not a data copy.
__device__ __forceinline__ void mma_commit_2cta_mask(uint32_t bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     bar),
                 "h"(cta_mask)
                 : "memory");
}

__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}

// Whole warp: lane i of warp w reads TMEM lane 32*(w%4)+i, 32 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two fp32 -> packed bf16x2, round-to-nearest-even; `lo` lands at the lower address.
__device__ __forceinline__ uint32_t pack_bf16x2(uint32_t lo_f32_bits, uint32_t hi_f32_bits)
{
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi_f32_bits)), "f"(__uint_as_float(lo_f32_bits)));
    return d;
}

// Programmatic dependent launch.  launch_dependents: this CTA no longer objects to the next kernel of the
// stream being scheduled (it starts on SMs as they free up).  wait: block until every kernel this one
// depends on has completed and its memory is visible; a no-op when the launch carried no such dependency.
__device__ __forceinline__ void grid_dependency_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

}  // namespace ptx
}  // namespace maize
