// Replication of A for the N-sharded multi-GPU GEMM without spending SMs on the receivers:
// the root pushes each row slab ONCE through its NVSwitch multicast address (multimem.st), the
// switch writes it into every GPU's landing buffer, and a flag word published the same way tells
// the receivers how many slabs have landed.  Receivers only run one-warp kernels that watch the flag
// (bounded, like every wait in this library) ahead of each GEMM launch.
//
// The push kernel is thin (no shared memory, few registers) so that its CTAs share SMs with the
// resident CTAs of the persistent GEMM instead of queueing behind them, which is what a
// library broadcast with its wide CTAs ends up doing.
//
// The reference has no multi-GPU code; this serves the N-sharding that lifts its column-panel
// split (crates/maize_tile/src/gmem/col_panel.rs:88-124) across GPUs.
#pragma once
#include "gemm_common.cuh"

namespace maize {

__device__ __forceinline__ void multimem_st_v4(void *mc_addr, const uint4 &v)
{
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

__device__ __forceinline__ void multimem_st_release_u32(void *mc_addr, uint32_t v)
{
    asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

// Streaming 16-byte loads for the copy kernels: the bytes pass through once, so they must not
// displace the GEMM's operand tiles from L1 / L2 (`policy` = an evict-first createpolicy value).
__device__ __forceinline__ uint4 ld_stream_nc(const uint4 *p, uint64_t policy)  // read-only data (the caller's A)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}

__device__ __forceinline__ uint4 ld_stream(const uint4 *p, uint64_t policy)  // data another GPU may have just written
{
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys_u32(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait of one thread until *flag has reached `value` (values only grow; wrap-around safe).
__device__ __forceinline__ bool flag_wait_bounded(const uint32_t *flag, uint32_t value, DeviceStatus *status,
                                                  uint64_t budget_ns, int role)
{
    const uint64_t t0 = ptx::global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        if (static_cast<int32_t>(ld_acquire_sys_u32(flag) - value) >= 0)
            return true;
        if ((it & 63u) == 63u && ptx::global_timer_ns() - t0 > budget_ns) {
            if (atomicMax(&status->code, kStatusTimeout) < kStatusTimeout) {
                status->role = role;
                status->cta = static_cast<int>(blockIdx.x);
            }
            return false;
        }
        __nanosleep(100);
    }
}

// Copies n16 16-byte units from local `src` to every replica behind `mc_dst`; the last CTA to
// finish publishes `flag_value` at `mc_flag` on every GPU.  `done_counter` is zero between launches.
// If `wait_flag` is not null the copy first waits (bounded) for *wait_flag >= wait_value: the source
// is then itself a landing area that another GPU is still filling.  A CTA whose wait expires skips its
// part of the copy, and the flag is then not published, so that nobody consumes bytes that never arrived;
// the status word reports it.  The grid has at most 65535 CTAs (the host caps it far below).
__global__ void __launch_bounds__(512) mc_push_kernel(const uint4 *src, uint4 *mc_dst, uint64_t n16,
                                                      unsigned int *done_counter, uint32_t *mc_flag,
                                                      uint32_t flag_value, const uint32_t *wait_flag,
                                                      uint32_t wait_value, DeviceStatus *status, uint64_t budget_ns)
{
    __shared__ int landed;
    if (threadIdx.x == 0)
        landed = (wait_flag == nullptr || flag_wait_bounded(wait_flag, wait_value, status, budget_ns, 7)) ? 1 : 0;
    __syncthreads();
    if (landed) {
        const uint64_t pol = ptx::policy_evict_first();
        const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
        uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
        for (; i + 3 * stride < n16; i += 4 * stride) {
            // plain (coherent) loads: the source may have been written by another GPU moments ago
            const uint4 v0 = ld_stream(src + i, pol), v1 = ld_stream(src + i + stride, pol),
                        v2 = ld_stream(src + i + 2 * stride, pol), v3 = ld_stream(src + i + 3 * stride, pol);
            multimem_st_v4(mc_dst + i, v0);
            multimem_st_v4(mc_dst + i + stride, v1);
            multimem_st_v4(mc_dst + i + 2 * stride, v2);
            multimem_st_v4(mc_dst + i + 3 * stride, v3);
        }
        for (; i < n16; i += stride)
            multimem_st_v4(mc_dst + i, ld_stream(src + i, pol));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // Every CTA arrives, also one whose wait ran out (it marks the upper half of the counter), so that the
        // counter is back at zero for the next launch whatever happened; the flag is published only if all copied.
        __threadfence_system();
        const unsigned int arrived = atomicAdd(done_counter, landed ? 1u : 0x10001u);
        if ((arrived & 0xffffu) == gridDim.x - 1) {
            *done_counter = 0u;
            __threadfence_system();
            if (landed && (arrived >> 16) == 0u)
                multimem_st_release_u32(mc_flag, flag_value);
        }
    }
}

// Root side of the two-stage replication: chunk p of the source (an equal share in 16-byte units)
// goes to GPU p's landing buffer with ordinary stores through its peer mapping; when the last CTA
// working for GPU p is done it publishes `flag_value` in that GPU's "my chunk has landed" word.
// The root's own chunk is skipped (the root multicasts it straight from the source).
constexpr uint32_t kMaxPeers = 16;
struct ScatterTargets {
    uint4 *dst[kMaxPeers];      // landing buffer of each rank at the slab's offset (peer-mapped)
    uint32_t *flag[kMaxPeers];  // "chunk landed" word of each rank (peer-mapped)
};

__global__ void __launch_bounds__(512) scatter_push_kernel(const uint4 *__restrict__ src, ScatterTargets targets,
                                                           uint64_t n16, uint32_t world, uint32_t root,
                                                           uint32_t flag_value, unsigned int *done_counters)
{
    const uint32_t peers = world - 1;
    const uint32_t g = blockIdx.x % peers;          // which peer this CTA serves
    const uint32_t p = g < root ? g : g + 1;        // its rank
    const uint32_t ctas_for_p = gridDim.x / peers + (g < gridDim.x % peers ? 1u : 0u);
    const uint32_t my_index = blockIdx.x / peers;   // index among the CTAs serving p
    const uint64_t lo = n16 * p / world, hi = n16 * (p + 1) / world;
    uint4 *dst = targets.dst[p];
    const uint64_t pol = ptx::policy_evict_first();
    const uint64_t stride = static_cast<uint64_t>(ctas_for_p) * blockDim.x;
    uint64_t i = lo + static_cast<uint64_t>(my_index) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < hi; i += 4 * stride) {
        const uint4 v0 = ld_stream_nc(src + i, pol), v1 = ld_stream_nc(src + i + stride, pol),
                    v2 = ld_stream_nc(src + i + 2 * stride, pol), v3 = ld_stream_nc(src + i + 3 * stride, pol);
        dst[i] = v0;
        dst[i + stride] = v1;
        dst[i + 2 * stride] = v2;
        dst[i + 3 * stride] = v3;
    }
    for (; i < hi; i += stride)
        dst[i] = ld_stream_nc(src + i, pol);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int arrived = atomicAdd(done_counters + p, 1u);
        if (arrived == ctas_for_p - 1) {
            done_counters[p] = 0u;
            __threadfence_system();
            st_release_sys_u32(targets.flag[p], flag_value);
        }
    }
}

// Waits (bounded) until every one of `count` flag words has reached `value`; lane i watches flag i.
// Values only grow; the comparison is wrap-around safe.
__global__ void flags_wait_kernel(const uint32_t *flags, uint32_t count, uint32_t value, DeviceStatus *status,
                                  uint64_t budget_ns)
{
    if (threadIdx.x >= count)
        return;
    const uint32_t *flag = flags + threadIdx.x;
    const uint64_t t0 = ptx::global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        if (static_cast<int32_t>(ld_acquire_sys_u32(flag) - value) >= 0)
            return;
        if ((it & 63u) == 63u && ptx::global_timer_ns() - t0 > budget_ns) {
            if (atomicMax(&status->code, kStatusTimeout) < kStatusTimeout) {
                status->role = 8;
                status->cta = static_cast<int>(threadIdx.x);
            }
            return;
        }
        __nanosleep(100);
    }
}

// Publishes `value` in a flag word (possibly in a peer GPU's memory) after everything this stream did before.
__global__ void flag_store_kernel(uint32_t *flag, uint32_t value)
{
    if (threadIdx.x == 0) {
        __threadfence_system();
        st_release_sys_u32(flag, value);
    }
}

// One step of a rank's forwarding in the chain, as ONE launch between two copies: publish `store_value` in
// `store_flag` (the next rank's count of landed chunks; everything this stream did before, i.e. the copy of that
// chunk, is visible first), then wait (bounded) until this rank's own count `wait_flag` has reached `wait_value`
// (the next chunk to forward has landed here).  Either half is skipped when its pointer is null.
__global__ void chain_step_kernel(uint32_t *store_flag, uint32_t store_value, const uint32_t *wait_flag,
                                  uint32_t wait_value, DeviceStatus *status, uint64_t budget_ns)
{
    if (threadIdx.x != 0)
        return;
    if (store_flag) {
        __threadfence_system();
        st_release_sys_u32(store_flag, store_value);
    }
    if (wait_flag)
        (void)flag_wait_bounded(wait_flag, wait_value, status, budget_ns, 8);
}

}  // namespace maize
