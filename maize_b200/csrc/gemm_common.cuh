// Pieces shared by the sm_100a GEMM kernels: the device status word, bounded
// mbarrier waits, the tile order, kernel parameters and the bf16 epilogue.
#pragma once
#include "ptx_sm100.cuh"

namespace maize {

constexpr int kStatusOk = 0;
constexpr int kStatusTimeout = 4;      // == MAIZE_ERR_TIMEOUT
constexpr int kStatusDeviceAbort = 5;  // == MAIZE_ERR_DEVICE_ABORT

// Device status block: worst status code, role that gave up, its CTA, spare.
struct DeviceStatus {
    int code;
    int role;
    int cta;
    int detail;
};

constexpr uint32_t kBlockM = 128;  // rows of C per CTA = TMEM lanes
constexpr uint32_t kBlockK = 64;   // bf16 elements per k-block = one 128-byte swizzle row
constexpr uint32_t kUmmaK = 16;    // K per tcgen05.mma for 16-bit operands
constexpr uint32_t kNumThreads = 192;
constexpr uint32_t kNumEpilogueThreads = 128;
constexpr uint32_t kNumEpilogueWarps = 4;

// Per-warp staging for the ragged epilogue: 32 rows of 32 bf16 (64 B) padded to
// 80 B so that the 16-byte row writes of a quarter warp hit distinct banks.
constexpr uint32_t kStageRowBytes = 80;
constexpr uint32_t kStageWarpBytes = 32 * kStageRowBytes;
constexpr uint32_t kStageBytesTotal = kNumEpilogueWarps * kStageWarpBytes;
// Per-warp staging of the TMA-store epilogue: two buffers of 32 rows x 64 bf16 (128 B, 128-byte swizzle) = 2 x 4 KiB.
// The ragged epilogue's staging above is carved out of the same area.
constexpr uint32_t kTmaStoreBufBytes = 32 * 128;
constexpr uint32_t kTmaStageWarpBytes = 2 * kTmaStoreBufBytes;
constexpr uint32_t kTmaStageBytesTotal = kNumEpilogueWarps * kTmaStageWarpBytes;

struct WaitCtl {
    volatile int *abort_flag;  // shared memory, CTA-wide
    DeviceStatus *status;      // global memory
    uint64_t budget_ns;
};

__device__ __forceinline__ void record_timeout(const WaitCtl &ctl, int role)
{
    *ctl.abort_flag = 1;
    if (atomicMax(&ctl.status->code, kStatusTimeout) < kStatusTimeout) {
        ctl.status->role = role;
        ctl.status->cta = static_cast<int>(blockIdx.x);
    }
}

// Bounded wait on an mbarrier phase.  Returns false if the budget ran out or
// another role of this CTA already gave up.  CLUSTER = acquire at cluster scope
// (the barrier is completed by arrivals or copies of the peer CTA).
template <bool CLUSTER = false>
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtl &ctl, int role)
{
    auto probe = [&]() { return CLUSTER ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity); };
    if (probe())
        return true;
    const uint64_t t0 = ptx::global_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (probe())
            return true;
        if ((it & 31u) == 0u) {
            if (*ctl.abort_flag)
                return false;
            if (ptx::global_timer_ns() - t0 > ctl.budget_ns) {
                record_timeout(ctl, role);
                return false;
            }
        }
    }
}

struct GemmParams {
    __nv_bfloat16 *c;
    uint64_t ldc;  // elements
    uint32_t m, n, k;
    uint32_t tiles_m, tiles_n;  // in units of the kernel's tile (per CTA pair for the 2-CTA kernel)
    uint32_t group_m;
    uint32_t pdl = 0;         // 1: launched with programmatic stream serialization (see the kernels' set-up)
    uint32_t serpentine = 0;  // 1: odd groups of row-blocks sweep the column-blocks backwards
    uint32_t c_vec_ok;  // 1: every C row starts 16-byte aligned (ldc % 8 == 0 and base aligned)
    uint32_t c_evict_first = 0;  // 1: TMA stores of C carry an evict-first L2 hint
    uint32_t c_tma_ok = 0;  // 1: the kernel's C tensor map is valid: full tiles leave through shared memory and TMA stores
    DeviceStatus *status;
    uint64_t timeout_ns;
    // Optional per-CTA cycle accounting (null in normal use): kProfileSlots counters per CTA.
    unsigned long long *profile;
    // Diagnostic switches for performance analysis (0 in normal use; results are wrong when set):
    //   bit 0: every load fetches tile (0, 0), so all operand traffic hits in L2;
    //   bit 1: no loads at all, the producer only signals "full" (upper bound of the MMA issue path).
    uint32_t debug_flags;
    // Optional gate on the rows of A (null in normal use).  A may still be arriving, in order of its rows, while
    // the kernel runs: whoever delivers it counts chunks of `gate_rows` rows in the 32-bit word `*gate`, and rows
    // [0, r) may be read once the word has reached gate_base + ceil(r / gate_rows).  The producer of a CTA waits
    // (bounded) for the rows of its tile before the tile's first load; the word may live in this GPU's memory,
    // a peer's or in mapped host memory.
    const uint32_t *gate = nullptr;
    uint32_t gate_base = 0;
    uint32_t gate_rows = 1;
};

// Tile order: groups of `group_m` row-blocks sweep all column-blocks, so that the
// CTAs running at one time share A row panels and B column panels in L2.  With
// `serpentine` odd groups sweep the column-blocks in descending order, so that a group
// starts on the column panels of B that the previous group left in L2.  This
// is the grid-stride over (row panel, column panel) pairs of the reference
// (src/main.rs:56-73, crates/maize_tile/src/gmem/row_panel.rs:95-109) with an
// L2-aware order.
struct TileCoord {
    uint32_t m_blk, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(uint32_t t, const GemmParams &p)
{
    const uint32_t per_group = p.group_m * p.tiles_n;
    const uint32_t g = t / per_group;
    const uint32_t first_m = g * p.group_m;
    const uint32_t rows = min(p.tiles_m - first_m, p.group_m);
    const uint32_t r = t - g * per_group;
    TileCoord c;
    c.m_blk = first_m + r % rows;
    c.n_blk = r / rows;
    if (p.serpentine && (g & 1u))
        c.n_blk = p.tiles_n - 1u - c.n_blk;
    return c;
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Producer-side wait for rows [0, row_end) of a gated A.  `seen` caches the chunk count read last, so that a
// tile whose rows are known to have landed costs no load.  Role 5 in the status word = this wait gave up.
__device__ __forceinline__ bool gate_rows_landed(const GemmParams &p, uint32_t row_end, int32_t &seen, const WaitCtl &ctl)
{
    if (p.gate == nullptr)
        return true;
    const int32_t need = static_cast<int32_t>((min(row_end, p.m) + p.gate_rows - 1) / p.gate_rows);
    if (seen >= need)
        return true;
    const uint64_t t0 = ptx::global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        seen = static_cast<int32_t>(ld_acquire_sys_u32(p.gate) - p.gate_base);  // wrap-around safe
        if (seen >= need)
            break;
        if ((it & 15u) == 15u) {
            if (*ctl.abort_flag)
                return false;
            if (ptx::global_timer_ns() - t0 > ctl.budget_ns) {
                record_timeout(ctl, 5);
                return false;
            }
        }
        __nanosleep(200);
    }
    // the tile loads that follow go through the async proxy: order them after the acquire above
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return true;
}

// Slots of the per-CTA profile: cycles a role spent blocked in its waits, and the CTA's lifetime.
enum ProfileSlot {
    kProfProducerWaitEmpty = 0,
    kProfMmaWaitFull = 1,
    kProfMmaWaitAccEmpty = 2,
    kProfEpilogueWaitAccFull = 3,
    kProfEpilogueDrain = 4,
    kProfCtaCycles = 5,
    kProfTiles = 6,
    kProfileSlots = 8
};

// Adds the cycles of one wait to a role-local counter when profiling is on.
struct WaitTimer {
    bool on;
    long long t0;
    __device__ __forceinline__ explicit WaitTimer(bool enabled) : on(enabled), t0(enabled ? ptx::sm_clock64() : 0) {}
    __device__ __forceinline__ void stop(unsigned long long &acc)
    {
        if (on)
            acc += static_cast<unsigned long long>(ptx::sm_clock64() - t0);
    }
};

// Store one 32-row x 32-column chunk of C held by a warp as 32 fp32 accumulators
// per lane (lane = row).  `row0` is the first of the warp's 32 rows, `col0` the
// first column; both are warp-uniform, so every branch below is too.
//   aligned + full chunk : four 16-byte stores per lane straight from registers
//   otherwise            : transpose through the warp's staging buffer and write
//                          each row as one run of consecutive 2-byte elements
//                          (coalesced, any alignment), masked at the M and N edges.
__device__ __forceinline__ void store_chunk(const GemmParams &p, uint8_t *stage_warp, uint32_t row0, uint32_t col0,
                                            uint32_t lane, const uint32_t (&acc)[32])
{
    if (row0 >= p.m || col0 >= p.n)
        return;
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        packed[i] = ptx::pack_bf16x2(acc[2 * i], acc[2 * i + 1]);

    if (p.c_vec_ok && col0 + 32 <= p.n) {
        const uint32_t row = row0 + lane;
        if (row < p.m) {
            uint4 *dst = reinterpret_cast<uint4 *>(p.c + static_cast<uint64_t>(row) * p.ldc + col0);
#pragma unroll
            for (int v = 0; v < 4; ++v)
                dst[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
        }
        return;
    }

    uint4 *mine = reinterpret_cast<uint4 *>(stage_warp + lane * kStageRowBytes);
#pragma unroll
    for (int v = 0; v < 4; ++v)
        mine[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
    __syncwarp();
    const uint32_t rows = min(32u, p.m - row0);
    const bool col_ok = col0 + lane < p.n;
    __nv_bfloat16 *dst = p.c + static_cast<uint64_t>(row0) * p.ldc + col0 + lane;
    const uint8_t *src = stage_warp + lane * 2;
#pragma unroll 8
    for (uint32_t r = 0; r < rows; ++r) {
        const __nv_bfloat16 v = *reinterpret_cast<const __nv_bfloat16 *>(src + r * kStageRowBytes);
        if (col_ok)
            dst[static_cast<uint64_t>(r) * p.ldc] = v;
    }
    __syncwarp();
}

// Drain one 128-row x BN-column fp32 accumulator from TMEM to C.  Executed by the
// four epilogue warps; `quarter` = warp index % 4 selects the 32 TMEM lanes the
// warp may read; `tile_row0` / `tile_col0` locate the CTA's 128 x BN block in C.
template <uint32_t BN>
__device__ __forceinline__ void drain_accumulator(const GemmParams &p, uint8_t *stage_warp, uint32_t tmem_acc,
                                                  uint32_t quarter, uint32_t lane, uint32_t tile_row0,
                                                  uint32_t tile_col0)
{
    const uint32_t taddr = tmem_acc + ((quarter * 32u) << 16);
    const uint32_t row0 = tile_row0 + quarter * 32u;
#pragma unroll 1
    for (uint32_t c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
        ptx::tmem_ld_wait();
        store_chunk(p, stage_warp, row0, tile_col0 + c * 32u, lane, v);
    }
}

// Copies up to two row-major matrices of `rows` x (16 * cols16) bytes to another row pitch, 16 bytes per thread and
// step, in one launch (segment 0 takes the first `rows0` values of the row index, segment 1 the rest).
// Used ahead of the GEMM for operands whose pitch is not a multiple of 128 bytes: every 128-byte row of a TMA
// box then straddles two lines, which was measured to cost a third of the GEMM's rate (4111 x 3967 x 4104: 0.164 ms
// with pitch 8208 B, 0.108 ms with 8320 B); a pre-pass costs two passes over the operand at the HBM rate.
struct RepackSegment {
    const uint4 *src;
    uint4 *dst;
    uint64_t src_pitch16, dst_pitch16;  // row pitches in 16-byte units
    uint32_t rows;
};

__global__ void __launch_bounds__(256) repack_rows_kernel(RepackSegment s0, RepackSegment s1, uint32_t cols16)
{
    // a GEMM launched behind this copy with programmatic stream serialization may do its set-up meanwhile (it
    // waits for this grid to complete before it loads anything)
    ptx::grid_dependency_launch_dependents();
    // The 16-byte pieces of both segments form one index space that the grid strides over, four loads in flight
    // per thread: a few CTAs per SM with work for all their lanes, instead of a CTA per 4 KiB of a row.
    const uint64_t total = static_cast<uint64_t>(s0.rows + s1.rows) * cols16;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    auto locate = [&](uint64_t idx, const uint4 *&src, uint4 *&dst) {
        const uint32_t r = static_cast<uint32_t>(idx / cols16);
        const uint32_t c = static_cast<uint32_t>(idx - static_cast<uint64_t>(r) * cols16);
        const bool first = r < s0.rows;
        const RepackSegment &g = first ? s0 : s1;
        const uint32_t row = first ? r : r - s0.rows;
        src = g.src + static_cast<uint64_t>(row) * g.src_pitch16 + c;
        dst = g.dst + static_cast<uint64_t>(row) * g.dst_pitch16 + c;
    };
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 4 * stride) {
        uint4 v[4];
        uint4 *d[4];
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            const uint64_t idx = i + u * stride;
            d[u] = nullptr;
            if (idx < total) {
                const uint4 *s;
                locate(idx, s, d[u]);
                v[u] = __ldg(s);
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
            if (d[u])
                *d[u] = v[u];
    }
}

// The same drain through shared memory and TMA stores, for a C whose rows are 16-byte aligned (c_tma_ok): per 64
// columns the warp converts its 32 rows to bf16, writes them as 128-byte rows into one of its two 4 KiB staging
// buffers in the layout the tensor map's 128-byte swizzle expects (16-byte chunk j of row r sits at chunk
// j ^ (r & 7)), and one lane hands the 32 x 64 box to the TMA unit, which writes whole 128-byte lines and clips
// what lies beyond M or N.  The stores are asynchronous: `buf` alternates between the two buffers, and a buffer is
// rewritten only after the store that last used it has read it.  `stage_u32` = shared-window address of the
// warp's 8 KiB staging area (1024-byte aligned).  The caller ends with tma_store_drain() before the CTA exits.
template <uint32_t BN>
__device__ __forceinline__ void drain_accumulator_tma(const GemmParams &p, const CUtensorMap *tma_c, uint32_t stage_u32,
                                                      uint32_t tmem_acc, uint32_t quarter, uint32_t lane,
                                                      uint32_t tile_row0, uint32_t tile_col0, uint32_t &buf)
{
    static_assert(BN % 64 == 0, "the TMA-store epilogue works in groups of 64 columns");
    const uint32_t taddr = tmem_acc + ((quarter * 32u) << 16);
    const uint32_t row0 = tile_row0 + quarter * 32u;
    if (row0 >= p.m)
        return;
#pragma unroll 1
    for (uint32_t g = 0; g < BN / 64; ++g) {
        const uint32_t col0 = tile_col0 + g * 64u;
        if (col0 >= p.n)
            break;
        uint32_t v0[32], v1[32];
        ptx::tmem_ld_32x32b_x32(taddr + g * 64u, v0);
        ptx::tmem_ld_32x32b_x32(taddr + g * 64u + 32u, v1);
        ptx::tmem_ld_wait();
        if (lane == 0)
            ptx::bulk_wait_group_read<1>();  // the store before the last one (same buffer) has read its source
        __syncwarp();
        const uint32_t base = stage_u32 + buf * kTmaStoreBufBytes;
        const uint32_t row = base + lane * 128u;
        const uint32_t sw = lane & 7u;
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            ptx::st_shared_v4(row + ((j ^ sw) << 4), ptx::pack_bf16x2(v0[8 * j], v0[8 * j + 1]),
                              ptx::pack_bf16x2(v0[8 * j + 2], v0[8 * j + 3]), ptx::pack_bf16x2(v0[8 * j + 4], v0[8 * j + 5]),
                              ptx::pack_bf16x2(v0[8 * j + 6], v0[8 * j + 7]));
            ptx::st_shared_v4(row + (((j + 4u) ^ sw) << 4), ptx::pack_bf16x2(v1[8 * j], v1[8 * j + 1]),
                              ptx::pack_bf16x2(v1[8 * j + 2], v1[8 * j + 3]), ptx::pack_bf16x2(v1[8 * j + 4], v1[8 * j + 5]),
                              ptx::pack_bf16x2(v1[8 * j + 6], v1[8 * j + 7]));
        }
        ptx::fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) {
            // C passes through L2 once: its lines are the first to go, so that they do not push operand panels out
            if (p.c_evict_first)
                ptx::tma_store_2d_hint(tma_c, base, static_cast<int32_t>(col0), static_cast<int32_t>(row0),
                                       ptx::policy_evict_first());
            else
                ptx::tma_store_2d(tma_c, base, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
            ptx::bulk_commit_group();
        }
        buf ^= 1u;
    }
}

// Waits until every TMA store this warp issued has been performed (lane 0 issued them).
__device__ __forceinline__ void tma_store_drain(uint32_t lane)
{
    if (lane == 0)
        ptx::bulk_wait_group<0>();
    __syncwarp();
}

// One CTA waits on a barrier that nothing completes; exercises the bounded wait.
__global__ void wait_expires_kernel(DeviceStatus *status, uint64_t budget_ns)
{
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        ptx::fence_barrier_init();
        const WaitCtl ctl{&abort_flag, status, budget_ns};
        (void)wait_bounded(ptx::smem_u32(&bar), 0, ctl, 9);
    }
}

}  // namespace maize
