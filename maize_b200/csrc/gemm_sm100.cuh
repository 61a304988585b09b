// Persistent, warp-specialised BF16 GEMM for sm_100a, one CTA per SM:
//   C[M x N] (bf16) = A[M x K] (bf16, row-major) * B[N x K]^T (bf16, row-major), fp32 accumulate.
//
// It takes over the role of the reference's per-warp tile GEMM
// sm80_gemm_smem_multibuffer (crates/maize_tile/src/gemm/mod.rs:37-90) and of the
// grid-stride panel loops around it (src/main.rs:56-73), restated for Blackwell:
//
//   reference                                       here
//   ---------------------------------------------   ------------------------------------------
//   16x16 C tile per warp, 4 warps duplicate it     128 x BN C tile per CTA (BN = 256/128/64/32)
//   cp.async 16-B copies, unswizzled smem           TMA boxes, 128-byte swizzle, zero fill at the
//     (gmem_tile.rs:42-239)                           ragged M/N/K edges
//   commit_group / wait_group ring, depth 4         full/empty mbarrier ring, STAGES deep
//     (cp_async.rs:98-253)
//   ldmatrix + 2x mma.m16n8k16 per k-step           4x tcgen05.mma (128 x BN x 16) per 64-wide k-block,
//     (gemm/mod.rs:18-33, mma/sm80.rs:136-160)        issued by one thread, fp32 accumulator in TMEM
//   accumulators summed and dropped (main.rs:71)    tcgen05.ld -> cvt.rn.bf16x2 -> stores with row/col masks
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2-5 = epilogue (warp w reads TMEM lanes 32*(w%4)...).  Two accumulator
// buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
// No wait in this file is unbounded: each try_wait loop carries a time budget and
// watches a CTA-wide abort flag.  On expiry the kernel records MAIZE_ERR_TIMEOUT in
// the status word, every role falls through to the common teardown, in-flight
// copies get time to land, TMEM is freed and the kernel returns.  Nothing traps.
#pragma once
#include "ptx_sm100.cuh"

namespace maize {

constexpr int kStatusOk = 0;
constexpr int kStatusTimeout = 4;      // == MAIZE_ERR_TIMEOUT
constexpr int kStatusDeviceAbort = 5;  // == MAIZE_ERR_DEVICE_ABORT

// Device status block: [0] worst status code, [1] role that gave up, [2] CTA, [3] spare.
struct DeviceStatus {
    int code;
    int role;
    int cta;
    int detail;
};

constexpr uint32_t kBlockM = 128;  // rows of C per CTA tile = TMEM lanes = UMMA M
constexpr uint32_t kBlockK = 64;   // bf16 elements per k-block = one 128-byte swizzle row
constexpr uint32_t kUmmaK = 16;    // K per tcgen05.mma for 16-bit operands
constexpr uint32_t kNumThreads = 192;
constexpr uint32_t kNumEpilogueThreads = 128;

struct WaitCtl {
    volatile int *abort_flag;  // shared memory, CTA-wide
    DeviceStatus *status;      // global memory
    uint64_t budget_ns;
};

// Bounded wait on an mbarrier phase.  Returns false if the budget ran out or some
// other role of this CTA already gave up.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const WaitCtl &ctl, int role)
{
    if (ptx::mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = ptx::global_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (ptx::mbar_try_wait(bar, parity))
            return true;
        if ((it & 31u) == 0u) {
            if (*ctl.abort_flag)
                return false;
            if (ptx::global_timer_ns() - t0 > ctl.budget_ns) {
                *ctl.abort_flag = 1;
                if (atomicMax(&ctl.status->code, kStatusTimeout) < kStatusTimeout) {
                    ctl.status->role = role;
                    ctl.status->cta = static_cast<int>(blockIdx.x);
                }
                return false;
            }
        }
    }
}

// Tile order: groups of kGroupM row-blocks sweep all column-blocks, so that the
// CTAs running at one time share A row panels and B column panels in L2.
struct TileCoord {
    uint32_t m_blk, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m)
{
    const uint32_t per_group = group_m * tiles_n;
    const uint32_t g = t / per_group;
    const uint32_t first_m = g * group_m;
    const uint32_t rows = min(tiles_m - first_m, group_m);
    const uint32_t r = t - g * per_group;
    TileCoord c;
    c.m_blk = first_m + r % rows;
    c.n_blk = r / rows;
    return c;
}

template <uint32_t BN, uint32_t STAGES>
struct GemmSmemLayout {
    static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;  // 16 KiB
    static constexpr uint32_t kBBytes = BN * kBlockK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    // after the ring: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot, abort flag
    static constexpr uint32_t kBarOffset = kRingBytes;
    static constexpr uint32_t kNumBars = 2 * STAGES + 4;
    static constexpr uint32_t kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr uint32_t kAbortOffset = kTmemSlotOffset + 4;
    static constexpr uint32_t kUsedBytes = kAbortOffset + 4;
    static constexpr uint32_t kDynamicBytes = kUsedBytes + 1024;  // slack for the 1024-byte alignment
    static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128B swizzle");
    static_assert(kDynamicBytes <= 232448, "exceeds 227 KiB of shared memory per CTA");
};

struct GemmParams {
    __nv_bfloat16 *c;
    uint64_t ldc;  // elements
    uint32_t m, n, k;
    uint32_t tiles_m, tiles_n;
    uint32_t group_m;
    uint32_t c_vec_ok;  // 1: C rows start 16-byte aligned (ldc % 8 == 0 and base aligned)
    DeviceStatus *status;
    uint64_t timeout_ns;
};

// Convert 32 fp32 accumulators of one C row to bf16 and store columns [col0, col0+32) ∩ [0, n).
__device__ __forceinline__ void store_row_chunk(const GemmParams &p, uint32_t row, uint32_t col0,
                                                const uint32_t (&acc)[32])
{
    if (row >= p.m || col0 >= p.n)
        return;
    __nv_bfloat16 *dst = p.c + static_cast<uint64_t>(row) * p.ldc + col0;
    if (p.c_vec_ok && col0 + 32 <= p.n) {
        uint4 *dst4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint4 q;
            q.x = ptx::pack_bf16x2(acc[8 * v + 0], acc[8 * v + 1]);
            q.y = ptx::pack_bf16x2(acc[8 * v + 2], acc[8 * v + 3]);
            q.z = ptx::pack_bf16x2(acc[8 * v + 4], acc[8 * v + 5]);
            q.w = ptx::pack_bf16x2(acc[8 * v + 6], acc[8 * v + 7]);
            dst4[v] = q;
        }
    } else {
        const uint32_t valid = min(32u, p.n - col0);
#pragma unroll
        for (uint32_t j = 0; j < 32; ++j) {
            if (j < valid)
                dst[j] = __float2bfloat16_rn(__uint_as_float(acc[j]));
        }
    }
}

template <uint32_t BN, uint32_t STAGES>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_1cta(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const GemmParams p)
{
    using L = GemmSmemLayout<BN, STAGES>;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "UMMA N for M = 128 must be a multiple of 16 up to 256");
    constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers; 64..512, a power of two
    static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols >= 32 && kTmemCols <= 512, "bad TMEM size");
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kBlockM, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + L::kTmemSlotOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + L::kAbortOffset);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t num_kb = (p.k + kBlockK - 1) / kBlockK;
    const WaitCtl ctl{abort_flag, p.status, p.timeout_ns};

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tma_a);
        ptx::prefetch_tensormap(&tma_b);
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(acc_full_bar(b), 1);
            ptx::mbar_init(acc_empty_bar(b), kNumEpilogueThreads);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_1cta(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish_1cta();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                const TileCoord tc = tile_coord(t, p.tiles_m, p.tiles_n, p.group_m);
                const int32_t m0 = static_cast<int32_t>(tc.m_blk * kBlockM);
                const int32_t n0 = static_cast<int32_t>(tc.n_blk * BN);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = wait_bounded(empty_bar(stage), phase ^ 1u, ctl, 1)))
                        break;
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + L::kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                    ptx::tma_load_2d(sa, &tma_a, full_bar(stage), static_cast<int32_t>(kb * kBlockK), m0);
                    ptx::tma_load_2d(sb, &tma_b, full_bar(stage), static_cast<int32_t>(kb * kBlockK), n0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                if (!(ok = wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2)))
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = wait_bounded(full_bar(stage), phase, ctl, 2)))
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint64_t da = ptx::make_smem_desc_sw128(sa);
                    const uint64_t db = ptx::make_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
                    for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k) {
                        // +32 bytes per 16-element K step: +2 in the (address >> 4) field
                        ptx::mma_bf16_1cta(tmem_d, da + 2u * k, db + 2u * k, kIdesc, (kb | k) != 0u ? 1u : 0u);
                    }
                    ptx::mma_commit_1cta(empty_bar(stage));  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_1cta(acc_full_bar(acc));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue --
        const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(t, p.tiles_m, p.tiles_n, p.group_m);
            const uint32_t row = tc.m_blk * kBlockM + quarter * 32u + lane;
            const uint32_t n0 = tc.n_blk * BN;
            ok = wait_bounded(acc_full_bar(acc), acc_phase, ctl, 3);
            // keep the warp converged for the .sync.aligned TMEM loads
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * BN;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                ptx::tmem_ld_wait();
                store_row_chunk(p, row, n0 + c * 32u, v);
            }
            ptx::tcgen05_fence_before();
            ptx::mbar_arrive(acc_empty_bar(acc));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------------------------------------------------------- teardown --
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            // A role gave up: let TMA copies and MMAs still in flight finish before
            // shared memory and TMEM are handed back (bounded: about 0.3 ms).
            for (int i = 0; i < 256; ++i)
                __nanosleep(1000);
        }
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc_1cta(tmem_base, kTmemCols);
    }
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
