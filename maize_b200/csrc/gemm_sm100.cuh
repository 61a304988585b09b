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
//   accumulators summed and dropped (main.rs:71)    tcgen05.ld -> cvt.rn.bf16x2 -> swizzled shared memory -> TMA stores
//                                                     (aligned C rows) or masked direct stores (any other C)
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
#include "gemm_common.cuh"

namespace maize {

template <uint32_t BN, uint32_t STAGES>
struct GemmSmemLayout {
    static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;  // 16 KiB
    static constexpr uint32_t kBBytes = BN * kBlockK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    // after the ring: epilogue staging, then full[STAGES], empty[STAGES], acc_full[2], acc_empty[2],
    // the TMEM base slot and the abort flag
    static constexpr uint32_t kStagingOffset = kRingBytes;
    static constexpr uint32_t kBarOffset = kStagingOffset + kTmaStageBytesTotal;
    static constexpr uint32_t kNumBars = 2 * STAGES + 4;
    static constexpr uint32_t kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr uint32_t kAbortOffset = kTmemSlotOffset + 4;
    static constexpr uint32_t kUsedBytes = kAbortOffset + 4;
    static constexpr uint32_t kDynamicBytes = kUsedBytes + 1024;  // slack for the 1024-byte alignment
    static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128B swizzle");
    static_assert(kBarOffset % 16 == 0, "barriers need 8-byte, staging rows 16-byte alignment");
    static_assert(kDynamicBytes <= 232448, "exceeds 227 KiB of shared memory per CTA");
    // one CTA per SM by construction, so the 2*BN TMEM columns never oversubscribe the SM's 512
    static_assert(kDynamicBytes > 116224, "two CTAs could share an SM and contend for TMEM");
};

// B_KN: B is given K x N row-major (N contiguous) instead of N x K; its tiles are then loaded as BN / 64
// boxes of {64 columns, 64 k-rows} and read by the MMA as an MN-major operand.
template <uint32_t BN, uint32_t STAGES, bool B_KN = false>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_1cta(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_c, const GemmParams p)
{
    using L = GemmSmemLayout<BN, STAGES>;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "UMMA N for M = 128 must be a multiple of 16 up to 256");
    constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers; 64..512, a power of two
    static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols >= 32 && kTmemCols <= 512, "bad TMEM size");
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kBlockM, BN, B_KN);
    constexpr uint32_t kChunkBytes = kBlockK * 128;  // one 64-column chunk of a K x N tile: 64 k-rows x 128 B
    static_assert(!B_KN || BN % 64 == 0, "K x N tiles are loaded in chunks of 64 columns");

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
    const bool prof = p.profile != nullptr;
    unsigned long long *prof_out = prof ? p.profile + static_cast<size_t>(blockIdx.x) * kProfileSlots : nullptr;
    const long long t_start = prof ? ptx::sm_clock64() : 0;

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tma_a);
        ptx::prefetch_tensormap(&tma_b);
        if (p.c_tma_ok)
            ptx::prefetch_tensormap(&tma_c);
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
    if (p.pdl) {
        // Launched with programmatic stream serialization: the set-up above overlapped the tail of the stream's
        // previous kernel; nothing below (operand loads, stores to C) may run before that kernel has completed.
        if (threadIdx.x == 0)
            ptx::grid_dependency_launch_dependents();  // the next kernel may be scheduled as SMs free up
        ptx::grid_dependency_wait();
    }

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            unsigned long long w_empty = 0;
            int32_t gate_seen = 0;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                const TileCoord tc = tile_coord(t, p);
                const bool hot = (p.debug_flags & 1u) != 0u;
                const int32_t m0 = hot ? 0 : static_cast<int32_t>(tc.m_blk * kBlockM);
                const int32_t n0 = hot ? 0 : static_cast<int32_t>(tc.n_blk * BN);
                if (!(ok = gate_rows_landed(p, static_cast<uint32_t>(m0) + kBlockM, gate_seen, ctl)))
                    break;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    WaitTimer wt(prof);
                    ok = wait_bounded(empty_bar(stage), phase ^ 1u, ctl, 1);
                    wt.stop(w_empty);
                    if (!ok)
                        break;
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + L::kABytes;
                    if (p.debug_flags & 2u) {
                        ptx::mbar_arrive(full_bar(stage));
                    } else {
                        ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                        ptx::tma_load_2d(sa, &tma_a, full_bar(stage), static_cast<int32_t>(kb * kBlockK), m0);
                        if constexpr (B_KN) {
#pragma unroll
                            for (uint32_t j = 0; j < BN / 64; ++j)  // x = column, y = k row
                                ptx::tma_load_2d(sb + j * kChunkBytes, &tma_b, full_bar(stage),
                                                 n0 + static_cast<int32_t>(64u * j), static_cast<int32_t>(kb * kBlockK));
                        } else {
                            ptx::tma_load_2d(sb, &tma_b, full_bar(stage), static_cast<int32_t>(kb * kBlockK), n0);
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (prof)
                prof_out[kProfProducerWaitEmpty] = w_empty;
        }
        __syncwarp();
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            unsigned long long w_full = 0, w_acc = 0;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                {
                    WaitTimer wt(prof);
                    ok = wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2);
                    wt.stop(w_acc);
                }
                if (!ok)
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    {
                        WaitTimer wt(prof);
                        ok = wait_bounded(full_bar(stage), phase, ctl, 2);
                        wt.stop(w_full);
                    }
                    if (!ok)
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint64_t da = ptx::make_smem_desc_sw128(sa);
                    const uint64_t db = B_KN ? ptx::make_smem_desc_sw128_mn(sa + L::kABytes, kChunkBytes)
                                             : ptx::make_smem_desc_sw128(sa + L::kABytes);
                    // per 16-element K step: +32 bytes in a K-major tile (+2 in the address >> 4 field),
                    // +2048 bytes (two groups of 8 k-rows) in a K x N tile (+128)
                    constexpr uint32_t kStepB = B_KN ? 128u : 2u;
#pragma unroll
                    for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                        ptx::mma_bf16_1cta(tmem_d, da + 2u * k, db + kStepB * k, kIdesc, (kb | k) != 0u ? 1u : 0u);
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
            if (prof) {
                prof_out[kProfMmaWaitFull] = w_full;
                prof_out[kProfMmaWaitAccEmpty] = w_acc;
            }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue --
        const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
        uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        const uint32_t stage_u32 = smem_base + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        uint32_t store_buf = 0;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        unsigned long long w_accfull = 0, w_drain = 0, n_tiles_done = 0;
        for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
            const TileCoord tc = tile_coord(t, p);
            {
                WaitTimer wt(prof);
                ok = wait_bounded(acc_full_bar(acc), acc_phase, ctl, 3);
                wt.stop(w_accfull);
            }
            // keep the warp converged for the .sync.aligned TMEM loads
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            WaitTimer dt(prof);
            if constexpr (BN % 64 == 0) {
                if (p.c_tma_ok)
                    drain_accumulator_tma<BN>(p, &tma_c, stage_u32, tmem_base + acc * BN, quarter, lane, tc.m_blk * kBlockM,
                                              tc.n_blk * BN, store_buf);
                else
                    drain_accumulator<BN>(p, stage_warp, tmem_base + acc * BN, quarter, lane, tc.m_blk * kBlockM,
                                          tc.n_blk * BN);
            } else {
                drain_accumulator<BN>(p, stage_warp, tmem_base + acc * BN, quarter, lane, tc.m_blk * kBlockM,
                                      tc.n_blk * BN);
            }
            dt.stop(w_drain);
            ++n_tiles_done;
            ptx::tcgen05_fence_before();
            ptx::mbar_arrive(acc_empty_bar(acc));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (p.c_tma_ok)
            tma_store_drain(lane);  // the staging buffers must outlive the stores that read them
        if (prof && warp == 2 && lane == 0) {
            prof_out[kProfEpilogueWaitAccFull] = w_accfull;
            prof_out[kProfEpilogueDrain] = w_drain;
            prof_out[kProfTiles] = n_tiles_done;
        }
    }

    // ---------------------------------------------------------------- teardown --
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (prof && threadIdx.x == 0)
        prof_out[kProfCtaCycles] = static_cast<unsigned long long>(ptx::sm_clock64() - t_start);
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

}  // namespace maize
