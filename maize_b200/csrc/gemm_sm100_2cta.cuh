// CTA-pair (cta_group::2) variant of the persistent BF16 GEMM: two CTAs on the two
// SMs of a TPC compute one 256 x 256 tile of C together.
//
//   - CTA r of the pair (r = %cluster_ctarank, 0 = leader) owns rows r*128..r*128+127
//     of the tile: it loads those 128 rows of A and ONE HALF (128 of 256 rows) of the
//     B tile per k-block into its own shared memory, so each SM pulls 32 KiB per
//     k-block instead of 48 KiB and the ring holds 6 k-blocks instead of 4.
//   - Every CTA issues its own TMA loads (none is shared between CTAs); the peer's loads
//     signal their bytes on the LEADER's full barrier, which expects both halves.
//   - One thread of the leader issues tcgen05.mma.cta_group::2 (M = 256, N = 256,
//     K = 16); the hardware reads A and B from both CTAs' shared memory at equal
//     offsets and writes rows 0-127 of the accumulator to the leader's TMEM and
//     rows 128-255 to the peer's.
//   - Stage release and accumulator hand-over are one tcgen05.commit each that
//     arrives on the barrier of both CTAs (two separate commits, one per CTA, cost
//     7% more cycles when measured).
//   - Both CTAs drain their own 128 x 256 accumulator half; one lane per epilogue
//     warp arrives on the leader's acc_empty barrier (8 arrivals per buffer).
//   - KBS = k-blocks per ring stage (1 or 2): with 2 the leader commits once per
//     eight MMAs instead of once per four.
//
// Role split, bounded waits and teardown follow the one-CTA kernel; a cluster
// barrier brackets the body so that no CTA exits while its peer can still signal
// one of its barriers or read its shared memory.
#pragma once
#include "gemm_common.cuh"

namespace maize {

constexpr uint32_t kPairBlockM = 256;

template <uint32_t BN, uint32_t KBS, uint32_t STAGES>
struct PairSmemLayout {
    static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;          // this CTA's 128 rows of A, one k-block
    static constexpr uint32_t kBBytes = (BN / 2) * kBlockK * 2;         // this CTA's half of the B tile, one k-block
    static constexpr uint32_t kStageBytes = KBS * (kABytes + kBBytes);  // [A0..A(KBS-1), B0..B(KBS-1)]
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    static constexpr uint32_t kStagingOffset = kRingBytes;
    static constexpr uint32_t kBarOffset = kStagingOffset + kTmaStageBytesTotal;
    static constexpr uint32_t kNumBars = 2 * STAGES + 4;
    static constexpr uint32_t kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr uint32_t kAbortOffset = kTmemSlotOffset + 4;
    static constexpr uint32_t kUsedBytes = kAbortOffset + 4;
    static constexpr uint32_t kDynamicBytes = kUsedBytes + 1024;
    static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128B swizzle");
    static_assert(kDynamicBytes <= 232448, "exceeds 227 KiB of shared memory per CTA");
    static_assert(kDynamicBytes > 116224, "two CTAs could share an SM and contend for TMEM");
};

// B_KN: B is given K x N row-major; this CTA's 128-column half of the B tile is loaded as two boxes of
// {64 columns, 64 k-rows} per k-block and read by the MMA as an MN-major operand.
template <uint32_t BN, uint32_t KBS, uint32_t STAGES, bool B_KN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_2cta(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_c, const GemmParams p)
{
    using L = PairSmemLayout<BN, KBS, STAGES>;
    static_assert(BN == 256, "pair tile is 256 x 256");
    static_assert(KBS == 1 || KBS == 2, "one or two k-blocks per stage");
    constexpr uint32_t kTmemCols = 2 * BN;  // two BN-column accumulator buffers per CTA
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kPairBlockM, BN, B_KN);
    constexpr uint32_t kStepK = KBS * kBlockK;
    constexpr uint32_t kChunkBytes = kBlockK * 128;  // one 64-column chunk of a K x N tile: 64 k-rows x 128 B

    extern __shared__ uint8_t smem_raw[];
    // Both CTAs of the pair see the same dynamic shared-memory base offset, so the aligned
    // bases agree; the MMA needs identical operand offsets in the two CTAs.
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
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t num_steps = (p.k + kStepK - 1) / kStepK;
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
            ptx::mbar_init(full_bar(s), 1);   // the leader's producer; bytes of both CTAs
            ptx::mbar_init(empty_bar(s), 1);  // one tcgen05.commit of the leader
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(acc_full_bar(b), 1);
            ptx::mbar_init(acc_empty_bar(b), 2 * kNumEpilogueWarps);  // one lane per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_2cta(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish_2cta();
    }
    ptx::tcgen05_fence_before();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.pdl) {
        // Launched with programmatic stream serialization: the set-up above overlapped the tail of the stream's
        // previous kernel; nothing below (operand loads, stores to C) may run before that kernel has completed.
        if (threadIdx.x == 0)
            ptx::grid_dependency_launch_dependents();  // the next kernel may be scheduled as SMs free up
        ptx::grid_dependency_wait();
    }

    bool role_ok = true;
    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            unsigned long long w_empty = 0;
            int32_t gate_seen = 0;
            // L2 policy: the row panel of A is re-read by every column block of the sweep, B passes once
            const bool hints = (p.debug_flags & 4u) != 0u;
            const uint64_t pol_a = hints ? ptx::policy_evict_last() : ptx::policy_evict_normal();
            const uint64_t pol_b = (p.debug_flags & 8u) ? ptx::policy_evict_first() : ptx::policy_evict_normal();
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                const TileCoord tc = tile_coord(t, p);
                const bool hot = (p.debug_flags & 1u) != 0u;
                const int32_t m0 = static_cast<int32_t>((hot ? 0 : tc.m_blk * kPairBlockM) + cta_rank * kBlockM);
                const int32_t n0 = static_cast<int32_t>((hot ? 0 : tc.n_blk * BN) + cta_rank * (BN / 2));
                if (!(ok = gate_rows_landed(p, static_cast<uint32_t>(m0) + kBlockM, gate_seen, ctl)))
                    break;
                for (uint32_t step = 0; step < num_steps; ++step) {
                    WaitTimer wt(prof);
                    ok = wait_bounded<true>(empty_bar(stage), phase ^ 1u, ctl, 1);
                    wt.stop(w_empty);
                    if (!ok)
                        break;
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + KBS * L::kABytes;
                    const uint32_t leader_full = ptx::mapa_shared(full_bar(stage), 0);
                    if (p.debug_flags & 2u) {
                        if (cta_rank == 0)
                            ptx::mbar_arrive(full_bar(stage));
                    } else {
                        if (cta_rank == 0)
                            ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
#pragma unroll
                        for (uint32_t sub = 0; sub < KBS; ++sub) {
                            // a k-block past the end of K is fetched all the same: TMA fills it with zeros
                            const int32_t kx = static_cast<int32_t>((step * KBS + sub) * kBlockK);
                            ptx::tma_load_2d_pair_hint(sa + sub * L::kABytes, &tma_a, leader_full, kx, m0, pol_a);
                            if constexpr (B_KN) {
#pragma unroll
                                for (uint32_t j = 0; j < BN / 128; ++j)  // x = column, y = k row
                                    ptx::tma_load_2d_pair_hint(sb + sub * L::kBBytes + j * kChunkBytes, &tma_b, leader_full,
                                                               n0 + static_cast<int32_t>(64u * j), kx, pol_b);
                            } else {
                                ptx::tma_load_2d_pair_hint(sb + sub * L::kBBytes, &tma_b, leader_full, kx, n0, pol_b);
                            }
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            role_ok = ok;
            if (prof)
                prof_out[kProfProducerWaitEmpty] = w_empty;
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------- MMA issuer (leader only) --
        if (lane == 0 && cta_rank == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            unsigned long long w_full = 0, w_acc = 0;
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                {
                    WaitTimer wt(prof);
                    ok = wait_bounded<true>(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2);
                    wt.stop(w_acc);
                }
                if (!ok)
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t step = 0; step < num_steps; ++step) {
                    {
                        WaitTimer wt(prof);
                        ok = wait_bounded<true>(full_bar(stage), phase, ctl, 2);
                        wt.stop(w_full);
                    }
                    if (!ok)
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + KBS * L::kABytes;
#pragma unroll
                    for (uint32_t sub = 0; sub < KBS; ++sub) {
                        const uint64_t da = ptx::make_smem_desc_sw128(sa + sub * L::kABytes);
                        const uint64_t db = B_KN ? ptx::make_smem_desc_sw128_mn(sb + sub * L::kBBytes, kChunkBytes)
                                                 : ptx::make_smem_desc_sw128(sb + sub * L::kBBytes);
                        constexpr uint32_t kStepB = B_KN ? 128u : 2u;  // +2048 B or +32 B per 16-wide K step
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                            ptx::mma_bf16_2cta(tmem_d, da + 2u * k, db + kStepB * k, kIdesc,
                                               (step | sub | k) != 0u ? 1u : 0u);
                    }
                    ptx::mma_commit_2cta_mask(empty_bar(stage), 3);  // stage s of both CTAs is free
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_2cta_mask(acc_full_bar(acc), 3);  // both halves of the accumulator are complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            role_ok = ok;
            if (prof) {
                prof_out[kProfMmaWaitFull] = w_full;
                prof_out[kProfMmaWaitAccEmpty] = w_acc;
            }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue --
        const uint32_t quarter = warp & 3u;
        uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        const uint32_t stage_u32 = smem_base + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        uint32_t store_buf = 0;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        unsigned long long w_accfull = 0, w_drain = 0, n_tiles_done = 0;
        for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
            const TileCoord tc = tile_coord(t, p);
            {
                WaitTimer wt(prof);
                ok = wait_bounded<true>(acc_full_bar(acc), acc_phase, ctl, 3);
                wt.stop(w_accfull);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            WaitTimer dt(prof);
            if (p.c_tma_ok)
                drain_accumulator_tma<BN>(p, &tma_c, stage_u32, tmem_base + acc * BN, quarter, lane,
                                          tc.m_blk * kPairBlockM + cta_rank * kBlockM, tc.n_blk * BN, store_buf);
            else
                drain_accumulator<BN>(p, stage_warp, tmem_base + acc * BN, quarter, lane,
                                      tc.m_blk * kPairBlockM + cta_rank * kBlockM, tc.n_blk * BN);
            dt.stop(w_drain);
            ++n_tiles_done;
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive_cluster_addr(ptx::mapa_shared(acc_empty_bar(acc), 0));
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
        role_ok = ok;
    }
    if (!role_ok) {
        // tell the peer CTA too, so that its roles stop waiting on us
        ptx::st_shared_cluster_u32(ptx::mapa_shared(ptx::smem_u32(const_cast<int *>(abort_flag)), cta_rank ^ 1u), 1u);
    }

    // ---------------------------------------------------------------- teardown --
    __syncwarp();
    ptx::tcgen05_fence_before();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (prof && threadIdx.x == 0)
        prof_out[kProfCtaCycles] = static_cast<unsigned long long>(ptx::sm_clock64() - t_start);
    if (warp == 1) {
        if (*abort_flag) {
            for (int i = 0; i < 256; ++i)
                __nanosleep(1000);
        }
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

}  // namespace maize
