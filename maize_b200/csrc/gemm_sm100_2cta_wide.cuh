// CTA-pair (cta_group::2) BF16 GEMM with a 256 x 512 tile of C per pair: the widest tile the 512 columns of
// tensor memory hold.
//
// Against the 256 x 256 pair kernel of gemm_sm100_2cta.cuh it trades the second accumulator buffer for a
// second half of the tile.  Per 64-wide k-block a CTA loads its 128 rows of A (16 KiB) and its 128-row halves of
// TWO 256-row blocks of B (32 KiB) and the leader issues two M = 256, N = 256 MMAs per 16-wide k-step that share
// the A operand: 48 KiB per 128 x 512 x 64 multiply-accumulates per CTA instead of 32 KiB per 128 x 256 x 64, a
// quarter less traffic from L2 to shared memory per flop, and with twice the tile area in flight per wave about a
// third less traffic from DRAM.  The part is power-limited, so bytes not moved are clock gained.
//
// The price is that the epilogue can no longer hide behind the next tile's whole main loop.  What is left of
// the overlap: the epilogue drains the accumulator's first half (columns 0..255 of tensor memory), releases it,
// then drains the second half; the MMA thread starts the next tile on the first half as soon as that is free and
// runs it ahead by up to a ring's worth of k-blocks (their stages stay held until the second half has used them
// too), then waits for the second half.  The host picks this kernel only for long K, where the exposed part of
// the drain is about a percent of a tile's time.
//
// Roles, barriers, bounded waits and teardown otherwise follow gemm_sm100_2cta.cuh: every CTA issues its own TMA
// loads (none is shared between CTAs) whose bytes are counted on the LEADER's full barrier; one tcgen05.commit
// with a CTA mask releases a stage in both CTAs; a cluster barrier brackets the body.
//
// In the reference's terms this is still the per-tile GEMM of crates/maize_tile/src/gemm/mod.rs:37-90 under the
// grid-stride over (row panel, column panel) pairs of src/main.rs:56-73, with a column panel 512 wide.
#pragma once
#include "gemm_sm100_2cta.cuh"

namespace maize {

constexpr uint32_t kWideBlockN = 512;

template <uint32_t STAGES>
struct WideSmemLayout {
    static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;     // this CTA's 128 rows of A, one k-block: 16 KiB
    static constexpr uint32_t kBHalfBytes = 128 * kBlockK * 2;     // this CTA's half of one 256-row block of B: 16 KiB
    static constexpr uint32_t kStageBytes = kABytes + 2 * kBHalfBytes;  // [A, B block 0 half, B block 1 half]
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    static constexpr uint32_t kStagingOffset = kRingBytes;
    static constexpr uint32_t kBarOffset = kStagingOffset + kTmaStageBytesTotal;
    // full[STAGES], empty[STAGES], acc_full, acc_free[2]
    static constexpr uint32_t kNumBars = 2 * STAGES + 3;
    static constexpr uint32_t kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr uint32_t kAbortOffset = kTmemSlotOffset + 4;
    static constexpr uint32_t kUsedBytes = kAbortOffset + 4;
    static constexpr uint32_t kDynamicBytes = kUsedBytes + 1024;
    static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128B swizzle");
    static_assert(kDynamicBytes <= 232448, "exceeds 227 KiB of shared memory per CTA");
    static_assert(kDynamicBytes > 116224, "two CTAs could share an SM and contend for TMEM");
};

template <uint32_t STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_2cta_wide(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                          const __grid_constant__ CUtensorMap tma_c, const GemmParams p)
{
    using L = WideSmemLayout<STAGES>;
    constexpr uint32_t kHalfN = 256;                 // columns per MMA and per half of the accumulator
    constexpr uint32_t kTmemCols = 2 * kHalfN;       // ONE accumulator of 512 columns
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kPairBlockM, kHalfN, false);

    extern __shared__ uint8_t smem_raw[];
    // Both CTAs of the pair see the same dynamic shared-memory base offset, so the aligned bases agree; the MMA
    // needs identical operand offsets in the two CTAs.
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * STAGES);
    auto acc_free_bar = [&](uint32_t h) { return bar_base + 8u * (2 * STAGES + 1 + h); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + L::kTmemSlotOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + L::kAbortOffset);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;  // tiles of 256 x 512
    const uint32_t num_kb = (p.k + kBlockK - 1) / kBlockK;
    const WaitCtl ctl{abort_flag, p.status, p.timeout_ns};

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tma_a);
        ptx::prefetch_tensormap(&tma_b);
        if (p.c_tma_ok)
            ptx::prefetch_tensormap(&tma_c);
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);   // the leader's producer; bytes of both CTAs
            ptx::mbar_init(empty_bar(s), 1);  // one tcgen05.commit of the leader
        }
        ptx::mbar_init(acc_full_bar, 1);
        for (uint32_t h = 0; h < 2; ++h)
            ptx::mbar_init(acc_free_bar(h), 2 * kNumEpilogueWarps);  // one lane per epilogue warp of both CTAs
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
            ptx::grid_dependency_launch_dependents();
        ptx::grid_dependency_wait();
    }

    bool role_ok = true;
    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int32_t gate_seen = 0;
            const uint64_t pol = ptx::policy_evict_normal();
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                const TileCoord tc = tile_coord(t, p);
                const int32_t m0 = static_cast<int32_t>(tc.m_blk * kPairBlockM + cta_rank * kBlockM);
                const int32_t n0 = static_cast<int32_t>(tc.n_blk * kWideBlockN + cta_rank * 128u);
                if (!(ok = gate_rows_landed(p, static_cast<uint32_t>(m0) + kBlockM, gate_seen, ctl)))
                    break;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = wait_bounded<true>(empty_bar(stage), phase ^ 1u, ctl, 1);
                    if (!ok)
                        break;
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + L::kABytes;
                    const uint32_t leader_full = ptx::mapa_shared(full_bar(stage), 0);
                    if (cta_rank == 0)
                        ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
                    // a k-block past the end of K, rows past M and rows of B past N are fetched all the same: TMA
                    // fills them with zeros
                    const int32_t kx = static_cast<int32_t>(kb * kBlockK);
                    ptx::tma_load_2d_pair_hint(sa, &tma_a, leader_full, kx, m0, pol);
                    ptx::tma_load_2d_pair_hint(sb, &tma_b, leader_full, kx, n0, pol);
                    ptx::tma_load_2d_pair_hint(sb + L::kBHalfBytes, &tma_b, leader_full, kx, n0 + static_cast<int32_t>(kHalfN),
                                               pol);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            role_ok = ok;
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------- MMA issuer (leader only) --
        if (lane == 0 && cta_rank == 0) {
            uint32_t stage = 0, phase = 0;  // next stage to consume
            uint32_t free_phase = 0;        // phase of the acc_free barriers for the current tile
            bool ok = true;
            auto issue_half = [&](uint32_t st, uint32_t half, bool first_kb) {
                const uint32_t sa = smem_base + st * L::kStageBytes;
                const uint64_t da = ptx::make_smem_desc_sw128(sa);
                const uint64_t db = ptx::make_smem_desc_sw128(sa + L::kABytes + half * L::kBHalfBytes);
                const uint32_t tmem_d = tmem_base + half * kHalfN;
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                    ptx::mma_bf16_2cta(tmem_d, da + 2u * k, db + 2u * k, kIdesc, (!first_kb || k != 0u) ? 1u : 0u);
            };
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                // Head of the tile: the first half of the accumulator is free before the second (the epilogue
                // drains them in that order), so the first `head` k-blocks go into half 0 alone ...
                const uint32_t head = num_kb < STAGES ? num_kb : STAGES;
                if (!(ok = wait_bounded<true>(acc_free_bar(0), free_phase ^ 1u, ctl, 2)))
                    break;
                ptx::tcgen05_fence_after();
                uint32_t st = stage, ph = phase;
                for (uint32_t kb = 0; kb < head; ++kb) {
                    if (!(ok = wait_bounded<true>(full_bar(st), ph, ctl, 2)))
                        break;
                    ptx::tcgen05_fence_after();
                    issue_half(st, 0, kb == 0);
                    if (++st == STAGES) {
                        st = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok)
                    break;
                // ... then half 1 catches up on the same stages and releases them
                if (!(ok = wait_bounded<true>(acc_free_bar(1), free_phase ^ 1u, ctl, 2)))
                    break;
                ptx::tcgen05_fence_after();
                for (uint32_t kb = 0; kb < head; ++kb) {
                    issue_half(stage, 1, kb == 0);
                    ptx::mma_commit_2cta_mask(empty_bar(stage), 3);  // stage of both CTAs is free
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                // body: both halves per k-block
                for (uint32_t kb = head; kb < num_kb; ++kb) {
                    if (!(ok = wait_bounded<true>(full_bar(stage), phase, ctl, 2)))
                        break;
                    ptx::tcgen05_fence_after();
                    issue_half(stage, 0, false);
                    issue_half(stage, 1, false);
                    ptx::mma_commit_2cta_mask(empty_bar(stage), 3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_2cta_mask(acc_full_bar, 3);  // the whole 256 x 512 accumulator is complete
                free_phase ^= 1u;
            }
            role_ok = ok;
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue --
        const uint32_t quarter = warp & 3u;
        uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        const uint32_t stage_u32 = smem_base + L::kStagingOffset + (warp - 2u) * kTmaStageWarpBytes;
        uint32_t store_buf = 0;
        uint32_t full_phase = 0;
        bool ok = true;
        for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
            const TileCoord tc = tile_coord(t, p);
            ok = wait_bounded<true>(acc_full_bar, full_phase, ctl, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            const uint32_t row0 = tc.m_blk * kPairBlockM + cta_rank * kBlockM;
#pragma unroll 1
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t col0 = tc.n_blk * kWideBlockN + h * kHalfN;
                if (p.c_tma_ok)
                    drain_accumulator_tma<kHalfN>(p, &tma_c, stage_u32, tmem_base + h * kHalfN, quarter, lane, row0, col0,
                                                  store_buf);
                else
                    drain_accumulator<kHalfN>(p, stage_warp, tmem_base + h * kHalfN, quarter, lane, row0, col0);
                // this half of the accumulator may be overwritten by the next tile
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive_cluster_addr(ptx::mapa_shared(acc_free_bar(h), 0));
            }
            full_phase ^= 1u;
        }
        if (p.c_tma_ok)
            tma_store_drain(lane);  // the staging buffers must outlive the stores that read them
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
