// Skinny-M BF16 GEMM for 32 < M <= 128 with K split across a CTA pair and the two halves added through
// distributed shared memory: the taller sibling of gemm_sm100_skinny_pair.cuh (which replicates M <= 32
// rows of A into the four TMEM quarters).  Here the 128-row A tile is loaded once per k-block (rows past M
// arrive as zeros and are never stored), epilogue warp q owns rows 32q..32q+31 of the tile over all its
// columns, and the exchange of the peer's fp32 accumulator (up to 128 x 256 x 4 B = 128 KiB) uses the
// LEADER's whole operand ring, which is free once both main loops are over.  Everything else (one pair per
// tile, tile width chosen on the host so that the pairs fill the machine in one wave, fixed summation order,
// bounded waits, programmatic dependent launch) is as in the M <= 32 kernel.
//
// In the reference's terms: the per-tile GEMM of crates/maize_tile/src/gemm/mod.rs:37-90 over a
// column panel of B (crates/maize_tile/src/gmem/col_panel.rs:88-124), its k loop cut in two.
#pragma once
#include "gemm_sm100_skinny_pair.cuh"

namespace maize {

// B_KN: B is given K x N row-major; the tile's bn columns (a multiple of 64 then) are loaded as bn / 64 boxes of
// {64 columns, 64 k-rows} and read by the MMA as an MN-major operand.
template <uint32_t STAGES, bool B_KN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_skinny_pair_tall(const __grid_constant__ CUtensorMap tma_x /* A: M x K, box 128 x 64 */,
                                 const __grid_constant__ CUtensorMap tma_w /* B: N x K, box bn x 64 */,
                                 const SkinnyPairParams p)
{
    using L = SkinnySmemLayout<STAGES>;  // stages are sized for the widest tile (256 rows of B)
    constexpr uint32_t kTmemCols = 256;  // one accumulator of up to 256 columns
    // exchange area = the LEADER's operand ring, free once both main loops are over:
    // [warp q][chunk of 32 columns][group of 4 columns][lane][4 columns] fp32 = 4 KiB per chunk, 32 KiB per warp
    constexpr uint32_t kExchangeChunkBytes = 32 * 32 * 4;
    constexpr uint32_t kExchangeWarpBytes = 8 * kExchangeChunkBytes;
    static_assert(4 * kExchangeWarpBytes <= L::kRingBytes, "exchange area must fit in the operand ring");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + b); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + L::kTmemSlotOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + L::kAbortOffset);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const uint32_t idesc = ptx::make_instr_desc_bf16(kBlockM, p.bn, B_KN);
    constexpr uint32_t kChunkBytes = kBlockK * 128;  // one 64-column chunk of a K x N tile: 64 k-rows x 128 B
    const uint32_t stage_tx = L::kXBytes + p.bn * kBlockK * 2;  // bytes one stage receives
    // this CTA's half of the k-blocks (the first half gets the odd one)
    const uint32_t kb_half = (p.num_kb + 1) / 2;
    const uint32_t kb_lo = cta_rank == 0 ? 0u : kb_half;
    const uint32_t kb_hi = cta_rank == 0 ? kb_half : p.num_kb;
    const WaitCtl ctl{abort_flag, p.g.status, p.g.timeout_ns};
    const uint32_t t = blockIdx.x >> 1;  // this pair's tile
    const bool have_tile = t < p.tiles_n;

    // Producer state: thread 0 fills the ring before the block-wide barrier, so that the first loads are in
    // flight while TMEM is being allocated.
    uint32_t pr_stage = 0, pr_phase = 0, pr_kb = kb_lo;
    uint64_t pol_stream = 0, pol_keep = 0;
    auto issue_w = [&](uint32_t kb, uint32_t stage) {  // B tile of one k-block (and the stage's byte count)
        const uint32_t sw = smem_base + stage * L::kStageBytes + L::kXBytes;
        ptx::mbar_arrive_expect_tx(full_bar(stage), stage_tx);
        if constexpr (B_KN) {
            for (uint32_t j = 0; j < p.bn / 64u; ++j)  // x = column, y = k row
                ptx::tma_load_2d_hint(sw + j * kChunkBytes, &tma_w, full_bar(stage), static_cast<int32_t>(t * p.bn + 64u * j),
                                      static_cast<int32_t>(kb * kBlockK), pol_stream);
        } else {
            ptx::tma_load_2d_hint(sw, &tma_w, full_bar(stage), static_cast<int32_t>(kb * kBlockK),
                                  static_cast<int32_t>(t * p.bn), pol_stream);
        }
    };
    auto issue_x = [&](uint32_t kb, uint32_t stage) {  // the 128-row A tile (rows past M are zero-filled)
        const uint32_t sx = smem_base + stage * L::kStageBytes;
        ptx::tma_load_2d_hint(sx, &tma_x, full_bar(stage), static_cast<int32_t>(kb * kBlockK), 0, pol_keep);
    };
    auto issue_kb = [&](uint32_t kb, uint32_t stage) {
        issue_w(kb, stage);
        issue_x(kb, stage);
    };
    const bool early_b = p.pdl != 0u && p.b_static != 0u;  // B may be fetched before the dependency wait
    uint32_t prefilled = 0;                                // stages whose B load was issued early

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tma_w);
        ptx::prefetch_tensormap(&tma_x);
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(acc_full_bar(0), 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        pol_stream = ptx::policy_evict_first();
        pol_keep = ptx::policy_evict_last();
        if (p.pdl)
            ptx::grid_dependency_launch_dependents();  // the next kernel may be scheduled as SMs free up
        if (have_tile && (early_b || !p.pdl)) {
            for (uint32_t s = 0; s < STAGES && pr_kb < kb_hi; ++s) {  // first lap: every stage is free
                if (early_b) {
                    issue_w(pr_kb++, pr_stage);  // A follows after the dependency wait
                    ++prefilled;
                } else {
                    issue_kb(pr_kb++, pr_stage);
                }
                if (++pr_stage == STAGES) {
                    pr_stage = 0;
                    pr_phase ^= 1u;
                }
            }
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc_1cta(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish_1cta();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.pdl)
        ptx::grid_dependency_wait();  // everything below may read A and write C

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0 && have_tile) {
            for (uint32_t s = 0; s < prefilled; ++s)  // the A tiles of the stages whose B was fetched early
                issue_x(kb_lo + s, s);
            while (pr_kb < kb_hi) {
                if (!wait_bounded(empty_bar(pr_stage), pr_phase ^ 1u, ctl, 1))
                    break;
                issue_kb(pr_kb++, pr_stage);
                if (++pr_stage == STAGES) {
                    pr_stage = 0;
                    pr_phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer --
        if (lane == 0 && have_tile) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
                if (!(ok = wait_bounded(full_bar(stage), phase, ctl, 2)))
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t sx = smem_base + stage * L::kStageBytes;
                const uint64_t dx = ptx::make_smem_desc_sw128(sx);               // A tile: the MMA's M side
                const uint64_t dw = B_KN ? ptx::make_smem_desc_sw128_mn(sx + L::kXBytes, kChunkBytes)
                                         : ptx::make_smem_desc_sw128(sx + L::kXBytes);  // B tile: its N side
                constexpr uint32_t kStepW = B_KN ? 128u : 2u;  // +2048 B or +32 B per 16-wide K step
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                    ptx::mma_bf16_1cta(tmem_base, dx + 2u * k, dw + kStepW * k, idesc, (kb != kb_lo || k != 0u) ? 1u : 0u);
                ptx::mma_commit_1cta(empty_bar(stage));
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok)
                ptx::mma_commit_1cta(acc_full_bar(0));  // this half of K is in TMEM
        }
        __syncwarp();
    }

    // ------------------------------------------- epilogue (warps 2-5) and pair barriers (everyone) --
    // ALL threads of both CTAs pass two cluster barriers (they are .aligned: whole warps, no early exit):
    //   B1: both halves are complete (every epilogue warp has seen its CTA's accumulator) -> the leader's
    //       operand ring is no longer read by any MMA and may serve as the exchange area;
    //   B2: the peer's accumulator has been written there -> the leader may read it.
    const uint32_t quarter = warp & 3u;
    uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp >= 2u ? (warp - 2u) : 0u) * kStageWarpBytes;
    const bool have_k = kb_hi > kb_lo;  // false only for the peer when there is a single k-block
    const uint32_t exch_off = quarter * kExchangeWarpBytes;
    const uint32_t chunks = p.bn / 32u;
    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
    bool ok = true;
    if (warp >= 2u && have_tile && have_k) {
        ok = wait_bounded(acc_full_bar(0), 0, ctl, 3);
        ok = __all_sync(0xffffffffu, ok);
        ptx::tcgen05_fence_after();
    }
    ptx::cluster_arrive();  // B1
    ptx::cluster_wait();
    if (warp >= 2u && have_tile && ok && cta_rank == 1u) {
        const uint32_t remote = ptx::mapa_shared(smem_base + exch_off, 0);
#pragma unroll 1
        for (uint32_t c = 0; c < chunks; ++c) {
            uint32_t v[32];
            if (have_k) {
                ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                ptx::tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    v[j] = 0u;
            }
#pragma unroll
            for (uint32_t j = 0; j < 32; j += 4)
                st_shared_cluster_v4(remote + c * kExchangeChunkBytes + ((j / 4) * 32u + lane) * 16u, __uint_as_float(v[j]),
                                     __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        }
    }
    ptx::cluster_arrive();  // B2 (release / acquire at cluster scope orders the stores above)
    ptx::cluster_wait();
    if (warp >= 2u && have_tile && ok && cta_rank == 0u) {
        const uint8_t *mine = smem_gen + exch_off;
#pragma unroll 1
        for (uint32_t c = 0; c < chunks; ++c) {
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (uint32_t j = 0; j < 32; j += 4) {
                const float4 q4 = *reinterpret_cast<const float4 *>(mine + c * kExchangeChunkBytes + ((j / 4) * 32u + lane) * 16u);
                // fixed order: first half of K (this CTA) + second half (the peer)
                v[j] = __float_as_uint(__uint_as_float(v[j]) + q4.x);
                v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + q4.y);
                v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + q4.z);
                v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + q4.w);
            }
            store_chunk(p.g, stage_warp, quarter * 32u, t * p.bn + c * 32u, lane, v);
        }
    }

    // ---------------------------------------------------------------- teardown --
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            for (int i = 0; i < 256; ++i)
                __nanosleep(1000);
        }
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc_1cta(tmem_base, kTmemCols);
    }
}

}  // namespace maize
