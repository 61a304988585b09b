// Skinny-M BF16 GEMM (M <= 32) with K split across a CTA pair and the two halves added through
// distributed shared memory.
//
// The stream-K kernel of gemm_sm100_skinny.cuh balances any N over the SMs, but CTAs that share a
// tile exchange their partial sums through global memory and a counter, and since they all finish
// together that exchange (store, fence, atomic, load: ~4 us of dependent latency) sits at the end
// of the kernel.  Here the two CTAs of a cluster own one tile: CTA r runs the k-blocks of half r
// into its own TMEM accumulator with ordinary one-CTA MMAs, then CTA 1 writes its fp32 accumulator
// straight into CTA 0's shared memory (st.shared::cluster), a cluster barrier publishes it, and
// CTA 0 adds its own half in a fixed order (reproducible), rounds once to bf16 and stores.  No
// global scratch, no counters, about 1.5 us of tail.
//
// The tile width BN (multiple of 32, up to 256) is chosen on the host so that the tile pairs fill
// the machine: N = 16384 on 148 SMs gives BN = 224, 74 tiles, one pair each.  BN is a run-time
// value: it enters the MMA through the instruction descriptor and the loads through B's tensor map.
// A pair computes exactly ONE tile (the host launches one pair per tile and uses this kernel only
// when the tiles fit in one wave); shapes with more tiles go to the stream-K kernel.
//
// As in the stream-K kernel, B is the N side of the MMA and the M <= 32 rows of A are replicated
// into the four 32-row quarters of the A tile, so that warp q of the epilogue finds rows 0..31 of C
// in its own TMEM quarter and handles columns [64q, 64q + 64) of the tile.
//
// In the reference's terms: the per-tile GEMM of crates/maize_tile/src/gemm/mod.rs:37-90 over a
// column panel of B (crates/maize_tile/src/gmem/col_panel.rs:88-124), its k loop cut in two.
#pragma once
#include "gemm_sm100_skinny.cuh"

namespace maize {

struct SkinnyPairParams {
    GemmParams g;      // c, ldc, m, n, k, c_vec_ok, status, timeout_ns (tile fields unused)
    uint32_t bn;       // tile width: rows of B per tile, multiple of 32, 32..256
    uint32_t tiles_n;  // ceil(N / bn)
    uint32_t num_kb;   // ceil(K / 64)
    // Launched with programmatic stream serialization: the kernel may start before the previous kernel of the
    // stream has finished and orders itself with griddepcontrol.wait.  With b_static (the caller guarantees
    // that no earlier work of the stream writes B, e.g. inference weights) the first lap of B loads is issued
    // BEFORE that wait, so the weights stream in while the previous kernel drains.
    uint32_t pdl;
    uint32_t b_static;
};

__device__ __forceinline__ void st_shared_cluster_v4(uint32_t cluster_addr, float a, float b, float c, float d)
{
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c),
                 "f"(d)
                 : "memory");
}

// B_KN: B is given K x N row-major; the tile's bn columns (a multiple of 64 then) are loaded as bn / 64 boxes of
// {64 columns, 64 k-rows} and read by the MMA as an MN-major operand.
template <uint32_t STAGES, bool B_KN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_skinny_pair(const __grid_constant__ CUtensorMap tma_x /* A: M x K, box 32 x 64 */,
                            const __grid_constant__ CUtensorMap tma_w /* B: N x K, box bn x 64 */,
                            const SkinnyPairParams p)
{
    using L = SkinnySmemLayout<STAGES>;  // stages are sized for the widest tile (256 rows of B)
    constexpr uint32_t kTmemCols = 256;  // one accumulator of up to 256 columns
    // exchange area = the first ring stage of the LEADER, free once both main loops are over:
    // [warp q][column 0..63][lane 0..31] fp32 = 8 KiB per warp
    constexpr uint32_t kExchangeWarpBytes = 64 * 32 * 4;
    static_assert(4 * kExchangeWarpBytes <= L::kStageBytes, "exchange area must fit in one ring stage");

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
    auto issue_x = [&](uint32_t kb, uint32_t stage) {  // the same 32 rows of A into each quarter of the A tile
        const uint32_t sx = smem_base + stage * L::kStageBytes;
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q)
            ptx::tma_load_2d_hint(sx + q * (L::kXBytes / 4), &tma_x, full_bar(stage),
                                  static_cast<int32_t>(kb * kBlockK), 0, pol_keep);
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
    //       first ring stage is no longer read by any MMA and may serve as the exchange area;
    //   B2: the peer's accumulator has been written there -> the leader may read it.
    const uint32_t quarter = warp & 3u;
    uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp >= 2u ? (warp - 2u) : 0u) * kStageWarpBytes;
    const bool have_k = kb_hi > kb_lo;  // false only for the peer when there is a single k-block
    const uint32_t exch_off = quarter * kExchangeWarpBytes;  // inside ring stage 0
    uint32_t v0[32], v1[32];
    bool ok = true;
    if (warp >= 2u && have_tile) {
        if (have_k) {
            ok = wait_bounded(acc_full_bar(0), 0, ctl, 3);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && have_k) {
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + quarter * 64u;
            if (quarter * 64u < p.bn) {
                ptx::tmem_ld_32x32b_x32(taddr, v0);
                if (quarter * 64u + 32u < p.bn)
                    ptx::tmem_ld_32x32b_x32(taddr + 32u, v1);
                ptx::tmem_ld_wait();
            }
        }
        if (!have_k) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                v0[j] = v1[j] = 0u;
        }
    }
    ptx::cluster_arrive();  // B1
    ptx::cluster_wait();
    if (warp >= 2u && have_tile && ok && cta_rank == 1u && quarter * 64u < p.bn) {
        // write this warp's 64 columns x 32 rows into the leader's exchange area, laid out as
        // [group of 4 columns][lane][4 columns]: 16 bytes per lane per group, consecutive across the warp
        const uint32_t remote = ptx::mapa_shared(smem_base + exch_off, 0);
#pragma unroll
        for (uint32_t j = 0; j < 32; j += 4) {
            const uint32_t a0 = remote + ((j / 4) * 32u + lane) * 16u;
            st_shared_cluster_v4(a0, __uint_as_float(v0[j]), __uint_as_float(v0[j + 1]), __uint_as_float(v0[j + 2]),
                                 __uint_as_float(v0[j + 3]));
            const uint32_t a1 = remote + ((8u + j / 4) * 32u + lane) * 16u;
            st_shared_cluster_v4(a1, __uint_as_float(v1[j]), __uint_as_float(v1[j + 1]), __uint_as_float(v1[j + 2]),
                                 __uint_as_float(v1[j + 3]));
        }
    }
    ptx::cluster_arrive();  // B2 (release / acquire at cluster scope orders the stores above)
    ptx::cluster_wait();
    if (warp >= 2u && have_tile && ok && cta_rank == 0u && quarter * 64u < p.bn) {
        const uint8_t *mine = smem_gen + exch_off;
#pragma unroll
        for (uint32_t j = 0; j < 32; j += 4) {
            const float4 p0 = *reinterpret_cast<const float4 *>(mine + ((j / 4) * 32u + lane) * 16u);
            const float4 p1 = *reinterpret_cast<const float4 *>(mine + ((8u + j / 4) * 32u + lane) * 16u);
            // fixed order: first half of K (this CTA) + second half (the peer)
            v0[j] = __float_as_uint(__uint_as_float(v0[j]) + p0.x);
            v0[j + 1] = __float_as_uint(__uint_as_float(v0[j + 1]) + p0.y);
            v0[j + 2] = __float_as_uint(__uint_as_float(v0[j + 2]) + p0.z);
            v0[j + 3] = __float_as_uint(__uint_as_float(v0[j + 3]) + p0.w);
            v1[j] = __float_as_uint(__uint_as_float(v1[j]) + p1.x);
            v1[j + 1] = __float_as_uint(__uint_as_float(v1[j + 1]) + p1.y);
            v1[j + 2] = __float_as_uint(__uint_as_float(v1[j + 2]) + p1.z);
            v1[j + 3] = __float_as_uint(__uint_as_float(v1[j + 3]) + p1.w);
        }
        const uint32_t col0 = t * p.bn + quarter * 64u;
        store_chunk(p.g, stage_warp, 0u, col0, lane, v0);
        if (quarter * 64u + 32u < p.bn)
            store_chunk(p.g, stage_warp, 0u, col0 + 32u, lane, v1);
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
