// CTA-pair GEMM (see gemm_sm100_2cta.cuh for the roles, barriers and teardown, which are the same
// here) whose LAST, partial round of tiles is split along K.
//
// With P pairs and T tiles the plain persistent schedule runs ceil(T / P) rounds, and the last round keeps only
// T mod P pairs busy (4096^3: 256 tiles on 74 pairs = 3 full rounds and a fourth with 34 tiles).  Here
// the `tail` = T mod P tiles of that round are cut into `split` ranges of k-steps each, one (tile, range) unit per
// pair, so that the round takes 1 / split of a tile's time plus the exchange:
//
//   rounds 0 .. full_rounds-1 : pair p computes tile r * P + p over all of K, as before;
//   last round                : pair p < tail * split computes k-steps
//                               [part * steps / split, (part + 1) * steps / split) of tile full_rounds * P + p / split,
//                               part = p % split.
//
// The parts of a tile are combined without any wait: every epilogue warp publishes its 32 x 256 fp32 partial in
// a scratch slot and bumps a counter; the warp that arrives last keeps its own partial in registers and adds all
// parts IN PART ORDER (so the result does not depend on which one was last), converts and stores C.  Counters
// return to zero for the next launch.  A pair's CTA r only ever exchanges with CTA r of the other pairs (same rows).
#pragma once
#include "gemm_sm100_2cta.cuh"

namespace maize {

struct TailParams {
    GemmParams g;
    uint32_t full_rounds;    // rounds in which every pair computes one whole tile
    uint32_t tail_tiles;     // tiles of the last round (0: there is none)
    uint32_t split;          // k-ranges per tile of the last round (1: it is an ordinary round)
    float *partials;         // [tail_tiles][split][2 CTAs] slots of 128 x 256 fp32
    unsigned int *counters;  // [tail_tiles][2 CTAs][4 quarters], zero between launches
};

constexpr uint32_t kTailSlotFloats = kBlockM * 256u;

struct TailWork {
    uint32_t tile;
    uint32_t step_lo, step_hi;
    uint32_t part, parts;
    uint32_t tail_index;
};

// The i-th piece of work of a pair; false when there is none.
__device__ __forceinline__ bool tail_work(const TailParams &p, uint32_t pair, uint32_t num_pairs, uint32_t num_steps,
                                          uint32_t i, TailWork &w)
{
    if (i < p.full_rounds) {
        w.tile = i * num_pairs + pair;
        w.step_lo = 0;
        w.step_hi = num_steps;
        w.part = 0;
        w.parts = 1;
        w.tail_index = 0;
        return true;
    }
    if (i > p.full_rounds || pair >= p.tail_tiles * p.split)
        return false;
    w.tail_index = pair / p.split;
    w.part = pair - w.tail_index * p.split;
    w.parts = p.split;
    w.tile = p.full_rounds * num_pairs + w.tail_index;
    w.step_lo = static_cast<uint32_t>(static_cast<uint64_t>(w.part) * num_steps / p.split);
    w.step_hi = static_cast<uint32_t>(static_cast<uint64_t>(w.part + 1u) * num_steps / p.split);
    return true;
}

__device__ __forceinline__ unsigned int tail_ld_acquire_gpu(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <uint32_t KBS, uint32_t STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_2cta_tail(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                          const __grid_constant__ CUtensorMap tma_c, const TailParams tp)
{
    constexpr uint32_t BN = 256;
    using L = PairSmemLayout<BN, KBS, STAGES>;
    constexpr uint32_t kTmemCols = 2 * BN;
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kPairBlockM, BN, false);
    constexpr uint32_t kStepK = KBS * kBlockK;
    const GemmParams &p = tp.g;

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
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    const uint32_t num_steps = (p.k + kStepK - 1) / kStepK;
    const WaitCtl ctl{abort_flag, p.status, p.timeout_ns};

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
            ptx::mbar_init(acc_empty_bar(b), 2 * kNumEpilogueWarps);
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
            const uint64_t pol = ptx::policy_evict_normal();
            int32_t gate_seen = 0;
            TailWork w;
            for (uint32_t i = 0; ok && tail_work(tp, pair, num_pairs, num_steps, i, w); ++i) {
                const TileCoord tc = tile_coord(w.tile, p);
                const int32_t m0 = static_cast<int32_t>(tc.m_blk * kPairBlockM + cta_rank * kBlockM);
                const int32_t n0 = static_cast<int32_t>(tc.n_blk * BN + cta_rank * (BN / 2));
                if (!(ok = gate_rows_landed(p, static_cast<uint32_t>(m0) + kBlockM, gate_seen, ctl)))
                    break;
                for (uint32_t step = w.step_lo; step < w.step_hi; ++step) {
                    ok = wait_bounded<true>(empty_bar(stage), phase ^ 1u, ctl, 1);
                    if (!ok)
                        break;
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + KBS * L::kABytes;
                    const uint32_t leader_full = ptx::mapa_shared(full_bar(stage), 0);
                    if (cta_rank == 0)
                        ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
#pragma unroll
                    for (uint32_t sub = 0; sub < KBS; ++sub) {
                        const int32_t kx = static_cast<int32_t>((step * KBS + sub) * kBlockK);
                        ptx::tma_load_2d_pair_hint(sa + sub * L::kABytes, &tma_a, leader_full, kx, m0, pol);
                        ptx::tma_load_2d_pair_hint(sb + sub * L::kBBytes, &tma_b, leader_full, kx, n0, pol);
                    }
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
            uint32_t stage = 0, phase = 0;
            uint32_t acc = 0, acc_phase = 0;
            bool ok = true;
            TailWork w;
            for (uint32_t i = 0; ok && tail_work(tp, pair, num_pairs, num_steps, i, w); ++i) {
                ok = wait_bounded<true>(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2);
                if (!ok)
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t step = w.step_lo; step < w.step_hi; ++step) {
                    ok = wait_bounded<true>(full_bar(stage), phase, ctl, 2);
                    if (!ok)
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * L::kStageBytes;
                    const uint32_t sb = sa + KBS * L::kABytes;
#pragma unroll
                    for (uint32_t sub = 0; sub < KBS; ++sub) {
                        const uint64_t da = ptx::make_smem_desc_sw128(sa + sub * L::kABytes);
                        const uint64_t db = ptx::make_smem_desc_sw128(sb + sub * L::kBBytes);
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                            ptx::mma_bf16_2cta(tmem_d, da + 2u * k, db + 2u * k, kIdesc,
                                               (step != w.step_lo || (sub | k) != 0u) ? 1u : 0u);
                    }
                    ptx::mma_commit_2cta_mask(empty_bar(stage), 3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_2cta_mask(acc_full_bar(acc), 3);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
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
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        TailWork w;
        for (uint32_t i = 0; ok && tail_work(tp, pair, num_pairs, num_steps, i, w); ++i) {
            const TileCoord tc = tile_coord(w.tile, p);
            ok = wait_bounded<true>(acc_full_bar(acc), acc_phase, ctl, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            const uint32_t tile_row0 = tc.m_blk * kPairBlockM + cta_rank * kBlockM;
            const uint32_t tile_col0 = tc.n_blk * BN;
            if (w.parts == 1 && p.c_tma_ok) {
                drain_accumulator_tma<BN>(p, &tma_c, stage_u32, tmem_base + acc * BN, quarter, lane, tile_row0, tile_col0,
                                          store_buf);
            } else if (w.parts == 1) {
                drain_accumulator<BN>(p, stage_warp, tmem_base + acc * BN, quarter, lane, tile_row0, tile_col0);
            } else {
                if (p.c_tma_ok)
                    tma_store_drain(lane);  // the combining path below re-uses the staging area
                // slot of (tile of the last round, part, this CTA's half): [column][row] so that a warp's 32 lanes
                // (= rows) touch 32 consecutive floats
                const uint32_t taddr = tmem_base + acc * BN + ((quarter * 32u) << 16);
                const uint32_t slot_row = quarter * 32u + lane;
                float *tile_slots = tp.partials + (static_cast<size_t>(w.tail_index) * w.parts * 2u) * kTailSlotFloats;
                auto slot_of = [&](uint32_t part) {
                    return tile_slots + (static_cast<size_t>(part) * 2u + cta_rank) * kTailSlotFloats;
                };
                unsigned int *counter = tp.counters + (w.tail_index * 2u + cta_rank) * 4u + quarter;
                // publish this warp's 32 x 256 partial, then learn whether it was the last of the tile's parts
                float *mine = slot_of(w.part);
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j)
                        __stcg(mine + (c * 32u + j) * kBlockM + slot_row, __uint_as_float(v[j]));
                }
                __threadfence();
                __syncwarp();
                unsigned int seen = 0;
                if (lane == 0)
                    seen = atomicAdd(counter, 1u);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen + 1u == w.parts) {
                    if (lane == 0)
                        *counter = 0u;  // ready for the next launch
                    __threadfence();    // every lane orders its reads of the parts after the counter update
#pragma unroll 1
                    for (uint32_t c = 0; c < BN / 32; ++c) {
                        // own part from TMEM, the others from their slots, added in part order
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                        ptx::tmem_ld_wait();
                        float s[32];
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            s[j] = 0.0f;
                        for (uint32_t part = 0; part < w.parts; ++part) {
                            if (part == w.part) {
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    s[j] += __uint_as_float(v[j]);
                            } else {
                                const float *src = slot_of(part) + (c * 32u) * kBlockM + slot_row;
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    s[j] += __ldcg(src + j * kBlockM);
                            }
                        }
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            v[j] = __float_as_uint(s[j]);
                        store_chunk(p, stage_warp, tile_row0 + quarter * 32u, tile_col0 + c * 32u, lane, v);
                    }
                }
            }
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
        role_ok = ok;
    }
    if (!role_ok) {
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
