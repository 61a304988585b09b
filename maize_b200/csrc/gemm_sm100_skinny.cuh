// Skinny-M ("decode") BF16 GEMM for sm_100a: C[M x N] = A[M x K] * B[N x K]^T with M <= 128.
//
// The shape is bound by streaming B (the weights) from HBM once, so the kernel is
// built around that stream:
//
//   - B is the N side of the MMA, 256 rows per tile: a tcgen05.mma with M = 128 takes
//     about 130 cycles whatever its N (its M-side operand streams one row per cycle),
//     so N = 256 moves 8 KiB of weights per MMA where a swapped layout with the weights
//     on the M side would move 4 KiB and leave the kernel bound by the tensor pipe;
//   - A is the M side.  With M <= 32 (REPL) its rows are loaded four times, into rows
//     0-31, 32-63, 64-95 and 96-127 of the shared-memory tile, so that every 32-lane
//     quarter of TMEM holds the same M rows of C and each of the four epilogue warps
//     (which can only read its own quarter) drains a 64-column quarter of the tile.
//     With 32 < M <= 128 the tile is loaded once and warp q drains rows 32q..32q+31;
//     rows past M are zero-filled by TMA and never stored;
//   - work is cut into units of one (256-row B tile, 64-wide k-block) = 32 KiB of B,
//     laid out tile-major, and dealt to the CTAs in equal contiguous ranges
//     (stream-K), so every SM streams the same number of bytes whatever N is;
//   - a CTA whose range covers only part of a tile's K writes its fp32 partial to a
//     scratch slot [tile][part]; the LAST warp to arrive for a (tile, quarter) adds
//     the parts in part order (reproducible), rounds once to bf16 and stores.  Arrival
//     is a global counter per (tile, quarter) that the last warp resets, so no CTA
//     ever waits for another CTA;
//   - a CTA works on the piece it shares with the NEXT CTA first and on the piece it
//     shares with the PREVIOUS CTA afterwards, so the partner's partial is normally
//     published long before a CTA's last piece is done: that piece then finds the
//     counter complete, adds the published parts to its registers and stores, without
//     publishing anything itself (if the partner is late, the ordinary protocol runs);
//   - the producer fills the ring before the block-wide set-up barrier, so the first
//     loads are in flight while TMEM is being allocated; B is loaded with an
//     evict-first L2 hint (read once), A with evict-last (re-read by every CTA).
//
// In the reference's terms this is still the per-tile GEMM of
// crates/maize_tile/src/gemm/mod.rs:37-90 driven over column panels of B
// (crates/maize_tile/src/gmem/col_panel.rs:88-124), with the k loop of one panel
// shared between CTAs.  Roles, bounded waits and teardown follow gemm_sm100.cuh.
#pragma once
#include "gemm_common.cuh"

namespace maize {

constexpr uint32_t kSkinnyTileN = 256;  // rows of B per tile = accumulator columns

template <uint32_t STAGES>
struct SkinnySmemLayout {
    static constexpr uint32_t kXBytes = kBlockM * kBlockK * 2;       // A tile, 128 rows (16 KiB)
    static constexpr uint32_t kWBytes = kSkinnyTileN * kBlockK * 2;  // B tile, 256 rows (32 KiB)
    static constexpr uint32_t kStageBytes = kXBytes + kWBytes;
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    static constexpr uint32_t kStagingOffset = kRingBytes;
    static constexpr uint32_t kBarOffset = kStagingOffset + kStageBytesTotal;
    static constexpr uint32_t kNumBars = 2 * STAGES + 4;
    static constexpr uint32_t kTmemSlotOffset = kBarOffset + kNumBars * 8;
    static constexpr uint32_t kAbortOffset = kTmemSlotOffset + 4;
    static constexpr uint32_t kUsedBytes = kAbortOffset + 4;
    static constexpr uint32_t kDynamicBytes = kUsedBytes + 1024;
    static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned for the 128B swizzle");
    static_assert(kDynamicBytes <= 232448, "exceeds 227 KiB of shared memory per CTA");
    static_assert(kDynamicBytes > 116224, "two CTAs could share an SM and contend for TMEM");
};

struct SkinnyParams {
    GemmParams g;            // c, ldc, m, n, k, c_vec_ok, status, timeout_ns, debug_flags (tile fields unused)
    uint32_t tiles_n;        // ceil(N / 256)
    uint32_t num_kb;         // ceil(K / 64)
    uint32_t units_per_cta;  // Q: CTA i owns units [i*Q, min((i+1)*Q, tiles_n*num_kb))
    uint32_t max_parts;      // scratch slots per tile
    float *partials;         // [tiles_n][max_parts][256 columns][ROWS] fp32, ROWS = 32 (REPL) or 128
    unsigned int *counters;  // [tiles_n][4], zero between launches
};

// One contiguous run of k-blocks of one tile inside a CTA's unit range.
struct SkinnySegment {
    uint32_t tile, kb_lo, kb_hi;  // [kb_lo, kb_hi)
    uint32_t part, parts;         // this CTA's slot and the number of CTAs sharing the tile
};

__device__ __forceinline__ SkinnySegment skinny_segment(uint32_t u, uint32_t u_end, uint32_t num_kb, uint32_t q)
{
    SkinnySegment s;
    s.tile = u / num_kb;
    const uint32_t tile_u0 = s.tile * num_kb;
    s.kb_lo = u - tile_u0;
    s.kb_hi = min(u_end, tile_u0 + num_kb) - tile_u0;
    const uint32_t first_cta = tile_u0 / q;
    const uint32_t last_cta = (tile_u0 + num_kb - 1) / q;
    s.part = u / q - first_cta;
    s.parts = last_cta - first_cta + 1;
    return s;
}

// Processing order of a CTA's unit range [u_begin, u_end): if the range ends inside a tile and
// holds more than that piece, the piece goes first ([split, u_end)), the rest after ([u_begin, split)).
struct SkinnyOrder {
    uint32_t lo0, hi0, lo1, hi1;
    __device__ __forceinline__ uint32_t lo(uint32_t r) const { return r == 0 ? lo0 : lo1; }
    __device__ __forceinline__ uint32_t hi(uint32_t r) const { return r == 0 ? hi0 : hi1; }
};

__device__ __forceinline__ SkinnyOrder skinny_order(uint32_t u_begin, uint32_t u_end, uint32_t num_kb)
{
    SkinnyOrder o;
    uint32_t split = u_begin;
    if (u_end > u_begin && u_end % num_kb != 0u) {
        const uint32_t last_tile_u0 = (u_end / num_kb) * num_kb;
        if (last_tile_u0 > u_begin)
            split = last_tile_u0;
    }
    if (split > u_begin) {
        o.lo0 = split;
        o.hi0 = u_end;
        o.lo1 = u_begin;
        o.hi1 = split;
    } else {
        o.lo0 = u_begin;
        o.hi0 = u_end;
        o.lo1 = o.hi1 = u_end;
    }
    return o;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// REPL: M <= 32, A replicated into the four TMEM quarters (tma_x box = 32 rows);
// otherwise M <= 128 and tma_x box = 128 rows.
template <bool REPL, uint32_t STAGES>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_skinny(const __grid_constant__ CUtensorMap tma_x /* A: M x K */,
                       const __grid_constant__ CUtensorMap tma_w /* B: N x K, box 256 x 64 */, const SkinnyParams p)
{
    using L = SkinnySmemLayout<STAGES>;
    constexpr uint32_t BN = kSkinnyTileN;
    constexpr uint32_t kTmemCols = 2 * BN;
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kBlockM, BN);
    constexpr uint32_t kRows = REPL ? 32u : 128u;          // rows of a scratch slot
    constexpr uint32_t kColsPerWarp = REPL ? BN / 4 : BN;  // columns one epilogue warp drains
    constexpr uint32_t kSlotFloats = BN * kRows;

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
    const uint32_t total_units = p.tiles_n * p.num_kb;
    const uint32_t u_begin = min(total_units, blockIdx.x * p.units_per_cta);
    const uint32_t u_end = min(total_units, u_begin + p.units_per_cta);
    const WaitCtl ctl{abort_flag, p.g.status, p.g.timeout_ns};
    const SkinnyOrder order = skinny_order(u_begin, u_end, p.num_kb);

    // Producer state; thread 0 starts the ring before the block-wide barrier.
    uint32_t pr_stage = 0, pr_phase = 0, pr_range = 0, pr_u = order.lo0;
    uint64_t pol_stream = 0, pol_keep = 0;
    auto issue_unit = [&](uint32_t u, uint32_t stage) {
        const uint32_t tile_real = u / p.num_kb;
        const uint32_t kb = u - tile_real * p.num_kb;
        const uint32_t tile = (p.g.debug_flags & 1u) ? 0u : tile_real;
        const uint32_t sx = smem_base + stage * L::kStageBytes;
        const uint32_t sw = sx + L::kXBytes;
        if (p.g.debug_flags & 2u) {
            ptx::mbar_arrive(full_bar(stage));
            return;
        }
        const int32_t kx = static_cast<int32_t>(kb * kBlockK);
        ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
        ptx::tma_load_2d_hint(sw, &tma_w, full_bar(stage), kx, static_cast<int32_t>(tile * BN), pol_stream);
        if (REPL) {
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q)  // the same 32 rows of A into each quarter of the tile
                ptx::tma_load_2d_hint(sx + q * (L::kXBytes / 4), &tma_x, full_bar(stage), kx, 0, pol_keep);
        } else {
            ptx::tma_load_2d_hint(sx, &tma_x, full_bar(stage), kx, 0, pol_keep);
        }
    };
    // next unit in processing order; false when the CTA's range is exhausted
    auto next_unit = [&]() {
        while (pr_range < 2 && pr_u >= order.hi(pr_range)) {
            ++pr_range;
            if (pr_range < 2)
                pr_u = order.lo(pr_range);
        }
        return pr_range < 2;
    };

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tma_w);
        ptx::prefetch_tensormap(&tma_x);
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
        // first lap of the ring: every stage is free, no wait needed
        pol_stream = ptx::policy_evict_first();
        pol_keep = ptx::policy_evict_last();
        for (uint32_t s = 0; s < STAGES && next_unit(); ++s) {
            issue_unit(pr_u, pr_stage);
            ++pr_u;
            if (++pr_stage == STAGES) {
                pr_stage = 0;
                pr_phase ^= 1u;
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

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer --
        if (lane == 0) {
            while (next_unit()) {
                if (!wait_bounded(empty_bar(pr_stage), pr_phase ^ 1u, ctl, 1))
                    break;
                issue_unit(pr_u, pr_stage);
                ++pr_u;
                if (++pr_stage == STAGES) {
                    pr_stage = 0;
                    pr_phase ^= 1u;
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
            for (uint32_t r = 0; r < 2; ++r)
                for (uint32_t u = order.lo(r); ok && u < order.hi(r);) {
                    const SkinnySegment seg = skinny_segment(u, order.hi(r), p.num_kb, p.units_per_cta);
                    if (!(ok = wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2)))
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t tmem_d = tmem_base + acc * BN;
                    for (uint32_t kb = seg.kb_lo; kb < seg.kb_hi; ++kb) {
                        if (!(ok = wait_bounded(full_bar(stage), phase, ctl, 2)))
                            break;
                        ptx::tcgen05_fence_after();
                        const uint32_t sx = smem_base + stage * L::kStageBytes;
                        const uint64_t dx = ptx::make_smem_desc_sw128(sx);               // A tile: the MMA's M side
                        const uint64_t dw = ptx::make_smem_desc_sw128(sx + L::kXBytes);  // B tile: its N side
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                            ptx::mma_bf16_1cta(tmem_d, dx + 2u * k, dw + 2u * k, kIdesc,
                                               (kb != seg.kb_lo || k != 0u) ? 1u : 0u);
                        ptx::mma_commit_1cta(empty_bar(stage));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    if (!ok)
                        break;
                    ptx::mma_commit_1cta(acc_full_bar(acc));
                    if (++acc == 2) {
                        acc = 0;
                        acc_phase ^= 1u;
                    }
                    u += seg.kb_hi - seg.kb_lo;
                }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue --
        const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
        uint8_t *stage_warp = smem_gen + L::kStagingOffset + (warp - 2u) * kStageWarpBytes;
        // REPL: every quarter holds rows 0..31 of C, this warp takes columns [64q, 64q+64);
        // otherwise this warp takes rows 32q..32q+31 and all 256 columns.
        const uint32_t row0 = REPL ? 0u : quarter * 32u;
        const uint32_t col_first = REPL ? quarter * kColsPerWarp : 0u;
        const uint32_t slot_row = REPL ? lane : quarter * 32u + lane;
        const bool rows_live = row0 < p.g.m;  // warp-uniform: does this warp hold any row of C at all?
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t r = 0; r < 2; ++r)
            for (uint32_t u = order.lo(r); ok && u < order.hi(r);) {
                const SkinnySegment seg = skinny_segment(u, order.hi(r), p.num_kb, p.units_per_cta);
                const bool whole = seg.parts == 1;
                unsigned int *counter = p.counters + seg.tile * 4u + quarter;
                float *tile_parts = p.partials + static_cast<size_t>(seg.tile) * p.max_parts * kSlotFloats;

                // This CTA holds the LAST part of the tile (always true of the piece it works on last): if
                // every earlier part is already published, add them up in part order NOW, while the main
                // loop of this piece is still running, so that the tail is only TMEM load + add + store.
                bool prefetched = false;
                float pre[REPL ? kColsPerWarp : 1];
                if (REPL && rows_live && !whole && seg.part + 1u == seg.parts) {
                    unsigned int seen = 0;
                    if (lane == 0)
                        seen = ld_acquire_gpu(counter);
                    seen = __shfl_sync(0xffffffffu, seen, 0);
                    if (seen + 1u == seg.parts) {
                        __threadfence();  // every lane orders its reads of the parts after the counter read
                        prefetched = true;
#pragma unroll
                        for (uint32_t j = 0; j < kColsPerWarp; ++j)
                            pre[j] = 0.0f;
                        for (uint32_t part = 0; part + 1u < seg.parts; ++part) {
                            const float *src =
                                tile_parts + static_cast<size_t>(part) * kSlotFloats + col_first * kRows + slot_row;
#pragma unroll
                            for (uint32_t j = 0; j < kColsPerWarp; ++j)
                                pre[j] += __ldcg(src + j * kRows);
                        }
                    }
                }

                ok = wait_bounded(acc_full_bar(acc), acc_phase, ctl, 3);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * BN + col_first;
                const uint32_t tile_col0 = seg.tile * BN + col_first;

                if (rows_live && prefetched) {
                    if (lane == 0)
                        *counter = 0u;  // ready for the next launch
#pragma unroll
                    for (uint32_t c = 0; c < kColsPerWarp / 32; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            v[j] = __float_as_uint(pre[REPL ? c * 32u + j : 0] + __uint_as_float(v[j]));
                        store_chunk(p.g, stage_warp, row0, tile_col0 + c * 32u, lane, v);
                    }
                } else if (rows_live) {
                    bool last = whole;
                    bool own_in_regs = whole;  // this warp's own part comes from TMEM, not from the scratch
                    if (!whole) {
                        // have all the other parts been published already?  Then ours needs no publishing.
                        unsigned int seen = 0;
                        if (lane == 0)
                            seen = ld_acquire_gpu(counter);
                        seen = __shfl_sync(0xffffffffu, seen, 0);
                        if (seen + 1u == seg.parts) {
                            last = true;
                            own_in_regs = true;
                            if (lane == 0)
                                *counter = 0u;  // ready for the next launch
                            __threadfence();    // every lane orders its reads of the parts after the counter read
                        }
                    }
                    if (!last) {
                        // publish this CTA's partial, then find out whether this warp is the last to arrive
                        float *slot = tile_parts + static_cast<size_t>(seg.part) * kSlotFloats;
#pragma unroll 1
                        for (uint32_t c = 0; c < kColsPerWarp / 32; ++c) {
                            uint32_t v[32];
                            ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (uint32_t j = 0; j < 32; ++j)
                                __stcg(slot + (col_first + c * 32u + j) * kRows + slot_row, __uint_as_float(v[j]));
                        }
                        __threadfence();
                        __syncwarp();
                        unsigned int seen = 0;
                        if (lane == 0)
                            seen = atomicAdd(counter, 1u);
                        seen = __shfl_sync(0xffffffffu, seen, 0);
                        last = seen + 1u == seg.parts;
                        if (last) {
                            if (lane == 0)
                                *counter = 0u;  // ready for the next launch
                            __threadfence();
                        }
                    }
                    if (last) {
#pragma unroll 1
                        for (uint32_t c = 0; c < kColsPerWarp / 32; ++c) {
                            // parts are added in part order whoever finishes last, so the result is reproducible
                            uint32_t sum[32];
                            float own[32];
                            if (own_in_regs) {
                                uint32_t v[32];
                                ptx::tmem_ld_32x32b_x32(taddr + c * 32u, v);
                                ptx::tmem_ld_wait();
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    own[j] = __uint_as_float(v[j]);
                            }
                            if (whole) {
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    sum[j] = __float_as_uint(own[j]);
                            } else {
                                float s[32];
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    s[j] = 0.0f;
                                for (uint32_t part = 0; part < seg.parts; ++part) {
                                    if (own_in_regs && part == seg.part) {
#pragma unroll
                                        for (uint32_t j = 0; j < 32; ++j)
                                            s[j] += own[j];
                                    } else {
                                        const float *src = tile_parts + static_cast<size_t>(part) * kSlotFloats +
                                                           (col_first + c * 32u) * kRows + slot_row;
#pragma unroll
                                        for (uint32_t j = 0; j < 32; ++j)
                                            s[j] += __ldcg(src + j * kRows);
                                    }
                                }
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j)
                                    sum[j] = __float_as_uint(s[j]);
                            }
                            store_chunk(p.g, stage_warp, row0, tile_col0 + c * 32u, lane, sum);
                        }
                    }
                }
                ptx::tcgen05_fence_before();
                ptx::mbar_arrive(acc_empty_bar(acc));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
                u += seg.kb_hi - seg.kb_lo;
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
