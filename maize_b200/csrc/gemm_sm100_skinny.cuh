// Skinny-M ("decode") BF16 GEMM for sm_100a: C[M x N] = A[M x K] * B[N x K]^T with M <= 128.
//
// The shape is bound by streaming B (the weights) from HBM once, so the kernel is
// built around that stream:
//
//   - operands are swapped for the tensor core: 128 rows of B are the MMA's M side,
//     the M rows of A (padded by TMA zero fill to MMA_N = 16/32/64/128) its N side;
//     the accumulator D[n][m] sits in TMEM as 128 lanes x MMA_N columns and the
//     epilogue writes it transposed, C[m][n], as runs of 32 consecutive n per warp;
//   - work is cut into units of one (128-row B tile, 64-wide k-block) = 16 KiB of B,
//     laid out tile-major, and dealt to the CTAs in equal contiguous ranges
//     (stream-K), so every SM streams the same number of bytes whatever N is;
//   - a CTA whose range covers only part of a tile's K writes its fp32 partial to a
//     scratch slot [tile][part]; the LAST warp to arrive for a (tile, lane quarter)
//     adds the parts in part order (deterministic), rounds once to bf16 and stores.
//     Arrival is a global counter per (tile, quarter) that the last warp resets, so
//     no CTA ever waits for another CTA;
//   - a deep TMA ring (128-byte swizzle, mbarrier full/empty) keeps >= 150 KiB of
//     loads in flight per SM; B is loaded with an evict-first L2 hint (read once),
//     A with evict-last (re-read by every CTA).
//
// In the reference's terms this is still the per-tile GEMM of
// crates/maize_tile/src/gemm/mod.rs:37-90 driven over column panels of B
// (crates/maize_tile/src/gmem/col_panel.rs:88-124), with the k loop of one panel
// shared between CTAs.  Roles, bounded waits and teardown follow gemm_sm100.cuh.
#pragma once
#include "gemm_common.cuh"

namespace maize {

constexpr uint32_t kSkinnyTileN = 128;  // rows of B per tile = TMEM lanes

// KBS = 64-wide k-blocks per ring stage (1 or 2): with 2, a stage holds 256 contiguous bytes of
// every B row, fetched by two adjacent TMA boxes, and the barrier traffic per byte halves.
template <uint32_t MMA_N, uint32_t KBS, uint32_t STAGES>
struct SkinnySmemLayout {
    static constexpr uint32_t kWBytes = kSkinnyTileN * kBlockK * 2;  // one weights sub-tile, 16 KiB
    static constexpr uint32_t kXBytes = MMA_N * kBlockK * 2;         // one activation sub-tile
    static constexpr uint32_t kStageBytes = KBS * (kWBytes + kXBytes);  // [W0..W(KBS-1), X0..X(KBS-1)]
    static constexpr uint32_t kRingBytes = STAGES * kStageBytes;
    static constexpr uint32_t kBarOffset = kRingBytes;
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
    __nv_bfloat16 *c;
    uint64_t ldc;
    uint32_t m, n, k;
    uint32_t tiles_n;        // ceil(N / 128)
    uint32_t num_kb;         // k-steps per tile: ceil(K / (64 * KBS))
    uint32_t units_per_cta;  // Q: CTA i owns units [i*Q, min((i+1)*Q, tiles_n*num_kb))
    uint32_t max_parts;      // scratch slots per tile
    float *partials;         // [tiles_n][max_parts][MMA_N][128] fp32
    unsigned int *counters;  // [tiles_n][4], zero between launches
    DeviceStatus *status;
    uint64_t timeout_ns;
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

template <uint32_t MMA_N, uint32_t KBS, uint32_t STAGES>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_sm100_skinny(const __grid_constant__ CUtensorMap tma_w /* B: N x K, box 128 x 64 */,
                       const __grid_constant__ CUtensorMap tma_x /* A: M x K, box MMA_N x 64 */,
                       const SkinnyParams p)
{
    using L = SkinnySmemLayout<MMA_N, KBS, STAGES>;
    static_assert(KBS == 1 || KBS == 2, "one or two k-blocks per stage");
    static_assert(MMA_N == 16 || MMA_N == 32 || MMA_N == 64 || MMA_N == 128, "MMA N side: 16, 32, 64 or 128");
    constexpr uint32_t kTmemCols = (2 * MMA_N < 32) ? 32 : 2 * MMA_N;
    constexpr uint32_t kIdesc = ptx::make_instr_desc_bf16(kSkinnyTileN, MMA_N);

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
    const WaitCtl ctl{abort_flag, p.status, p.timeout_ns};

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
            const uint64_t pol_stream = ptx::policy_evict_first();
            const uint64_t pol_keep = ptx::policy_evict_last();
            uint32_t stage = 0, phase = 0;
            uint32_t tile = u_begin / p.num_kb;
            uint32_t kb = u_begin - tile * p.num_kb;
            for (uint32_t u = u_begin; u < u_end; ++u) {
                if (!wait_bounded(empty_bar(stage), phase ^ 1u, ctl, 1))
                    break;
                const uint32_t sw = smem_base + stage * L::kStageBytes;
                const uint32_t sx = sw + KBS * L::kWBytes;
                ptx::mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
#pragma unroll
                for (uint32_t sub = 0; sub < KBS; ++sub) {
                    // a sub-block past the end of K is fetched all the same: TMA fills it with zeros
                    const int32_t kx = static_cast<int32_t>((kb * KBS + sub) * kBlockK);
                    ptx::tma_load_2d_hint(sw + sub * L::kWBytes, &tma_w, full_bar(stage), kx,
                                          static_cast<int32_t>(tile * kSkinnyTileN), pol_stream);
                    ptx::tma_load_2d_hint(sx + sub * L::kXBytes, &tma_x, full_bar(stage), kx, 0, pol_keep);
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
                if (++kb == p.num_kb) {
                    kb = 0;
                    ++tile;
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
            for (uint32_t u = u_begin; ok && u < u_end;) {
                const SkinnySegment seg = skinny_segment(u, u_end, p.num_kb, p.units_per_cta);
                if (!(ok = wait_bounded(acc_empty_bar(acc), acc_phase ^ 1u, ctl, 2)))
                    break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * MMA_N;
                for (uint32_t kb = seg.kb_lo; kb < seg.kb_hi; ++kb) {
                    if (!(ok = wait_bounded(full_bar(stage), phase, ctl, 2)))
                        break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sw = smem_base + stage * L::kStageBytes;
                    const uint32_t sx = sw + KBS * L::kWBytes;
#pragma unroll
                    for (uint32_t sub = 0; sub < KBS; ++sub) {
                        const uint64_t dw = ptx::make_smem_desc_sw128(sw + sub * L::kWBytes);  // weights: M side
                        const uint64_t dx = ptx::make_smem_desc_sw128(sx + sub * L::kXBytes);  // activations: N side
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                            ptx::mma_bf16_1cta(tmem_d, dw + 2u * k, dx + 2u * k, kIdesc,
                                               (kb != seg.kb_lo || sub != 0u || k != 0u) ? 1u : 0u);
                    }
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
        const uint32_t quarter = warp & 3u;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t u = u_begin; ok && u < u_end;) {
            const SkinnySegment seg = skinny_segment(u, u_end, p.num_kb, p.units_per_cta);
            ok = wait_bounded(acc_full_bar(acc), acc_phase, ctl, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * MMA_N;
            const uint32_t n_local = quarter * 32u + lane;          // row of the B tile = TMEM lane
            const uint32_t n = seg.tile * kSkinnyTileN + n_local;   // column of C
            const bool whole = seg.parts == 1;

            bool last = whole;
            if (!whole) {
                // publish this CTA's partial, then find out whether this warp is the last for (tile, quarter)
                float *slot = p.partials + (static_cast<size_t>(seg.tile) * p.max_parts + seg.part) * (MMA_N * 128u);
#pragma unroll 1
                for (uint32_t c = 0; c < MMA_N / 16; ++c) {
                    uint32_t v[16];
                    ptx::tmem_ld_32x32b_x16(taddr + c * 16u, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j)
                        __stcg(slot + (c * 16u + j) * 128u + n_local, __uint_as_float(v[j]));
                }
                __threadfence();
                __syncwarp();
                unsigned int seen = 0;
                if (lane == 0)
                    seen = atomicAdd(p.counters + seg.tile * 4u + quarter, 1u);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                last = seen + 1u == seg.parts;
                if (last) {
                    if (lane == 0)
                        p.counters[seg.tile * 4u + quarter] = 0u;  // ready for the next launch
                    __threadfence();
                }
            }
            if (last) {
                const float *tile_parts = p.partials + static_cast<size_t>(seg.tile) * p.max_parts * (MMA_N * 128u);
#pragma unroll 1
                for (uint32_t c = 0; c < MMA_N / 16; ++c) {
                    float sum[16];
                    if (whole) {
                        uint32_t v[16];
                        ptx::tmem_ld_32x32b_x16(taddr + c * 16u, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j)
                            sum[j] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j)
                            sum[j] = 0.0f;
                        for (uint32_t part = 0; part < seg.parts; ++part) {
                            const float *src = tile_parts + static_cast<size_t>(part) * (MMA_N * 128u) + n_local;
#pragma unroll
                            for (uint32_t j = 0; j < 16; ++j)
                                sum[j] += __ldcg(src + (c * 16u + j) * 128u);
                        }
                    }
                    if (n < p.n) {
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            const uint32_t mrow = c * 16u + j;
                            if (mrow < p.m)
                                p.c[static_cast<uint64_t>(mrow) * p.ldc + n] = __float2bfloat16_rn(sum[j]);
                        }
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
