// C ABI of the B200 BF16 GEMM (declared in include/maize_gemm.h): argument
// validation, TMA tensor-map construction, kernel selection and launch.
//
// The reference reaches its GEMM through a trace-time builder and a six-scalar
// kernel argument list (src/main.rs:31-48); this file is the run-time boundary
// that stands in for it.  Nothing here falls back to the CPU: without a CUDA
// device every compute entry point returns an error.
#include "../../include/maize_gemm.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"
#include "gemm_sm100_2cta_tail.cuh"
#include "gemm_sm100_2cta_wide.cuh"
#include "gemm_sm100_skinny.cuh"
#include "gemm_sm100_skinny_pair.cuh"
#include "gemm_sm100_skinny_pair_tall.cuh"
#include "mc_bcast.cuh"

namespace {

using maize::DeviceStatus;
using maize::GemmParams;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct KernelVariant {
    const char *name;
    uint32_t block_m;  // rows of C per tile (per CTA pair for the 2-CTA kernel)
    uint32_t block_n;
    uint32_t box_rows_b;  // rows of B one TMA box brings in
    uint32_t ctas_per_tile;
};

// Index + 1 is the public kernel id.
const KernelVariant kVariants[] = {
    {"sm100_1cta_128x256x64_s4", 128, 256, 256, 1},
    {"sm100_1cta_128x128x64_s6", 128, 128, 128, 1},
    {"sm100_1cta_128x64x64_s8", 128, 64, 64, 1},
    {"sm100_1cta_128x32x64_s8", 128, 32, 32, 1},
    {"sm100_2cta_256x256x64_s6", 256, 256, 128, 2},
    {"sm100_2cta_256x256x128_s3", 256, 256, 128, 2},
    // stream-K kernels for M <= 128: block_m = rows of A they take, block_n = rows of B per tile
    {"sm100_skinny_m32_128x256x64_s4", 32, 256, 256, 1},
    {"sm100_skinny_m128_128x256x64_s4", 128, 256, 256, 1},
    // K split over a CTA pair, halves added through distributed shared memory; tile width chosen per shape
    {"sm100_skinny_pair_m32_128xNx64_s4", 32, 256, 256, 2},
    // the CTA-pair kernel with the last, partial round of tiles split along K (forced only for now)
    {"sm100_2cta_256x256x128_s3_tail", 256, 256, 128, 2},
    // the pair-split decode kernel for 32 < M <= 128: A tile loaded once, halves exchanged through the whole ring
    {"sm100_skinny_pair_m128_128xNx64_s4", 128, 256, 256, 2},
    // 256 x 512 per CTA pair, one accumulator filling tensor memory: a quarter less L2 traffic per flop, for long K
    {"sm100_2cta_256x512x64_s4", 256, 512, 128, 2},
};
constexpr int kPairWide = 5;     // index of the CTA-pair kernel with 128-wide stages
constexpr int kFirstSkinny = 6;  // indices of the skinny variants
constexpr int kLastSkinny = 7;
constexpr int kSkinnyPair = 8;
constexpr int kPairTail = 9;
constexpr int kSkinnyPairTall = 10;
constexpr int kPairWideTile = 11;
constexpr int kNumVariants = static_cast<int>(sizeof(kVariants) / sizeof(kVariants[0]));
constexpr int kMaxProfileCtas = 1024;
constexpr uint32_t kMaxChainLanes = 4;  // streams maize_chain_forward may spread its chunks over
constexpr int kMaxHostSlabs = 16;  // row slabs of A / C that the host entry point pipelines over PCIe
constexpr size_t kPartialsBytes = size_t(32) << 20;  // stream-K scratch per context
constexpr size_t kDefaultRepackBytes = size_t(128) << 20;  // scratch of the pitch-aligning pre-pass per context
constexpr uint32_t kMaxSkinnyTiles = 65536;          // 4 counters each; N up to 8M rows

class DeviceGuard {
public:
    explicit DeviceGuard(int device) : prev_(-1), changed_(false)
    {
        if (cudaGetDevice(&prev_) == cudaSuccess && prev_ != device) {
            changed_ = cudaSetDevice(device) == cudaSuccess;
        }
    }
    ~DeviceGuard()
    {
        if (changed_)
            cudaSetDevice(prev_);
    }

private:
    int prev_;
    bool changed_;
};

}  // namespace

struct maize_ctx {
    int device = 0;
    int sm_count = 0;
    DeviceStatus *d_status = nullptr;
    DeviceStatus *h_status = nullptr;  // pinned
    uint64_t timeout_ns = 2000000000ull;
    int force_kernel = 0;
    int last_kernel = 0;             // public id of the GEMM kernel the last call launched
    int max_ctas = 0;
    uint32_t debug_flags = 0;
    uint32_t group_rows = 0;         // rows of A scheduled together; 0 = by kernel (see tile_group_rows)
    uint32_t pdl = 1;       // launch the GEMM kernels with programmatic stream serialization
    uint32_t b_static = 0;  // the caller guarantees that nothing earlier in the stream writes B (weights)
    uint32_t push_threads = 512;  // threads per CTA of the copy kernels of the multi-GPU path
    uint32_t c_evict_first = 1;   // TMA stores of C carry an evict-first L2 hint
    uint64_t wide_max_gflop = 1000000;  // largest GEMM (2MNK / 1e9) that takes the wide tile
    uint32_t wide_tile = 1;       // use the 256 x 512 pair tile where it suits (long K, full rounds, about a millisecond of work)
    uint32_t tma_store = 1;       // tiled kernels: C through shared memory and TMA stores when its rows are 16-byte aligned
    uint32_t serpentine = 1;      // odd groups of row-blocks sweep the column-blocks backwards
    uint32_t tma_promotion = 3;   // CUtensorMapL2promotion of the operand maps: 0 none, 1 64 B, 2 128 B, 3 256 B
    uint32_t tail_split = 1;      // split the last partial round of pair tiles along K when pairs would idle
    uint32_t chain_stagger = 1;   // two lanes on a source that is all there: offset them by half a chunk
    uint32_t chain_streams = 2;   // 2: maize_chain_forward alternates chunks between the caller's stream and a helper
    cudaStream_t chain_helper[kMaxChainLanes] = {};  // lanes 1 .. L-1 of maize_chain_forward (lane 0 is the caller's stream)
    cudaEvent_t chain_ev_fork = nullptr;             // the caller's stream as of the call
    cudaEvent_t chain_ev_pub[kMaxChainLanes] = {};   // "chunk published" per lane
    cudaEvent_t chain_ev_part[kMaxChainLanes] = {};  // pieces of the first chunk sent (offsets the lanes)
    uint64_t launches = 0;
    EncodeTiledFn encode = nullptr;
    void *staging = nullptr;  // device staging for the *_host entry point
    size_t staging_bytes = 0;
    // B of the last *_host call, still in the staging area: re-used instead of re-uploaded under "b_static"
    const void *host_b_ptr = nullptr;
    uint32_t host_b_rows = 0, host_b_cols = 0;
    char *host_b_dev = nullptr;
    void *repack = nullptr;  // scratch for operands copied to a 128-byte-aligned pitch ("repack_bytes")
    size_t repack_bytes = 0;
    const void *repack_b_ptr = nullptr;  // B whose aligned-pitch copy sits at the front of `repack` ("b_static" only)
    uint32_t repack_b_rows = 0, repack_b_cols = 0;
    uint64_t repack_b_ld = 0;
    // helper streams and events of the *_host entry point (created on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_start = nullptr, ev_done = nullptr;
    cudaEvent_t ev_in[kMaxHostSlabs] = {}, ev_gemm[kMaxHostSlabs] = {};
    bool attr_set[kNumVariants] = {};
    bool attr_set_kn[kNumVariants] = {};  // the same for the K x N (MN-major B) instantiations
    float *d_partials = nullptr;        // stream-K scratch of the skinny kernels
    unsigned int *d_counters = nullptr;  // arrival counters, zero between launches
    unsigned int *d_push_counter = nullptr;  // [0]: CTA arrivals of the multicast push; [16 + p]: of the scatter per rank
    unsigned long long *d_profile = nullptr;  // kProfileSlots counters per CTA, allocated when "profile" is set
    int profile_ctas = 0;                      // CTAs of the last profiled launch
    std::string err;
};

namespace {

maize_status_t fail(maize_ctx_t *ctx, maize_status_t st, const std::string &msg)
{
    if (ctx)
        ctx->err = msg;
    return st;
}

maize_status_t fail_cuda(maize_ctx_t *ctx, const char *what, cudaError_t e)
{
    return fail(ctx, MAIZE_ERR_CUDA, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

// 2-D bf16 tensor map over a row-major [rows x cols] matrix with row pitch `ld`
// elements; box = [box_rows x 64 elements], 128-byte swizzle, zero fill outside.
maize_status_t make_operand_map(maize_ctx_t *ctx, CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                                uint64_t ld, uint32_t box_rows)
{
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {ld * 2};
    cuuint32_t box[2] = {maize::kBlockK, box_rows};
    cuuint32_t estride[2] = {1, 1};
    CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), gdim, gstride, box,
                             estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             static_cast<CUtensorMapL2promotion>(ctx->tma_promotion), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[160];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (CUresult %d) for %llu x %llu, ld %llu", (int)r,
                 (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
        return fail(ctx, MAIZE_ERR_CUDA, buf);
    }
    return MAIZE_OK;
}

// Launch with programmatic stream serialization: the kernel may begin (set-up only; it orders itself with
// griddepcontrol.wait) while the stream's previous kernel is still draining.
// 2-D bf16 tensor map over C (row-major [rows x cols], row pitch `ld` elements, a multiple of 8) for the TMA-store
// epilogue: box = [32 rows x 64 elements], 128-byte swizzle.  False if the driver refuses the shape.
bool make_store_map(maize_ctx_t *ctx, CUtensorMap *map, void *base, uint64_t rows, uint64_t cols, uint64_t ld)
{
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {ld * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estride[2] = {1, 1};
    return ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, gdim, gstride, box, estride,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename Kernel, typename... Args>
cudaError_t launch_pdl(Kernel kernel, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream, const Args &...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(maize::kNumThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// `args...` = the kernel's arguments: (A map, B map, params) for the one-CTA kernels, (A map, B map, C map, params)
// for the CTA-pair kernels.
template <typename Kernel, typename... Args>
maize_status_t launch_kernel(maize_ctx_t *ctx, int variant_index, Kernel kernel, uint32_t smem_bytes, uint32_t grid,
                             cudaStream_t stream, bool b_kn, bool pdl, const Args &...args)
{
    bool &attr_done = b_kn ? ctx->attr_set_kn[variant_index] : ctx->attr_set[variant_index];
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess)
            return fail_cuda(ctx, "cudaFuncSetAttribute(max dynamic smem)", e);
        attr_done = true;
    }
    cudaError_t e;
    if (pdl) {
        e = launch_pdl(kernel, grid, smem_bytes, stream, args...);
    } else {
        kernel<<<grid, maize::kNumThreads, smem_bytes, stream>>>(args...);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

template <uint32_t BN, uint32_t STAGES, bool B_KN = false>
maize_status_t launch_variant(maize_ctx_t *ctx, int variant_index, const CUtensorMap &ta, const CUtensorMap &tb,
                              const CUtensorMap &tc, const GemmParams &p, uint32_t grid, cudaStream_t stream)
{
    return launch_kernel(ctx, variant_index, maize::gemm_bf16_sm100_1cta<BN, STAGES, B_KN>,
                         maize::GemmSmemLayout<BN, STAGES>::kDynamicBytes, grid, stream, B_KN, p.pdl != 0, ta, tb, tc, p);
}

// Tile width for the pair-split skinny kernel: the narrowest multiple of 32 for which one pair per tile
// covers N in a single wave.  Returns 0 when that needs more than 256 columns per tile.  The estimates
// (microseconds) compare it with the stream-K kernel: bytes of B per CTA at the per-SM share of the HBM
// rate, plus the measured fixed costs (launch and set-up ~5 us; exchange of halves through shared memory
// ~1.5 us against ~4 us through global memory).
uint32_t skinny_pair_tile(uint32_t sms, uint32_t n, uint32_t k, double *est_pair_us, double *est_streamk_us)
{
    const uint32_t pairs = sms / 2;
    if (pairs == 0)
        return 0;
    uint32_t bn = ((n + pairs - 1) / pairs + 31) / 32 * 32;
    if (bn < 32)
        bn = 32;
    if (bn > 256)
        return 0;
    const double num_kb = (k + maize::kBlockK - 1) / maize::kBlockK;
    const double bytes_per_us_per_sm = 6.3e6 / sms;  // 6.3 TB/s while streaming, shared by all SMs
    const double kb_bytes = 128.0;                   // bytes of one row of B in one k-block
    *est_pair_us = bn * ((num_kb + 1) / 2) * kb_bytes / bytes_per_us_per_sm + 6.5;
    *est_streamk_us = double(n) * num_kb * kb_bytes / sms / bytes_per_us_per_sm + 9.0;
    return bn;
}

// Whether the 256 x 512 pair tile suits a shape: K long enough that the exposed part of its epilogue is small,
// little of the last column block wasted, and whole rounds of tiles nearly full (it has no K split for a partial
// last round).
bool wide_tile_suits(uint32_t sms, uint32_t m, uint32_t n, uint32_t k, uint64_t max_gflop, double min_fill = 0.86)
{
    const uint64_t pairs = sms / 2 ? sms / 2 : 1;
    if (k < 2048 || m <= 128 || n < 512)
        return false;
    // Measured: in fresh runs of tens to hundreds of milliseconds the wide tile gains 5-6 % on 8192^3 and 16384^3
    // (fewer bytes moved, higher clock under the power cap).  Run back to back for seconds the part settles at a
    // clock that no longer follows the bytes, and the 256 x 256 kernel's better hidden epilogue is then 1-3 % ahead
    // on multi-millisecond GEMMs: "wide_max_gflop" lets a caller in that regime cap the size.
    if (2.0 * double(m) * double(n) * double(k) > double(max_gflop) * 1e9)
        return false;
    const uint64_t cols = (uint64_t(n) + 511) / 512 * 512;
    if (double(n) < 0.94 * double(cols))
        return false;
    const uint64_t tiles = ((uint64_t(m) + 255) / 256) * (cols / 512);
    const uint64_t rounds = (tiles + pairs - 1) / pairs;
    // 0.865 (4096^3: 128 tiles in two rounds; 16384 x 2048 x 16384: 256 tiles in four) measured 3 % and 1 % ahead of
    // the 256 x 256 kernel with its K-split last round, 0.757 (8192 x 3584 x 8192) 1.5 % behind
    return double(tiles) >= min_fill * double(rounds * pairs);
}

int pick_variant(const maize_ctx_t *ctx, uint32_t m, uint32_t n, uint32_t k)
{
    if (ctx && ctx->force_kernel >= 1 && ctx->force_kernel <= kNumVariants)
        return ctx->force_kernel - 1;
    const uint32_t sms = ctx ? static_cast<uint32_t>(ctx->sm_count) : 148u;
    const uint64_t tiles_m = (m + maize::kBlockM - 1) / maize::kBlockM;
    // One row-block of A or less: the shape is bound by streaming B, take the stream-K kernels.
    if (m <= 32) {
        double pair_us = 0, streamk_us = 0;
        if (skinny_pair_tile(sms, n, k, &pair_us, &streamk_us) != 0 && pair_us <= streamk_us)
            return kSkinnyPair;
        return kFirstSkinny;
    }
    if (m <= 128 && (uint64_t(n) + 255) / 256 < 2ull * sms) {
        double pair_us = 0, streamk_us = 0;
        // the taller exchange (up to 128 KiB through shared memory) costs ~1.5 us more than the M <= 32 one
        if (skinny_pair_tile(sms, n, k, &pair_us, &streamk_us) != 0 && pair_us + 1.5 <= streamk_us)
            return kSkinnyPairTall;
        return kFirstSkinny + 1;
    }
    // A tcgen05.mma costs the same whatever its N, so the tile is as wide as N allows: 32 / 64 / 128 wide only
    // when N itself is that narrow, otherwise 256.  Between one CTA per 128 x 256 tile and a CTA pair per
    // 256 x 256 tile (same work per CTA and per tile time, a third less operand traffic for the pair) the
    // number of waves decides; ties go to the pair.
    if (n <= 32)
        return 3;
    if (n <= 64)
        return 2;
    if (n <= 128)
        return 1;
    const uint64_t tiles_n = (uint64_t(n) + 255) / 256;
    const uint64_t pairs = sms / 2 ? sms / 2 : 1;
    const uint64_t waves_pair = (((uint64_t(m) + 255) / 256) * tiles_n + pairs - 1) / pairs;
    const uint64_t waves_single = (tiles_m * tiles_n + sms - 1) / sms;
    if (waves_pair > waves_single)
        return 0;
    return (ctx && ctx->wide_tile && wide_tile_suits(sms, m, n, k, ctx->wide_max_gflop)) ? kPairWideTile : kPairWide;
}

template <bool REPL, uint32_t STAGES>
maize_status_t launch_skinny(maize_ctx_t *ctx, int vi, const CUtensorMap &tx, const CUtensorMap &tw,
                             maize::SkinnyParams p, cudaStream_t stream)
{
    using L = maize::SkinnySmemLayout<STAGES>;
    auto kernel = maize::gemm_bf16_sm100_skinny<REPL, STAGES>;
    if (!ctx->attr_set[vi]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
        if (e != cudaSuccess)
            return fail_cuda(ctx, "cudaFuncSetAttribute(max dynamic smem)", e);
        ctx->attr_set[vi] = true;
    }
    // Equal contiguous unit ranges per CTA; fall back to whole tiles per CTA when the scratch cannot hold
    // the partials, or when there is so much work that whole tiles balance within a few percent anyway.
    uint32_t cap = static_cast<uint32_t>(ctx->sm_count);
    if (ctx->max_ctas > 0 && static_cast<uint32_t>(ctx->max_ctas) < cap)
        cap = static_cast<uint32_t>(ctx->max_ctas);
    const uint64_t units = uint64_t(p.tiles_n) * p.num_kb;
    uint64_t q = (units + cap - 1) / cap;
    // every exchange of partials costs a few microseconds of latency: do not split below 8 k-blocks per CTA
    const uint64_t min_q = p.num_kb < 8 ? p.num_kb : 8;
    if (q < min_q)
        q = min_q;
    auto parts_bound = [&](uint64_t per_cta) { return (p.num_kb - 1 + per_cta - 1) / per_cta + 1; };
    const size_t slot_bytes = size_t(maize::kSkinnyTileN) * (REPL ? 32 : 128) * sizeof(float);
    const bool plenty = p.tiles_n >= 8ull * cap;
    if (plenty || p.tiles_n > kMaxSkinnyTiles || size_t(p.tiles_n) * parts_bound(q) * slot_bytes > kPartialsBytes)
        q = ((q + p.num_kb - 1) / p.num_kb) * p.num_kb;  // whole tiles: every tile has one part
    if (q > 0xffffffffull)
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "problem too large for the skinny kernel");
    p.units_per_cta = static_cast<uint32_t>(q);
    p.max_parts = (q % p.num_kb == 0) ? 1u : static_cast<uint32_t>(parts_bound(q));
    const uint32_t grid = static_cast<uint32_t>((units + q - 1) / q);
    kernel<<<grid, maize::kNumThreads, L::kDynamicBytes, stream>>>(tx, tw, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

// Rows of A that are still arriving while the kernel runs (maize_gemm_bf16_gated).
struct RowGate {
    const uint32_t *word;
    uint32_t base;
    uint32_t rows;
};

// b_kn: B is K x N row-major with row pitch ldb (C = A * B) instead of N x K (C = A * B^T).
maize_status_t gemm_impl(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b, uint64_t ldb, void *c,
                         uint64_t ldc, uint32_t m, uint32_t n, uint32_t k, cudaStream_t stream, bool b_kn = false,
                         const RowGate *gate = nullptr)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    ctx->err.clear();
    if (m == 0 || n == 0)
        return MAIZE_OK;
    if (!c)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "C pointer is null");
    if (ldc < n)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "ldc is smaller than N");
    if (reinterpret_cast<uintptr_t>(c) % 2 != 0)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "C must be 2-byte aligned");
    DeviceGuard guard(ctx->device);
    if (k == 0) {
        // empty sum: C = 0
        cudaError_t e = cudaMemset2DAsync(c, ldc * 2, 0, size_t(n) * 2, m, stream);
        return e == cudaSuccess ? MAIZE_OK : fail_cuda(ctx, "cudaMemset2DAsync", e);
    }
    if (!a || !b)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "A or B pointer is null");
    if (lda < k || ldb < (b_kn ? n : k))
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "lda/ldb is smaller than the row length");
    if (lda % 8 != 0 || ldb % 8 != 0 || (!b_kn && k % 8 != 0))
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "K, lda and ldb must be multiples of 8 (16-byte TMA row pitch)");
    if (reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0)
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "A and B must be 16-byte aligned");
    if (lda * 2 >= (1ull << 40) || ldb * 2 >= (1ull << 40))
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "row pitch beyond the TMA limit of 2^40 bytes");

    int vi = pick_variant(ctx, m, n, k);
    if (gate) {
        // only the tiled kernels watch the gate; a forced or chosen decode kernel is replaced
        if (vi >= kFirstSkinny && vi != kPairTail && vi != kPairWideTile)
            vi = n > 128 ? 0 : (n > 64 ? 1 : (n > 32 ? 2 : 3));
        // rows that land last are multiplied last, and a partial last round of wide tiles would leave twice the
        // work behind the last chunk: a gated launch takes the wide tile only when its rounds are nearly full
        if (vi == kPairWideTile && ctx->force_kernel == 0 &&
            !wide_tile_suits(static_cast<uint32_t>(ctx->sm_count), m, n, k, ctx->wide_max_gflop, 0.92))
            vi = kPairWide;
    }
    if (b_kn) {
        // K x N tiles come in 64-column chunks: the pair kernel or the one-CTA kernels of width >= 64
        if (ctx->force_kernel != 0) {
            if (vi == 3 || (vi >= kFirstSkinny && vi != kSkinnyPair && vi != kSkinnyPairTall))
                return fail(ctx, MAIZE_ERR_UNSUPPORTED, "this kernel variant does not take a K x N matrix B");
        } else if (vi == kSkinnyPair || vi == kSkinnyPairTall) {
            // the pair-split decode kernels take a K x N matrix B (their tile widened to a multiple of 64 columns);
            // the stream-K kernels do not
            double pair_us = 0, streamk_us = 0;
            if (skinny_pair_tile(static_cast<uint32_t>(ctx->sm_count), n, k, &pair_us, &streamk_us) == 0)
                vi = n > 128 ? 0 : (n > 64 ? 1 : 2);
        } else if (vi >= kFirstSkinny && vi != kPairTail && vi != kPairWideTile) {
            vi = n > 128 ? 0 : (n > 64 ? 1 : 2);
        } else if (vi == 3) {
            vi = 2;
        }
    }
    if (vi == kPairWideTile && b_kn) {
        if (ctx->force_kernel != 0)
            return fail(ctx, MAIZE_ERR_UNSUPPORTED, "the 256 x 512 pair kernel does not take a K x N matrix B");
        vi = kPairWide;
    }
    // The wide tile's epilogue is not hidden behind the next tile's main loop, so it has to be the fast one: rows
    // of C that TMA can store.  (4111 x 3967 x 4104, odd row pitch of C: 0.164 ms against 0.137 ms.)
    if (vi == kPairWideTile && ctx->force_kernel == 0 &&
        !(ctx->tma_store && ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0))
        vi = kPairWide;
    const KernelVariant &kv = kVariants[vi];
    ctx->last_kernel = vi + 1;

    if (vi == kSkinnyPair || vi == kSkinnyPairTall) {
        const bool tall = vi == kSkinnyPairTall;
        if (m > kv.block_m)
            return fail(ctx, MAIZE_ERR_UNSUPPORTED, "forced skinny kernel takes fewer rows of A than M");
        double pair_us = 0, streamk_us = 0;
        uint32_t bn = skinny_pair_tile(static_cast<uint32_t>(ctx->sm_count), n, k, &pair_us, &streamk_us);
        if (b_kn && bn != 0)
            bn = (bn + 63u) / 64u * 64u;  // K x N tiles come in chunks of 64 columns
        if (bn == 0)
            return fail(ctx, MAIZE_ERR_UNSUPPORTED, "forced pair-split skinny kernel: N needs more than one wave of tiles");
        CUtensorMap tx, tw;
        maize_status_t sst = make_operand_map(ctx, &tx, a, m, k, lda, tall ? 128 : 32);
        if (sst != MAIZE_OK)
            return sst;
        sst = b_kn ? make_operand_map(ctx, &tw, b, k, n, ldb, maize::kBlockK)  // boxes of 64 columns x 64 k-rows
                   : make_operand_map(ctx, &tw, b, n, k, ldb, bn);
        if (sst != MAIZE_OK)
            return sst;
        maize::SkinnyPairParams pp;
        pp.g.c = static_cast<__nv_bfloat16 *>(c);
        pp.g.ldc = ldc;
        pp.g.m = m;
        pp.g.n = n;
        pp.g.k = k;
        pp.g.tiles_m = 1;
        pp.g.tiles_n = 0;
        pp.g.group_m = 1;
        pp.g.c_vec_ok = (ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1u : 0u;
        pp.g.status = ctx->d_status;
        pp.g.timeout_ns = ctx->timeout_ns;
        pp.g.profile = nullptr;
        pp.g.debug_flags = 0;
        pp.bn = bn;
        pp.tiles_n = (n + bn - 1) / bn;
        pp.num_kb = (k + maize::kBlockK - 1) / maize::kBlockK;
        auto kernel = tall ? (b_kn ? maize::gemm_bf16_sm100_skinny_pair_tall<4, true> : maize::gemm_bf16_sm100_skinny_pair_tall<4, false>)
                           : (b_kn ? maize::gemm_bf16_sm100_skinny_pair<4, true> : maize::gemm_bf16_sm100_skinny_pair<4, false>);
        bool &attr_done = b_kn ? ctx->attr_set_kn[vi] : ctx->attr_set[vi];
        if (!attr_done) {
            cudaError_t ea = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  maize::SkinnySmemLayout<4>::kDynamicBytes);
            if (ea != cudaSuccess)
                return fail_cuda(ctx, "cudaFuncSetAttribute(max dynamic smem)", ea);
            attr_done = true;
        }
        pp.pdl = ctx->pdl;
        pp.b_static = ctx->b_static;
        cudaError_t el;
        if (ctx->pdl) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * pp.tiles_n);
            cfg.blockDim = dim3(maize::kNumThreads);
            cfg.dynamicSmemBytes = maize::SkinnySmemLayout<4>::kDynamicBytes;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            el = cudaLaunchKernelEx(&cfg, kernel, tx, tw, pp);
        } else {
            kernel<<<2 * pp.tiles_n, maize::kNumThreads, maize::SkinnySmemLayout<4>::kDynamicBytes, stream>>>(tx, tw, pp);
            el = cudaGetLastError();
        }
        if (el != cudaSuccess)
            return fail_cuda(ctx, "kernel launch", el);
        ctx->launches += 1;
        return MAIZE_OK;
    }
    if (vi >= kFirstSkinny && vi <= kLastSkinny) {
        if (m > kv.block_m)
            return fail(ctx, MAIZE_ERR_UNSUPPORTED, "forced skinny kernel takes fewer rows of A than M");
        const bool repl = vi == kFirstSkinny;
        CUtensorMap tx, tw;
        maize_status_t sst = make_operand_map(ctx, &tx, a, m, k, lda, repl ? 32 : 128);
        if (sst != MAIZE_OK)
            return sst;
        sst = make_operand_map(ctx, &tw, b, n, k, ldb, maize::kSkinnyTileN);
        if (sst != MAIZE_OK)
            return sst;
        maize::SkinnyParams sp;
        sp.g.c = static_cast<__nv_bfloat16 *>(c);
        sp.g.ldc = ldc;
        sp.g.m = m;
        sp.g.n = n;
        sp.g.k = k;
        sp.g.tiles_m = 1;
        sp.g.tiles_n = 0;
        sp.g.group_m = 1;
        sp.g.c_vec_ok = (ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1u : 0u;
        sp.g.status = ctx->d_status;
        sp.g.timeout_ns = ctx->timeout_ns;
        sp.g.profile = nullptr;
        sp.g.debug_flags = ctx->debug_flags;
        sp.tiles_n = (n + maize::kSkinnyTileN - 1) / maize::kSkinnyTileN;
        sp.num_kb = (k + maize::kBlockK - 1) / maize::kBlockK;
        sp.units_per_cta = 0;
        sp.max_parts = 1;
        sp.partials = ctx->d_partials;
        sp.counters = ctx->d_counters;
        return repl ? launch_skinny<true, 4>(ctx, vi, tx, tw, sp, stream)
                    : launch_skinny<false, 4>(ctx, vi, tx, tw, sp, stream);
    }

    // Operand pitches that are not multiples of 128 bytes: copy the operand to an aligned pitch first when the
    // context holds scratch for it ("repack_bytes") and the GEMM is long enough for the copy to pay (the loads of
    // a misaligned operand cost about a third of the GEMM's time; the copy moves 4 bytes per element at ~6 TB/s
    // plus a launch).  B goes to the front of the scratch; with "b_static" (nothing writes B: weights) the copy
    // of B is kept and reused by later calls with the same B.
    if (ctx->repack && !b_kn) {
        const uint64_t pitch = (uint64_t(k) + 63) / 64 * 64;  // elements; a multiple of 128 bytes
        const bool fix_a = (lda * 2) % 128 != 0 && !gate;     // a gated A is still arriving: leave it
        const bool fix_b = (ldb * 2) % 128 != 0;
        const bool b_cached = fix_b && ctx->b_static && ctx->repack_b_ptr == b && ctx->repack_b_rows == n &&
                              ctx->repack_b_cols == k && ctx->repack_b_ld == ldb;
        const double gemm_us = 2.0 * m * n * k / 1.3e9;       // at 1300 TFLOP/s
        const double copy_us = ((fix_a ? m : 0) + (fix_b && !b_cached ? n : 0)) * double(k) * 4.0 / 6.0e6 + 4.0;
        const size_t b_bytes = fix_b ? size_t(n) * pitch * 2 : 0;
        const size_t need = b_bytes + (fix_a ? size_t(m) * pitch * 2 : 0);
        if ((fix_a || fix_b) && need <= ctx->repack_bytes && copy_us < 0.3 * gemm_us) {
            char *base = static_cast<char *>(ctx->repack);
            maize::RepackSegment seg[2] = {};
            int nseg = 0;
            if (fix_b) {
                if (!b_cached) {
                    seg[nseg++] = {static_cast<const uint4 *>(b), reinterpret_cast<uint4 *>(base), ldb / 8, pitch / 8, n};
                    ctx->repack_b_ptr = ctx->b_static ? b : nullptr;
                    ctx->repack_b_rows = n;
                    ctx->repack_b_cols = k;
                    ctx->repack_b_ld = ldb;
                }
                b = base;
                ldb = pitch;
            } else if (fix_a) {
                ctx->repack_b_ptr = nullptr;  // A is about to overwrite the front of the scratch
            }
            if (fix_a) {
                seg[nseg++] = {static_cast<const uint4 *>(a), reinterpret_cast<uint4 *>(base + b_bytes), lda / 8, pitch / 8, m};
                a = base + b_bytes;
                lda = pitch;
            }
            if (nseg > 0) {
                const uint64_t pieces = uint64_t(seg[0].rows + seg[1].rows) * (k / 8);  // 16 bytes each
                const uint64_t want = (pieces + 1023) / 1024;                          // four per thread
                const uint64_t cap = uint64_t(ctx->sm_count) * 8;
                const uint32_t rgrid = static_cast<uint32_t>(want < cap ? (want ? want : 1) : cap);
                maize::repack_rows_kernel<<<rgrid, 256, 0, stream>>>(seg[0], seg[1], k / 8);
                ctx->launches += 1;
                cudaError_t er = cudaGetLastError();
                if (er != cudaSuccess)
                    return fail_cuda(ctx, "kernel launch", er);
            }
        }
    }

    CUtensorMap ta, tb;
    maize_status_t st = make_operand_map(ctx, &ta, a, m, k, lda, maize::kBlockM);
    if (st != MAIZE_OK)
        return st;
    st = b_kn ? make_operand_map(ctx, &tb, b, k, n, ldb, maize::kBlockK)  // boxes of 64 columns x 64 k-rows
              : make_operand_map(ctx, &tb, b, n, k, ldb, kv.box_rows_b);
    if (st != MAIZE_OK)
        return st;

    // C leaves the tiled kernels (tiles of 64 columns and more) through shared memory and TMA stores when its
    // rows are 16-byte aligned
    CUtensorMap tc;
    memset(&tc, 0, sizeof tc);
    const bool c_rows_aligned = ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0;
    const bool c_tma = ctx->tma_store && c_rows_aligned && kv.block_n >= 64 && ldc * 2 < (1ull << 40) &&
                       make_store_map(ctx, &tc, c, m, n, ldc);

    GemmParams p;
    p.c = static_cast<__nv_bfloat16 *>(c);
    p.ldc = ldc;
    p.m = m;
    p.n = n;
    p.k = k;
    p.tiles_m = (m + kv.block_m - 1) / kv.block_m;
    p.tiles_n = (n + kv.block_n - 1) / kv.block_n;
    // Row-blocks swept together, their rows of A staying hot in L2.  Measured on 16384^3 (DRAM bytes per launch):
    // 2048 rows are the minimum for the 256 x 256 tiles (13.7 GB; 15-19 GB at 1024-2560), 4096 rows for the
    // 256 x 512 tile (11.2 GB against 14.8 at 2048, 15.4 at 8192, 18.9 at 16384).  A gated launch keeps 2048: its
    // first tiles then wait for one chunk of A only.
    const uint32_t group_rows = ctx->group_rows != 0 ? ctx->group_rows : ((vi == kPairWideTile && !gate) ? 4096u : 2048u);
    p.group_m = group_rows / kv.block_m;
    if (p.group_m == 0)
        p.group_m = 1;
    p.serpentine = ctx->serpentine;
    p.pdl = ctx->pdl;
    p.c_tma_ok = c_tma ? 1u : 0u;
    p.c_evict_first = ctx->c_evict_first;
    p.c_vec_ok = (ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1u : 0u;
    p.status = ctx->d_status;
    p.timeout_ns = ctx->timeout_ns;
    p.profile = ctx->d_profile;
    p.debug_flags = ctx->debug_flags;
    if (gate) {
        p.gate = gate->word;
        p.gate_base = gate->base;
        p.gate_rows = gate->rows;
    }
    const uint64_t tiles = uint64_t(p.tiles_m) * p.tiles_n;
    if (tiles > 0x7fffffffull)
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "too many output tiles");
    uint32_t cap = static_cast<uint32_t>(ctx->sm_count);
    if (ctx->max_ctas > 0 && static_cast<uint32_t>(ctx->max_ctas) < cap)
        cap = static_cast<uint32_t>(ctx->max_ctas);
    cap /= kv.ctas_per_tile;  // tiles (CTAs or CTA pairs) in flight
    if (cap == 0)
        cap = 1;
    const uint32_t grid = (tiles < cap ? static_cast<uint32_t>(tiles) : cap) * kv.ctas_per_tile;
    if (ctx->d_profile) {
        ctx->profile_ctas = static_cast<int>(grid);
        cudaMemsetAsync(ctx->d_profile, 0, sizeof(unsigned long long) * maize::kProfileSlots * kMaxProfileCtas, stream);
    }

    // The CTA-pair kernel whose last, partial round of tiles is split along K: chosen whenever the split is more
    // than 1 (idle pairs in the last round and a K long enough to cut), or forced by id.
    if ((vi == kPairWide && ctx->tail_split && !b_kn) || vi == kPairTail) {
        if (b_kn)
            return fail(ctx, MAIZE_ERR_UNSUPPORTED, "the tail-split kernel does not take a K x N matrix B");
        // P pairs run full_rounds rounds of whole tiles; the remaining tiles are cut into `split` k-ranges each,
        // as many as there are idle pairs, but never fewer than 8 k-steps of 128 per part
        const uint32_t pairs = cap;  // all pairs, also when there are fewer tiles than pairs: those get split too
        const uint32_t steps = (k + 127) / 128;
        maize::TailParams tp;
        tp.g = p;
        tp.full_rounds = static_cast<uint32_t>(tiles / pairs);
        tp.tail_tiles = static_cast<uint32_t>(tiles % pairs);
        tp.split = 1;
        if (tp.tail_tiles > 0) {
            uint32_t s = pairs / tp.tail_tiles;
            if (s > 8)
                s = 8;
            if (s > steps / 8)
                s = steps / 8;
            const size_t slot_bytes = size_t(maize::kTailSlotFloats) * sizeof(float) * 2;  // both CTAs of a pair
            while (s > 1 && size_t(tp.tail_tiles) * s * slot_bytes > kPartialsBytes)
                --s;
            if (s > 1 && tp.tail_tiles * 8u <= 4u * kMaxSkinnyTiles)
                tp.split = s;
        }
        if (tp.split > 1 || vi == kPairTail) {
            tp.partials = ctx->d_partials;
            tp.counters = ctx->d_counters;
            auto kernel = maize::gemm_bf16_sm100_2cta_tail<2, 3>;
            const uint32_t smem = maize::PairSmemLayout<256, 2, 3>::kDynamicBytes;
            if (!ctx->attr_set[kPairTail]) {
                cudaError_t ea = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
                if (ea != cudaSuccess)
                    return fail_cuda(ctx, "cudaFuncSetAttribute(max dynamic smem)", ea);
                ctx->attr_set[kPairTail] = true;
            }
            const uint64_t busy = tp.full_rounds > 0 ? pairs : uint64_t(tp.tail_tiles) * tp.split;
            cudaError_t el;
            if (tp.g.pdl) {
                el = launch_pdl(kernel, static_cast<uint32_t>(2 * busy), smem, stream, ta, tb, tc, tp);
            } else {
                kernel<<<static_cast<uint32_t>(2 * busy), maize::kNumThreads, smem, stream>>>(ta, tb, tc, tp);
                el = cudaGetLastError();
            }
            if (el != cudaSuccess)
                return fail_cuda(ctx, "kernel launch", el);
            ctx->launches += 1;
            return MAIZE_OK;
        }
    }
    if (vi == kPairWideTile)
        return launch_kernel(ctx, vi, maize::gemm_bf16_sm100_2cta_wide<4>, maize::WideSmemLayout<4>::kDynamicBytes, grid,
                             stream, false, p.pdl != 0, ta, tb, tc, p);
    if (b_kn) {
        switch (vi) {
        case 0: return launch_variant<256, 4, true>(ctx, vi, ta, tb, tc, p, grid, stream);
        case 1: return launch_variant<128, 6, true>(ctx, vi, ta, tb, tc, p, grid, stream);
        case 2: return launch_variant<64, 8, true>(ctx, vi, ta, tb, tc, p, grid, stream);
        case 4:
            return launch_kernel(ctx, vi, maize::gemm_bf16_sm100_2cta<256, 1, 6, true>,
                                 maize::PairSmemLayout<256, 1, 6>::kDynamicBytes, grid, stream, true, p.pdl != 0, ta, tb, tc, p);
        default:
            return launch_kernel(ctx, vi, maize::gemm_bf16_sm100_2cta<256, 2, 3, true>,
                                 maize::PairSmemLayout<256, 2, 3>::kDynamicBytes, grid, stream, true, p.pdl != 0, ta, tb, tc, p);
        }
    }
    switch (vi) {
    case 0: return launch_variant<256, 4>(ctx, vi, ta, tb, tc, p, grid, stream);
    case 1: return launch_variant<128, 6>(ctx, vi, ta, tb, tc, p, grid, stream);
    case 2: return launch_variant<64, 8>(ctx, vi, ta, tb, tc, p, grid, stream);
    case 3: return launch_variant<32, 8>(ctx, vi, ta, tb, tc, p, grid, stream);
    case 4:
        return launch_kernel(ctx, vi, maize::gemm_bf16_sm100_2cta<256, 1, 6>,
                             maize::PairSmemLayout<256, 1, 6>::kDynamicBytes, grid, stream, false, p.pdl != 0, ta, tb, tc, p);
    default:
        return launch_kernel(ctx, vi, maize::gemm_bf16_sm100_2cta<256, 2, 3>,
                             maize::PairSmemLayout<256, 2, 3>::kDynamicBytes, grid, stream, false, p.pdl != 0, ta, tb, tc, p);
    }
}

}  // namespace

extern "C" {

int maize_version(void) { return 100; }

const char *maize_status_string(maize_status_t s)
{
    switch (s) {
    case MAIZE_OK: return "ok";
    case MAIZE_ERR_INVALID_ARG: return "invalid argument";
    case MAIZE_ERR_UNSUPPORTED: return "unsupported shape or alignment";
    case MAIZE_ERR_CUDA: return "CUDA error";
    case MAIZE_ERR_TIMEOUT: return "device wait timed out";
    case MAIZE_ERR_DEVICE_ABORT: return "device abort";
    case MAIZE_ERR_NO_DEVICE: return "no CUDA device";
    }
    return "unknown status";
}

maize_status_t maize_ctx_create(int device, maize_ctx_t **out)
{
    if (!out)
        return MAIZE_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return MAIZE_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count)
        return MAIZE_ERR_INVALID_ARG;
    maize_ctx_t *ctx = new (std::nothrow) maize_ctx();
    if (!ctx)
        return MAIZE_ERR_CUDA;
    ctx->device = device;
    DeviceGuard guard(device);
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        delete ctx;
        return MAIZE_ERR_CUDA;
    }
    if (prop.major != 10) {
        // sm_100a code only: refuse loudly instead of failing at the first launch
        delete ctx;
        return MAIZE_ERR_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        delete ctx;
        return MAIZE_ERR_CUDA;
    }
    ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
    if (cudaMalloc(&ctx->d_status, sizeof(DeviceStatus)) != cudaSuccess ||
        cudaMemset(ctx->d_status, 0, sizeof(DeviceStatus)) != cudaSuccess ||
        cudaMalloc(&ctx->d_partials, kPartialsBytes) != cudaSuccess ||
        cudaMalloc(&ctx->d_push_counter, sizeof(unsigned int) * 32) != cudaSuccess ||
        cudaMemset(ctx->d_push_counter, 0, sizeof(unsigned int) * 32) != cudaSuccess ||
        cudaMalloc(&ctx->d_counters, sizeof(unsigned int) * 4 * kMaxSkinnyTiles) != cudaSuccess ||
        cudaMemset(ctx->d_counters, 0, sizeof(unsigned int) * 4 * kMaxSkinnyTiles) != cudaSuccess ||
        cudaMallocHost(&ctx->h_status, sizeof(DeviceStatus)) != cudaSuccess ||
        cudaMalloc(&ctx->repack, kDefaultRepackBytes) != cudaSuccess) {
        maize_ctx_destroy(ctx);
        return MAIZE_ERR_CUDA;
    }
    ctx->repack_bytes = kDefaultRepackBytes;
    // MAIZE_<KEY>=<integer> in the environment presets a tunable of every context (same keys as maize_ctx_set)
    static const char *const kEnvKeys[] = {"pdl", "tma_store", "wide_tile", "wide_max_gflop", "c_evict_first", "serpentine", "tail_split", "group_rows", "tma_promotion",
                                           "chain_streams", "chain_stagger", "b_static", "timeout_ns", "max_ctas"};
    for (const char *key : kEnvKeys) {
        std::string name = "MAIZE_";
        for (const char *c = key; *c; ++c)
            name += static_cast<char>(*c >= 'a' && *c <= 'z' ? *c - 32 : *c);
        const char *text = getenv(name.c_str());
        if (text && *text) {
            char *end = nullptr;
            const long long v = strtoll(text, &end, 10);
            if (end && *end == '\0' && maize_ctx_set(ctx, key, v) != MAIZE_OK) {
                maize_ctx_destroy(ctx);
                return MAIZE_ERR_INVALID_ARG;
            }
        }
    }
    *out = ctx;
    return MAIZE_OK;
}

void maize_ctx_destroy(maize_ctx_t *ctx)
{
    if (!ctx)
        return;
    DeviceGuard guard(ctx->device);
    if (ctx->d_status)
        cudaFree(ctx->d_status);
    if (ctx->h_status)
        cudaFreeHost(ctx->h_status);
    if (ctx->staging)
        cudaFree(ctx->staging);
    if (ctx->repack)
        cudaFree(ctx->repack);
    for (uint32_t j = 0; j < kMaxChainLanes; ++j) {
        if (ctx->chain_helper[j])
            cudaStreamDestroy(ctx->chain_helper[j]);
        if (ctx->chain_ev_pub[j])
            cudaEventDestroy(ctx->chain_ev_pub[j]);
        if (ctx->chain_ev_part[j])
            cudaEventDestroy(ctx->chain_ev_part[j]);
    }
    if (ctx->chain_ev_fork)
        cudaEventDestroy(ctx->chain_ev_fork);
    if (ctx->copy_in)
        cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out)
        cudaStreamDestroy(ctx->copy_out);
    if (ctx->ev_start)
        cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_done)
        cudaEventDestroy(ctx->ev_done);
    for (int i = 0; i < kMaxHostSlabs; ++i) {
        if (ctx->ev_in[i])
            cudaEventDestroy(ctx->ev_in[i]);
        if (ctx->ev_gemm[i])
            cudaEventDestroy(ctx->ev_gemm[i]);
    }
    if (ctx->d_profile)
        cudaFree(ctx->d_profile);
    if (ctx->d_partials)
        cudaFree(ctx->d_partials);
    if (ctx->d_counters)
        cudaFree(ctx->d_counters);
    if (ctx->d_push_counter)
        cudaFree(ctx->d_push_counter);
    delete ctx;
}

const char *maize_last_error(const maize_ctx_t *ctx) { return ctx ? ctx->err.c_str() : "null context"; }

maize_status_t maize_gemm_bf16(maize_ctx_t *ctx, const void *a, uint32_t a_rows, uint32_t a_cols, const void *b,
                               uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows, uint32_t c_cols,
                               void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (a_cols != b_cols)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "a_cols != b_cols (both are K; B is stored N x K)");
    if (c_rows != a_rows || c_cols != b_rows)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "C must be a_rows x b_rows");
    return gemm_impl(ctx, a, a_cols, b, b_cols, c, c_cols, a_rows, b_rows, a_cols, static_cast<cudaStream_t>(cuda_stream));
}

maize_status_t maize_gemm_bf16_m(maize_ctx_t *ctx, const maize_global_matrix_t *a, const maize_global_matrix_t *b,
                                 const maize_global_matrix_t *c, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!a || !b || !c)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "null matrix descriptor");
    return maize_gemm_bf16(ctx, a->ptr, a->nrows, a->ncols, b->ptr, b->nrows, b->ncols, c->ptr, c->nrows, c->ncols,
                           cuda_stream);
}

maize_status_t maize_gemm_bf16_ld(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b, uint64_t ldb, void *c,
                                  uint64_t ldc, uint32_t m, uint32_t n, uint32_t k, void *cuda_stream)
{
    return gemm_impl(ctx, a, lda, b, ldb, c, ldc, m, n, k, static_cast<cudaStream_t>(cuda_stream));
}

maize_status_t maize_gemm_bf16_gated(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b, uint64_t ldb,
                                     void *c, uint64_t ldc, uint32_t m, uint32_t n, uint32_t k,
                                     const void *rows_landed, uint32_t landed_base, uint32_t rows_per_count,
                                     void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!rows_landed || reinterpret_cast<uintptr_t>(rows_landed) % 4 != 0 || rows_per_count == 0)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "gated GEMM: the counter must be a 4-byte aligned word and rows_per_count > 0");
    const RowGate gate{static_cast<const uint32_t *>(rows_landed), landed_base, rows_per_count};
    return gemm_impl(ctx, a, lda, b, ldb, c, ldc, m, n, k, static_cast<cudaStream_t>(cuda_stream), false, &gate);
}

maize_status_t maize_gemm_bf16_kn(maize_ctx_t *ctx, const void *a, uint32_t a_rows, uint32_t a_cols, const void *b,
                                  uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows, uint32_t c_cols,
                                  void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (a_cols != b_rows)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "a_cols != b_rows (both are K; B is stored K x N)");
    if (c_rows != a_rows || c_cols != b_cols)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "C must be a_rows x b_cols");
    return gemm_impl(ctx, a, a_cols, b, b_cols, c, c_cols, a_rows, b_cols, a_cols, static_cast<cudaStream_t>(cuda_stream),
                     true);
}

maize_status_t maize_gemm_bf16_kn_ld(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b, uint64_t ldb,
                                     void *c, uint64_t ldc, uint32_t m, uint32_t n, uint32_t k, void *cuda_stream)
{
    return gemm_impl(ctx, a, lda, b, ldb, c, ldc, m, n, k, static_cast<cudaStream_t>(cuda_stream), true);
}

maize_status_t maize_gemm_bf16_host(maize_ctx_t *ctx, const void *a_host, uint32_t a_rows, uint32_t a_cols,
                                    const void *b_host, uint32_t b_rows, uint32_t b_cols, void *c_host,
                                    uint32_t c_rows, uint32_t c_cols, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (a_cols != b_cols)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "a_cols != b_cols (both are K; B is stored N x K)");
    if (c_rows != a_rows || c_cols != b_rows)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "C must be a_rows x b_rows");
    if (a_rows == 0 || b_rows == 0)
        return MAIZE_OK;
    if (!c_host || ((!a_host || !b_host) && a_cols > 0))
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "null host pointer");
    DeviceGuard guard(ctx->device);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    auto round_up = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t a_bytes = size_t(a_rows) * a_cols * 2, b_bytes = size_t(b_rows) * b_cols * 2;
    const size_t c_bytes = size_t(c_rows) * c_cols * 2;
    const size_t need = round_up(a_bytes) + round_up(b_bytes) + round_up(c_bytes);
    if (need > ctx->staging_bytes) {
        if (ctx->staging) {
            cudaStreamSynchronize(stream);
            cudaFree(ctx->staging);
            ctx->staging = nullptr;
            ctx->staging_bytes = 0;
            ctx->host_b_ptr = nullptr;
        }
        cudaError_t e = cudaMalloc(&ctx->staging, need);
        if (e != cudaSuccess)
            return fail_cuda(ctx, "cudaMalloc(staging)", e);
        ctx->staging_bytes = need;
    }
    // B sits at the front of the staging area, so that a B declared static ("b_static": inference weights that
    // the caller does not change between calls) can stay there and need not cross PCIe again
    char *db = static_cast<char *>(ctx->staging);
    char *da = db + round_up(b_bytes);
    char *dc = da + round_up(a_bytes);
    const bool b_resident = ctx->b_static && ctx->host_b_ptr == b_host && ctx->host_b_rows == b_rows &&
                            ctx->host_b_cols == b_cols && ctx->host_b_dev == db;
    ctx->host_b_ptr = ctx->b_static ? b_host : nullptr;
    ctx->host_b_rows = b_rows;
    ctx->host_b_cols = b_cols;
    ctx->host_b_dev = db;
    cudaError_t e;
    // Small problems: one copy in, one GEMM, one copy out, all on the caller's stream.
    // Large ones: B goes first, then A in row slabs on a copy stream; the GEMM of slab i starts when slab i
    // has landed and the rows of C it produces go back on a second copy stream, so that the H2D of slab
    // i+1, the math of slab i and the D2H of slab i-1 overlap (PCIe is full duplex; the GPU has several
    // copy engines).  The call still returns only when C is complete in host memory.
    const uint32_t m = a_rows, n = b_rows, k = a_cols;
    uint32_t nslabs = 1;
    if (a_bytes + b_bytes + c_bytes >= (size_t(64) << 20) && m >= 1024 && k > 0) {
        nslabs = m / 1024;
        if (nslabs > static_cast<uint32_t>(kMaxHostSlabs))
            nslabs = kMaxHostSlabs;
    }
    if (nslabs <= 1) {
        if (a_bytes && (e = cudaMemcpyAsync(da, a_host, a_bytes, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
            return fail_cuda(ctx, "H2D copy of A", e);
        if (b_bytes && !b_resident && (e = cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
            return fail_cuda(ctx, "H2D copy of B", e);
        maize_status_t st = gemm_impl(ctx, da, k, db, k, dc, n, m, n, k, stream);
        if (st != MAIZE_OK)
            return st;
        if ((e = cudaMemcpyAsync(c_host, dc, c_bytes, cudaMemcpyDeviceToHost, stream)) != cudaSuccess)
            return fail_cuda(ctx, "D2H copy of C", e);
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess)
            return fail_cuda(ctx, "cudaStreamSynchronize", e);
        return MAIZE_OK;
    }
    if (!ctx->copy_in) {
        bool ok = cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&ctx->ev_start, cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&ctx->ev_done, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < kMaxHostSlabs; ++i)
            ok = cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&ctx->ev_gemm[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok)
            return fail_cuda(ctx, "creating the copy streams / events", cudaGetLastError());
    }
    const uint32_t slab_rows = ((m + nslabs - 1) / nslabs + 255) / 256 * 256;
    // the copies must come after whatever the caller queued before this call
    if ((e = cudaEventRecord(ctx->ev_start, stream)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(ctx->copy_in, ctx->ev_start, 0)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(ctx->copy_out, ctx->ev_start, 0)) != cudaSuccess)
        return fail_cuda(ctx, "ordering the copy streams", e);
    if (!b_resident && (e = cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, ctx->copy_in)) != cudaSuccess)
        return fail_cuda(ctx, "H2D copy of B", e);
    uint32_t used = 0;
    for (uint32_t row0 = 0; row0 < m; row0 += slab_rows, ++used) {
        const uint32_t rows = (m - row0 < slab_rows) ? (m - row0) : slab_rows;
        const size_t a_off = size_t(row0) * k * 2, c_off = size_t(row0) * n * 2;
        if ((e = cudaMemcpyAsync(da + a_off, static_cast<const char *>(a_host) + a_off, size_t(rows) * k * 2,
                                 cudaMemcpyHostToDevice, ctx->copy_in)) != cudaSuccess ||
            (e = cudaEventRecord(ctx->ev_in[used], ctx->copy_in)) != cudaSuccess ||
            (e = cudaStreamWaitEvent(stream, ctx->ev_in[used], 0)) != cudaSuccess)
            return fail_cuda(ctx, "H2D copy of an A slab", e);
        maize_status_t st = gemm_impl(ctx, da + a_off, k, db, k, dc + c_off, n, rows, n, k, stream);
        if (st != MAIZE_OK)
            return st;
        if ((e = cudaEventRecord(ctx->ev_gemm[used], stream)) != cudaSuccess ||
            (e = cudaStreamWaitEvent(ctx->copy_out, ctx->ev_gemm[used], 0)) != cudaSuccess ||
            (e = cudaMemcpyAsync(static_cast<char *>(c_host) + c_off, dc + c_off, size_t(rows) * n * 2,
                                 cudaMemcpyDeviceToHost, ctx->copy_out)) != cudaSuccess)
            return fail_cuda(ctx, "D2H copy of a C slab", e);
    }
    if ((e = cudaEventRecord(ctx->ev_done, ctx->copy_out)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(stream, ctx->ev_done, 0)) != cudaSuccess ||
        (e = cudaStreamSynchronize(stream)) != cudaSuccess)
        return fail_cuda(ctx, "waiting for C", e);
    return MAIZE_OK;
}

maize_status_t maize_ctx_poll(maize_ctx_t *ctx, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t e = cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess)
        e = cudaMemsetAsync(ctx->d_status, 0, sizeof(DeviceStatus), stream);
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess)
        return fail_cuda(ctx, "status read-back", e);
    const DeviceStatus s = *ctx->h_status;
    if (s.code == maize::kStatusOk)
        return MAIZE_OK;
    // A launch that gave up on a wait may have left arrival counters of the stream-K exchange or of the push
    // kernels half-way; the next launch must find them at zero again, or it would combine stale partial sums.
    cudaMemsetAsync(ctx->d_counters, 0, sizeof(unsigned int) * 4 * kMaxSkinnyTiles, stream);
    cudaMemsetAsync(ctx->d_push_counter, 0, sizeof(unsigned int) * 32, stream);
    cudaStreamSynchronize(stream);
    char buf[128];
    snprintf(buf, sizeof buf, "device status %d raised by role %d of CTA %d", s.code, s.role, s.cta);
    ctx->err = buf;
    return s.code == maize::kStatusTimeout ? MAIZE_ERR_TIMEOUT : MAIZE_ERR_DEVICE_ABORT;
}

maize_status_t maize_ctx_set(maize_ctx_t *ctx, const char *key, int64_t value)
{
    if (!ctx || !key)
        return MAIZE_ERR_INVALID_ARG;
    if (!strcmp(key, "timeout_ns")) {
        if (value <= 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "timeout_ns must be positive");
        ctx->timeout_ns = static_cast<uint64_t>(value);
    } else if (!strcmp(key, "force_kernel")) {
        if (value < 0 || value > kNumVariants)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "force_kernel out of range");
        ctx->force_kernel = static_cast<int>(value);
    } else if (!strcmp(key, "profile")) {
        // per-CTA cycle accounting of the next launches (a debugging aid; costs a few clock reads per wait)
        DeviceGuard guard(ctx->device);
        if (value && !ctx->d_profile) {
            cudaError_t e = cudaMalloc(&ctx->d_profile, sizeof(unsigned long long) * maize::kProfileSlots * kMaxProfileCtas);
            if (e != cudaSuccess)
                return fail_cuda(ctx, "cudaMalloc(profile)", e);
        } else if (!value && ctx->d_profile) {
            cudaDeviceSynchronize();
            cudaFree(ctx->d_profile);
            ctx->d_profile = nullptr;
            ctx->debug_flags = 0;
        }
    } else if (!strcmp(key, "repack_bytes")) {
        // Scratch for the pitch-aligning pre-pass (0 frees it).  Allocated here, never inside a GEMM call.
        if (value < 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "repack_bytes must be >= 0");
        DeviceGuard guard(ctx->device);
        ctx->repack_b_ptr = nullptr;
        if (ctx->repack) {
            cudaDeviceSynchronize();
            cudaFree(ctx->repack);
            ctx->repack = nullptr;
            ctx->repack_bytes = 0;
        }
        if (value > 0) {
            cudaError_t e = cudaMalloc(&ctx->repack, static_cast<size_t>(value));
            if (e != cudaSuccess)
                return fail_cuda(ctx, "cudaMalloc(repack)", e);
            ctx->repack_bytes = static_cast<size_t>(value);
        }
    } else if (!strcmp(key, "group_rows")) {
        if (value != 0 && (value < 128 || value > (1 << 24)))
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "group_rows out of range");
        ctx->group_rows = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "pdl")) {
        ctx->pdl = value ? 1u : 0u;
    } else if (!strcmp(key, "b_static")) {
        ctx->b_static = value ? 1u : 0u;
        ctx->repack_b_ptr = nullptr;  // a kept copy of B is only valid while the promise holds
        ctx->host_b_ptr = nullptr;
    } else if (!strcmp(key, "tma_promotion")) {
        if (value < 0 || value > 3)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "tma_promotion: 0 (none), 1 (64 B), 2 (128 B) or 3 (256 B)");
        ctx->tma_promotion = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "c_evict_first")) {
        ctx->c_evict_first = value ? 1u : 0u;
    } else if (!strcmp(key, "wide_max_gflop")) {
        if (value < 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "wide_max_gflop must be >= 0");
        ctx->wide_max_gflop = static_cast<uint64_t>(value);
    } else if (!strcmp(key, "wide_tile")) {
        ctx->wide_tile = value ? 1u : 0u;
    } else if (!strcmp(key, "tma_store")) {
        ctx->tma_store = value ? 1u : 0u;
    } else if (!strcmp(key, "serpentine")) {
        ctx->serpentine = value ? 1u : 0u;
    } else if (!strcmp(key, "tail_split")) {
        ctx->tail_split = value ? 1u : 0u;
    } else if (!strcmp(key, "chain_stagger")) {
        ctx->chain_stagger = value ? 1u : 0u;
    } else if (!strcmp(key, "chain_streams")) {
        if (value < 1 || value > static_cast<int64_t>(kMaxChainLanes))
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "chain_streams: 1 to 4");
        ctx->chain_streams = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "push_threads")) {
        if (value < 32 || value > 512 || value % 32 != 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "push_threads: a multiple of 32 in [32, 512]");
        ctx->push_threads = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "debug_flags")) {
        // these switches make results wrong on purpose; they are honoured only while "profile" is on
        if (value != 0 && !ctx->d_profile)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "debug_flags may only be set while \"profile\" is 1");
        ctx->debug_flags = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "max_ctas")) {
        if (value < 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "max_ctas must be >= 0");
        ctx->max_ctas = static_cast<int>(value);
    } else {
        return fail(ctx, MAIZE_ERR_INVALID_ARG, std::string("unknown key: ") + key);
    }
    return MAIZE_OK;
}

maize_status_t maize_ctx_get(const maize_ctx_t *ctx, const char *key, int64_t *value)
{
    if (!ctx || !key || !value)
        return MAIZE_ERR_INVALID_ARG;
    if (!strcmp(key, "timeout_ns"))
        *value = static_cast<int64_t>(ctx->timeout_ns);
    else if (!strcmp(key, "force_kernel"))
        *value = ctx->force_kernel;
    else if (!strcmp(key, "max_ctas"))
        *value = ctx->max_ctas;
    else if (!strcmp(key, "sm_count"))
        *value = ctx->sm_count;
    else if (!strcmp(key, "device"))
        *value = ctx->device;
    else if (!strcmp(key, "group_rows"))
        *value = ctx->group_rows;
    else if (!strcmp(key, "pdl"))
        *value = ctx->pdl;
    else if (!strcmp(key, "b_static"))
        *value = ctx->b_static;
    else if (!strcmp(key, "push_threads"))
        *value = ctx->push_threads;
    else if (!strcmp(key, "debug_flags"))
        *value = ctx->debug_flags;
    else if (!strcmp(key, "profile"))
        *value = ctx->d_profile ? 1 : 0;
    else if (!strcmp(key, "chain_streams"))
        *value = ctx->chain_streams;
    else if (!strcmp(key, "chain_stagger"))
        *value = ctx->chain_stagger;
    else if (!strcmp(key, "tail_split"))
        *value = ctx->tail_split;
    else if (!strcmp(key, "serpentine"))
        *value = ctx->serpentine;
    else if (!strcmp(key, "tma_store"))
        *value = ctx->tma_store;
    else if (!strcmp(key, "wide_tile"))
        *value = ctx->wide_tile;
    else if (!strcmp(key, "wide_max_gflop"))
        *value = static_cast<int64_t>(ctx->wide_max_gflop);
    else if (!strcmp(key, "c_evict_first"))
        *value = ctx->c_evict_first;
    else if (!strcmp(key, "tma_promotion"))
        *value = ctx->tma_promotion;
    else if (!strcmp(key, "repack_bytes"))
        *value = static_cast<int64_t>(ctx->repack_bytes);
    else if (!strcmp(key, "last_kernel"))
        *value = ctx->last_kernel;
    else
        return MAIZE_ERR_INVALID_ARG;
    return MAIZE_OK;
}

const char *maize_kernel_name(int id)
{
    if (id < 1 || id > kNumVariants)
        return nullptr;
    return kVariants[id - 1].name;
}

int maize_pick_kernel(const maize_ctx_t *ctx, uint32_t m, uint32_t n, uint32_t k) { return pick_variant(ctx, m, n, k) + 1; }

uint64_t maize_ctx_launch_count(const maize_ctx_t *ctx) { return ctx ? ctx->launches : 0; }

int maize_ctx_read_profile(maize_ctx_t *ctx, uint64_t *out, int max_ctas, void *cuda_stream)
{
    if (!ctx || !out || !ctx->d_profile || max_ctas <= 0)
        return 0;
    DeviceGuard guard(ctx->device);
    int n = ctx->profile_ctas < max_ctas ? ctx->profile_ctas : max_ctas;
    if (n > kMaxProfileCtas)
        n = kMaxProfileCtas;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (cudaStreamSynchronize(stream) != cudaSuccess)
        return 0;
    if (cudaMemcpy(out, ctx->d_profile, sizeof(uint64_t) * maize::kProfileSlots * n, cudaMemcpyDeviceToHost) != cudaSuccess)
        return 0;
    return n;
}

maize_status_t maize_mc_push_after(maize_ctx_t *ctx, const void *wait_flag, uint32_t wait_value, const void *src,
                                   void *mc_dst, uint64_t bytes, void *mc_flag, uint32_t flag_value, int ctas,
                                   void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!src || !mc_dst || !mc_flag)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "null pointer");
    if (bytes % 16 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0 || reinterpret_cast<uintptr_t>(mc_dst) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(mc_flag) % 4 != 0 || reinterpret_cast<uintptr_t>(wait_flag) % 4 != 0)
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "multicast push needs 16-byte aligned buffers and size");
    // Default: 16 CTAs of 512 threads.  One source saturates its multicast path (about 400 GB/s here)
    // from 16 CTAs on; spreading the copy as one small CTA per SM measured 15-20% slower per step.
    if (ctas <= 0)
        ctas = 16;
    if (ctas > 4 * ctx->sm_count)
        ctas = 4 * ctx->sm_count;
    DeviceGuard guard(ctx->device);
    maize::mc_push_kernel<<<ctas, ctx->push_threads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint4 *>(src), static_cast<uint4 *>(mc_dst), bytes / 16, ctx->d_push_counter,
        static_cast<uint32_t *>(mc_flag), flag_value, static_cast<const uint32_t *>(wait_flag), wait_value,
        ctx->d_status, ctx->timeout_ns);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

maize_status_t maize_mc_push(maize_ctx_t *ctx, const void *src, void *mc_dst, uint64_t bytes, void *mc_flag,
                             uint32_t flag_value, int ctas, void *cuda_stream)
{
    return maize_mc_push_after(ctx, nullptr, 0, src, mc_dst, bytes, mc_flag, flag_value, ctas, cuda_stream);
}

maize_status_t maize_scatter_push(maize_ctx_t *ctx, const void *src, void *const *peer_dst, void *const *peer_flag,
                                  uint32_t world, uint32_t root, uint64_t bytes, uint32_t flag_value, int ctas,
                                  void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!src || !peer_dst || !peer_flag || world < 2 || world > maize::kMaxPeers || root >= world)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "scatter: bad pointer, world size or root");
    if (bytes % 16 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0)
        return fail(ctx, MAIZE_ERR_UNSUPPORTED, "scatter needs 16-byte aligned buffers and size");
    maize::ScatterTargets t = {};
    for (uint32_t p = 0; p < world; ++p) {
        if (p == root)
            continue;
        if (!peer_dst[p] || !peer_flag[p] || reinterpret_cast<uintptr_t>(peer_dst[p]) % 16 != 0 ||
            reinterpret_cast<uintptr_t>(peer_flag[p]) % 4 != 0)
            return fail(ctx, MAIZE_ERR_INVALID_ARG, "scatter: bad peer pointer");
        t.dst[p] = static_cast<uint4 *>(peer_dst[p]);
        t.flag[p] = static_cast<uint32_t *>(peer_flag[p]);
    }
    const uint32_t peers = world - 1;
    if (ctas <= 0)
        ctas = 32;
    uint32_t grid = static_cast<uint32_t>(ctas);
    if (grid < peers)
        grid = peers;  // at least one CTA per peer
    grid = (grid + peers - 1) / peers * peers;
    DeviceGuard guard(ctx->device);
    maize::scatter_push_kernel<<<grid, ctx->push_threads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint4 *>(src), t, bytes / 16, world, root, flag_value, ctx->d_push_counter + 16);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

maize_status_t maize_copy_async(maize_ctx_t *ctx, void *dst, const void *src, uint64_t bytes, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (bytes == 0)
        return MAIZE_OK;
    if (!dst || !src)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "null pointer");
    DeviceGuard guard(ctx->device);
    // device-to-device; with a peer-mapped destination the copy engines move the bytes over NVLink, no SM involved
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess)
        return fail_cuda(ctx, "cudaMemcpyAsync", e);
    return MAIZE_OK;
}

maize_status_t maize_chain_forward(maize_ctx_t *ctx, const void *wait_flag, uint32_t first_value, void *dst,
                                   const void *src, uint64_t total_bytes, uint64_t chunk_bytes, void *dst_flag,
                                   void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!dst || !src || !dst_flag || chunk_bytes == 0 || reinterpret_cast<uintptr_t>(dst_flag) % 4 != 0 ||
        reinterpret_cast<uintptr_t>(wait_flag) % 4 != 0)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "chain: bad pointer or chunk size");
    DeviceGuard guard(ctx->device);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (ctx->chain_streams >= 2 && total_bytes > chunk_bytes) {
        // Chunks go round robin over L lanes (the caller's stream and L - 1 helper streams), so that the small
        // kernels around one chunk's copy run while other lanes' copies keep the link busy, and several copies are
        // in flight at once.  Counts are still published in chunk order: the publishing kernel of chunk i waits
        // (stream event) for the one of chunk i - 1.
        const uint32_t L = ctx->chain_streams;
        if (!ctx->chain_ev_fork) {
            bool ok = cudaEventCreateWithFlags(&ctx->chain_ev_fork, cudaEventDisableTiming) == cudaSuccess;
            for (uint32_t j = 0; ok && j < kMaxChainLanes; ++j)
                ok = cudaEventCreateWithFlags(&ctx->chain_ev_pub[j], cudaEventDisableTiming) == cudaSuccess &&
                     cudaEventCreateWithFlags(&ctx->chain_ev_part[j], cudaEventDisableTiming) == cudaSuccess &&
                     (j == 0 || cudaStreamCreateWithFlags(&ctx->chain_helper[j], cudaStreamNonBlocking) == cudaSuccess);
            if (!ok)
                return fail_cuda(ctx, "creating the chain's helper streams / events", cudaGetLastError());
        }
        cudaStream_t lanes[kMaxChainLanes];
        lanes[0] = stream;
        for (uint32_t j = 1; j < L; ++j)
            lanes[j] = ctx->chain_helper[j];
        cudaError_t e;
        // fork: the helpers start after whatever the caller queued on its stream before this call
        if ((e = cudaEventRecord(ctx->chain_ev_fork, stream)) != cudaSuccess)
            return fail_cuda(ctx, "forking the chain's helper streams", e);
        for (uint32_t j = 1; j < L; ++j)
            if ((e = cudaStreamWaitEvent(lanes[j], ctx->chain_ev_fork, 0)) != cudaSuccess)
                return fail_cuda(ctx, "forking the chain's helper streams", e);
        uint32_t v = first_value;
        uint32_t i = 0;
        for (uint64_t off = 0; off < total_bytes; off += chunk_bytes, ++v, ++i) {
            const uint64_t nbytes = total_bytes - off < chunk_bytes ? total_bytes - off : chunk_bytes;
            const uint32_t lane = i % L;
            cudaStream_t s = lanes[lane];
            if (wait_flag) {
                maize::chain_step_kernel<<<1, 32, 0, s>>>(nullptr, 0, static_cast<const uint32_t *>(wait_flag), v,
                                                          ctx->d_status, ctx->timeout_ns);
                ctx->launches += 1;
            }
            if (!wait_flag && i == 0 && nbytes >= 16 * L && ctx->chain_stagger) {
                // A source that is all there (the root's) would keep the lanes in lock step: equal copies started
                // together share the link and end together, and the link then idles while all lanes publish.  Offset
                // them: chunk 0 goes out in L pieces, and lane j starts when piece j has gone out.
                const uint64_t piece = (nbytes / L) & ~uint64_t(15);
                for (uint32_t j = 0; j < L; ++j) {
                    const uint64_t lo = j * piece, hi = j + 1 == L ? nbytes : (j + 1) * piece;
                    if ((e = cudaMemcpyAsync(static_cast<char *>(dst) + lo, static_cast<const char *>(src) + lo, hi - lo,
                                             cudaMemcpyDeviceToDevice, s)) != cudaSuccess)
                        return fail_cuda(ctx, "cudaMemcpyAsync (staggered first chunk)", e);
                    if (j + 1 < L && ((e = cudaEventRecord(ctx->chain_ev_part[j], s)) != cudaSuccess ||
                                      (e = cudaStreamWaitEvent(lanes[j + 1], ctx->chain_ev_part[j], 0)) != cudaSuccess))
                        return fail_cuda(ctx, "offsetting the chain's lanes", e);
                }
            } else if ((e = cudaMemcpyAsync(static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, nbytes,
                                            cudaMemcpyDeviceToDevice, s)) != cudaSuccess)
                return fail_cuda(ctx, "cudaMemcpyAsync", e);
            if (i > 0 && (e = cudaStreamWaitEvent(s, ctx->chain_ev_pub[(i - 1) % L], 0)) != cudaSuccess)
                return fail_cuda(ctx, "ordering the chain's publications", e);
            maize::chain_step_kernel<<<1, 32, 0, s>>>(static_cast<uint32_t *>(dst_flag), v, nullptr, 0, ctx->d_status,
                                                      ctx->timeout_ns);
            ctx->launches += 1;
            if ((e = cudaGetLastError()) != cudaSuccess)
                return fail_cuda(ctx, "kernel launch", e);
            if ((e = cudaEventRecord(ctx->chain_ev_pub[lane], s)) != cudaSuccess)
                return fail_cuda(ctx, "cudaEventRecord", e);
        }
        // join: the caller's stream continues after the last publication (which is after all earlier ones)
        if ((i - 1) % L != 0 && (e = cudaStreamWaitEvent(stream, ctx->chain_ev_pub[(i - 1) % L], 0)) != cudaSuccess)
            return fail_cuda(ctx, "joining the chain's helper streams", e);
        return MAIZE_OK;
    }
    // Per chunk: one copy and ONE one-thread kernel that publishes the chunk just copied and, on a rank that
    // receives, waits for the next chunk to forward (the first chunk's wait is a launch of its own).
    const uint32_t *wait = static_cast<const uint32_t *>(wait_flag);
    uint32_t *publish = static_cast<uint32_t *>(dst_flag);
    uint32_t value = first_value;
    if (wait && total_bytes > 0) {
        maize::chain_step_kernel<<<1, 32, 0, stream>>>(nullptr, 0, wait, value, ctx->d_status, ctx->timeout_ns);
        ctx->launches += 1;
    }
    for (uint64_t off = 0; off < total_bytes; off += chunk_bytes, ++value) {
        const uint64_t nbytes = total_bytes - off < chunk_bytes ? total_bytes - off : chunk_bytes;
        const bool more = off + chunk_bytes < total_bytes;
        cudaError_t e = cudaMemcpyAsync(static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, nbytes,
                                        cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess)
            return fail_cuda(ctx, "cudaMemcpyAsync", e);
        maize::chain_step_kernel<<<1, 32, 0, stream>>>(publish, value, (wait && more) ? wait : nullptr, value + 1,
                                                       ctx->d_status, ctx->timeout_ns);
        ctx->launches += 1;
        if ((e = cudaGetLastError()) != cudaSuccess)
            return fail_cuda(ctx, "kernel launch", e);
    }
    return MAIZE_OK;
}

maize_status_t maize_flags_wait(maize_ctx_t *ctx, const void *flags, uint32_t count, uint32_t value, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!flags || count == 0 || count > 32 || reinterpret_cast<uintptr_t>(flags) % 4 != 0)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "flags: 1 to 32 aligned 32-bit words");
    DeviceGuard guard(ctx->device);
    maize::flags_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint32_t *>(flags), count, value, ctx->d_status, ctx->timeout_ns);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

maize_status_t maize_flag_store(maize_ctx_t *ctx, void *flag, uint32_t value, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (!flag || reinterpret_cast<uintptr_t>(flag) % 4 != 0)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "flag: aligned 32-bit word");
    DeviceGuard guard(ctx->device);
    maize::flag_store_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(static_cast<uint32_t *>(flag), value);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

maize_status_t maize_debug_wait_expires(maize_ctx_t *ctx, uint64_t budget_ns, void *cuda_stream)
{
    if (!ctx)
        return MAIZE_ERR_INVALID_ARG;
    if (budget_ns == 0 || budget_ns > 1000000000ull)
        return fail(ctx, MAIZE_ERR_INVALID_ARG, "budget_ns must be in (0, 1e9]");
    DeviceGuard guard(ctx->device);
    maize::wait_expires_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(ctx->d_status, budget_ns);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail_cuda(ctx, "kernel launch", e);
    ctx->launches += 1;
    return MAIZE_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free skinny GEMM.
//
// Some hosts may not call cudaMalloc at the point where they need a decode-shaped GEMM: a service with
// a "no allocation after start-up" rule (everything is reserved up front so that a late allocation can
// neither fail nor stall the device), or a plugin whose host owns every byte of device memory and hands
// out only the operand buffers.  For them the stream-K scratch of the skinny kernel lives in the library
// image itself, in the file-scope array below, instead of in a context (creating a context allocates).
//
// The array belongs to the module: every GPU that loads this library holds kStaticScratchBytes of it
// until the process exits, whether or not the entry point is ever called.  In HOST code the array's
// name is only a handle for the runtime, not a device address; the address a kernel may use comes from
// cudaGetSymbolAddress, asked once per device with that device current (static_scratch_for_current_device).
//
// Every call on a device shares the one array, which keeps whatever the previous call left: the words
// that must start at zero (arrival counters, status) are cleared on the caller's stream before each
// launch; the partial-sum slots need no clearing because every slot is written before it is read.
// Two calls whose kernels overlap on the GPU (different streams, no dependency) would use the same
// slots and counters at once and corrupt each other: callers must order them.
constexpr size_t kStaticSlots = 256;                          // partial-sum slots of 256 columns x 32 rows fp32
constexpr size_t kStaticSlotBytes = size_t(256) * 32 * 4;     // 32 KiB
constexpr size_t kStaticCounters = 1024;                      // 4 per 256-column tile: N <= 65536
constexpr size_t kStaticHeaderBytes = 256 + kStaticCounters * sizeof(unsigned int);  // status word, counters
constexpr size_t kStaticScratchBytes = kStaticHeaderBytes + kStaticSlots * kStaticSlotBytes;  // 8 MiB + 4.25 KiB

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

struct StaticDeviceState {
    bool ready = false;
    unsigned char *scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
    EncodeTiledFn encode = nullptr;
};
constexpr int kMaxStaticDevices = 64;
StaticDeviceState g_static_state[kMaxStaticDevices];
std::mutex g_static_mutex;

void put_error(char *errbuf, size_t errbuf_len, const std::string &msg)
{
    if (errbuf && errbuf_len > 0) {
        const size_t n = msg.size() < errbuf_len - 1 ? msg.size() : errbuf_len - 1;
        memcpy(errbuf, msg.data(), n);
        errbuf[n] = '\0';
    }
}

// One-time set-up for the CURRENT device: resolve the device address of the scratch array, the SM count,
// the tensor-map encoder and the kernel's shared-memory limit.  Allocates nothing.
maize_status_t static_scratch_for_current_device(StaticDeviceState **out, char *errbuf, size_t errbuf_len)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0) {
        cudaGetLastError();
        put_error(errbuf, errbuf_len, "no current CUDA device");
        return MAIZE_ERR_NO_DEVICE;
    }
    if (dev >= kMaxStaticDevices) {
        put_error(errbuf, errbuf_len, "device ordinal beyond the table of the allocation-free entry point");
        return MAIZE_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticDeviceState &st = g_static_state[dev];
    if (!st.ready) {
        cudaDeviceProp prop;
        if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) {
            put_error(errbuf, errbuf_len, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
            return MAIZE_ERR_CUDA;
        }
        if (prop.major != 10) {
            put_error(errbuf, errbuf_len, "the kernels are built for sm_100a only");
            return MAIZE_ERR_UNSUPPORTED;
        }
        void *addr = nullptr;
        // The symbol's name is a host-side stand-in; this asks the runtime where the array lives on THIS device.
        if ((e = cudaGetSymbolAddress(&addr, g_static_scratch)) != cudaSuccess || !addr) {
            put_error(errbuf, errbuf_len, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
            return MAIZE_ERR_CUDA;
        }
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            put_error(errbuf, errbuf_len, "cuTensorMapEncodeTiled is not available from this driver");
            return MAIZE_ERR_CUDA;
        }
        e = cudaFuncSetAttribute(maize::gemm_bf16_sm100_skinny<true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 maize::SkinnySmemLayout<4>::kDynamicBytes);
        if (e != cudaSuccess) {
            put_error(errbuf, errbuf_len, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
            return MAIZE_ERR_CUDA;
        }
        st.scratch = static_cast<unsigned char *>(addr);
        st.sm_count = prop.multiProcessorCount;
        st.encode = reinterpret_cast<EncodeTiledFn>(fn);
        st.ready = true;
    }
    *out = &st;
    return MAIZE_OK;
}

bool encode_static_map(const StaticDeviceState &st, CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                       uint32_t box_rows)
{
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 2};
    cuuint32_t box[2] = {maize::kBlockK, box_rows};
    cuuint32_t estride[2] = {1, 1};
    return st.encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estride,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" maize_status_t maize_gemm_bf16_skinny_static(const void *a, uint32_t a_rows, uint32_t a_cols, const void *b,
                                                        uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows,
                                                        uint32_t c_cols, void *cuda_stream, void *device_status,
                                                        char *errbuf, size_t errbuf_len)
{
    put_error(errbuf, errbuf_len, "");
    if (a_cols != b_cols || c_rows != a_rows || c_cols != b_rows) {
        put_error(errbuf, errbuf_len, "shapes do not agree: A is M x K, B is N x K, C is M x N");
        return MAIZE_ERR_INVALID_ARG;
    }
    const uint32_t m = a_rows, n = b_rows, k = a_cols;
    if (m == 0 || n == 0)
        return MAIZE_OK;
    if (!c) {
        put_error(errbuf, errbuf_len, "C pointer is null");
        return MAIZE_ERR_INVALID_ARG;
    }
    if (k == 0) {
        // empty sum, as in maize_gemm_bf16: C = 0 (a memset on the caller's stream allocates nothing)
        cudaError_t ez = cudaMemsetAsync(c, 0, size_t(m) * n * 2, static_cast<cudaStream_t>(cuda_stream));
        if (ez != cudaSuccess) {
            put_error(errbuf, errbuf_len, std::string("cudaMemsetAsync: ") + cudaGetErrorString(ez));
            return MAIZE_ERR_CUDA;
        }
        return MAIZE_OK;
    }
    if (!a || !b) {
        put_error(errbuf, errbuf_len, "A or B pointer is null");
        return MAIZE_ERR_INVALID_ARG;
    }
    if (m > 32) {
        put_error(errbuf, errbuf_len, "the allocation-free entry point takes at most 32 rows of A (M <= 32)");
        return MAIZE_ERR_UNSUPPORTED;
    }
    if (k % 8 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(c) % 2 != 0 || reinterpret_cast<uintptr_t>(device_status) % 4 != 0) {
        put_error(errbuf, errbuf_len, "K must be a multiple of 8, A and B 16-byte aligned, C 2-byte aligned");
        return MAIZE_ERR_UNSUPPORTED;
    }
    StaticDeviceState *st = nullptr;
    maize_status_t rc = static_scratch_for_current_device(&st, errbuf, errbuf_len);
    if (rc != MAIZE_OK)
        return rc;

    maize::SkinnyParams sp;
    sp.tiles_n = (n + maize::kSkinnyTileN - 1) / maize::kSkinnyTileN;
    sp.num_kb = (k + maize::kBlockK - 1) / maize::kBlockK;
    const uint64_t units = uint64_t(sp.tiles_n) * sp.num_kb;
    const uint64_t cap = static_cast<uint64_t>(st->sm_count);
    uint64_t q = (units + cap - 1) / cap;
    const uint64_t min_q = sp.num_kb < 8 ? sp.num_kb : 8;
    if (q < min_q)
        q = min_q;
    const uint64_t parts = (q % sp.num_kb == 0) ? 1 : (sp.num_kb - 1 + q - 1) / q + 1;
    const uint64_t slots = parts == 1 ? 0 : uint64_t(sp.tiles_n) * parts;
    if (slots > kStaticSlots || uint64_t(sp.tiles_n) * 4 > kStaticCounters || q > 0xffffffffull) {
        char msg[200];
        snprintf(msg, sizeof msg,
                 "problem needs %llu partial-sum slots and %llu counters; the static scratch holds %llu and %llu "
                 "(use maize_gemm_bf16 with a context for larger N x K)",
                 (unsigned long long)slots, (unsigned long long)(uint64_t(sp.tiles_n) * 4),
                 (unsigned long long)kStaticSlots, (unsigned long long)kStaticCounters);
        put_error(errbuf, errbuf_len, msg);
        return MAIZE_ERR_UNSUPPORTED;
    }
    CUtensorMap tx, tw;
    if (!encode_static_map(*st, &tx, a, m, k, 32) || !encode_static_map(*st, &tw, b, n, k, maize::kSkinnyTileN)) {
        put_error(errbuf, errbuf_len, "cuTensorMapEncodeTiled rejected the operands");
        return MAIZE_ERR_CUDA;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    // Counters (and the library's own status word) must start at zero; the previous call, or one that gave
    // up on a wait, may have left them otherwise.  A memset on the caller's stream allocates nothing.
    cudaError_t e = cudaMemsetAsync(st->scratch, 0, kStaticHeaderBytes, stream);
    if (e != cudaSuccess) {
        put_error(errbuf, errbuf_len, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
        return MAIZE_ERR_CUDA;
    }
    sp.g.c = static_cast<__nv_bfloat16 *>(c);
    sp.g.ldc = n;
    sp.g.m = m;
    sp.g.n = n;
    sp.g.k = k;
    sp.g.tiles_m = 1;
    sp.g.tiles_n = 0;
    sp.g.group_m = 1;
    sp.g.c_vec_ok = (n % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1u : 0u;
    sp.g.status = device_status ? static_cast<DeviceStatus *>(device_status)
                                : reinterpret_cast<DeviceStatus *>(st->scratch);
    sp.g.timeout_ns = 2000000000ull;
    sp.g.profile = nullptr;
    sp.g.debug_flags = 0;
    sp.units_per_cta = static_cast<uint32_t>(q);
    sp.max_parts = static_cast<uint32_t>(parts);
    sp.counters = reinterpret_cast<unsigned int *>(st->scratch + 256);
    sp.partials = reinterpret_cast<float *>(st->scratch + kStaticHeaderBytes);
    const uint32_t grid = static_cast<uint32_t>((units + q - 1) / q);
    maize::gemm_bf16_sm100_skinny<true, 4>
        <<<grid, maize::kNumThreads, maize::SkinnySmemLayout<4>::kDynamicBytes, stream>>>(tx, tw, sp);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        put_error(errbuf, errbuf_len, std::string("kernel launch: ") + cudaGetErrorString(e));
        return MAIZE_ERR_CUDA;
    }
    return MAIZE_OK;
}
