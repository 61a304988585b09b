/*
 * maize_gemm.h - C ABI of the B200-native BF16 GEMM that stands in for the one
 * hot path of averyparr/maize: the pipelined tiled BF16 GEMM its demo traces.
 *
 * The reference has no runtime boundary for this path (it prints PTX), so each
 * entry point cites the reference interface whose role it takes over:
 *
 *   - the kernel argument list (A ptr, a_rows, a_cols, B ptr, b_rows, b_cols)
 *     of the traced GEMM kernel                             src/main.rs:32-39
 *   - the {ptr, nrows, ncols} argument bundle GlobalMatrix  src/main.rs:20-27
 *     and maize_tile::gmem::Matrix      crates/maize_tile/src/gmem/matrix.rs:13-18
 *   - the per-tile GEMM entry point sm80_gemm_smem_multibuffer
 *                                       crates/maize_tile/src/gemm/mod.rs:37-90
 *
 * Data contract (all entry points): bf16 operands, fp32 accumulation starting at
 * zero, one round-to-nearest-even conversion to bf16 on output.
 *   A : M x K, row-major                     (a_rows = M, a_cols = K)
 *   B : N x K, row-major, i.e. K-major       (b_rows = N, b_cols = K)
 *   C : M x N, row-major,  C = A * B^T       (c_rows = M, c_cols = N)
 * Ragged M, N and K are handled (the reference drops ragged panels,
 * src/main.rs:56-57).  Requirements of the TMA loads: K % 8 == 0 (16-byte row
 * pitch), A and B base addresses 16-byte aligned; otherwise
 * MAIZE_ERR_UNSUPPORTED is returned and nothing is launched.  C needs only
 * 2-byte alignment and any N.
 *
 * Every call enqueues work on the caller's CUDA stream and returns without
 * synchronising; no call allocates device memory except maize_ctx_create,
 * maize_ctx_set("profile" / "repack_bytes") and the *_host entry point (which
 * waits for the stream, frees and re-allocates its cached staging area whenever
 * a call needs more than the last one did, and waits for C before it returns).
 * Nothing here ever traps or asserts on the device: a device wait that runs
 * out of its time budget records MAIZE_ERR_TIMEOUT in a status word that
 * maize_ctx_poll reads back.
 *
 * Plain C: no CUDA or torch types appear in any signature; streams travel as
 * void* (a cudaStream_t / CUstream value, NULL = the legacy default stream).
 */
#ifndef MAIZE_GEMM_H
#define MAIZE_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MAIZE_API __attribute__((visibility("default")))
#else
#define MAIZE_API
#endif

typedef enum maize_status {
    MAIZE_OK = 0,
    MAIZE_ERR_INVALID_ARG = 1,  /* null pointer, mismatched shapes, bad leading dimension */
    MAIZE_ERR_UNSUPPORTED = 2,  /* K % 8 != 0, misaligned A/B, dimension beyond the kernel's range */
    MAIZE_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed; see maize_last_error */
    MAIZE_ERR_TIMEOUT = 4,      /* a bounded device wait expired (reported by maize_ctx_poll) */
    MAIZE_ERR_DEVICE_ABORT = 5, /* the kernel saw an inconsistent state and returned early */
    MAIZE_ERR_NO_DEVICE = 6     /* no usable CUDA device / driver */
} maize_status_t;

/* {ptr, nrows, ncols}: mirrors GlobalMatrix<T> (src/main.rs:20-27), 16 bytes, 16-byte aligned. */
typedef struct
#if defined(__GNUC__)
    __attribute__((aligned(16)))
#endif
    maize_global_matrix {
    void *ptr;      /* device pointer to bf16 elements, row-major, dense rows */
    uint32_t nrows;
    uint32_t ncols;
} maize_global_matrix_t;

typedef struct maize_ctx maize_ctx_t;

/* Library version, major * 10000 + minor * 100 + patch. */
MAIZE_API int maize_version(void);

/* Static text for a status code. */
MAIZE_API const char *maize_status_string(maize_status_t status);

/*
 * One context per host thread / stream.  Binds to `device`, queries its SM
 * count, and allocates the small device-side state the kernels need (status
 * word, split-K scratch).  Takes the role of the per-thread kernel builder of
 * the reference (crates/maize_core/src/codegen/mod.rs:21-26, 50-51).
 */
MAIZE_API maize_status_t maize_ctx_create(int device, maize_ctx_t **out);
MAIZE_API void maize_ctx_destroy(maize_ctx_t *ctx);

/* Last error text of this context ("" if none); valid until the next call on ctx. */
MAIZE_API const char *maize_last_error(const maize_ctx_t *ctx);

/*
 * C = A * B^T on device buffers; argument order follows the traced kernel's
 * (ptr, rows, cols) triples (src/main.rs:32-39) plus the C triple that the
 * reference never stores (src/main.rs:71).  Requires a_cols == b_cols,
 * c_rows == a_rows, c_cols == b_rows.  M == 0 or N == 0 is a no-op.
 */
MAIZE_API maize_status_t maize_gemm_bf16(maize_ctx_t *ctx, const void *a, uint32_t a_rows, uint32_t a_cols,
                                         const void *b, uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows,
                                         uint32_t c_cols, void *cuda_stream);

/* Same through the {ptr, nrows, ncols} bundles (src/main.rs:20-27). */
MAIZE_API maize_status_t maize_gemm_bf16_m(maize_ctx_t *ctx, const maize_global_matrix_t *a,
                                           const maize_global_matrix_t *b, const maize_global_matrix_t *c,
                                           void *cuda_stream);

/*
 * Same with explicit leading dimensions in elements (row pitch of A, B and C):
 * the stride_per_row of the reference's panels
 * (crates/maize_tile/src/gmem/col_panel.rs:88-124, row_panel.rs:85-127).
 * lda and ldb must be multiples of 8; ldc is free.  Used for row slabs of A/C
 * and column slices of C in the N-sharded multi-GPU path.
 */
MAIZE_API maize_status_t maize_gemm_bf16_ld(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b,
                                            uint64_t ldb, void *c, uint64_t ldc, uint32_t m, uint32_t n, uint32_t k,
                                            void *cuda_stream);

/*
 * C = A * B with B stored K x N row-major (N contiguous): the layout the reference's demo walks,
 * 16-column panels of a row-major matrix stepping 16 rows per k-step
 * (crates/maize_tile/src/gmem/col_panel.rs:88-124, gmem_tile.rs:416-432, src/main.rs:57).
 * a_cols == b_rows (= K), c is a_rows x b_cols.  Requires b_cols (ldb) % 8 == 0 and a_cols (lda) % 8 == 0,
 * 16-byte aligned A and B; K itself may be any value.  B's tiles are loaded as 64-column boxes and fed
 * to the tensor core as an MN-major operand; nothing is transposed in memory.  Decode shapes (M <= 128) run on
 * the pair-split kernels with tiles widened to a multiple of 64 columns; the stream-K kernels take N x K only.
 */
MAIZE_API maize_status_t maize_gemm_bf16_kn(maize_ctx_t *ctx, const void *a, uint32_t a_rows, uint32_t a_cols,
                                            const void *b, uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows,
                                            uint32_t c_cols, void *cuda_stream);
MAIZE_API maize_status_t maize_gemm_bf16_kn_ld(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b,
                                               uint64_t ldb, void *c, uint64_t ldc, uint32_t m, uint32_t n,
                                               uint32_t k, void *cuda_stream);

/*
 * End-to-end form with HOST buffers (pinned or pageable): copies A and B to the
 * device, runs the GEMM, copies C back, ordered after the earlier work of
 * `cuda_stream`, and waits for the result.  Large problems are pipelined: B first,
 * then A in row slabs whose GEMMs and C read-backs overlap the following uploads
 * (two helper streams of the context).  Device staging is cached in the context and
 * grows on demand.  With "b_static" set, a call that passes the same b_host, b_rows and
 * b_cols as the previous one re-uses the copy of B that is still on the device.
 * Stands where a host caller of the traced kernel (src/main.rs:31-90) would.
 */
MAIZE_API maize_status_t maize_gemm_bf16_host(maize_ctx_t *ctx, const void *a_host, uint32_t a_rows, uint32_t a_cols,
                                              const void *b_host, uint32_t b_rows, uint32_t b_cols, void *c_host,
                                              uint32_t c_rows, uint32_t c_cols, void *cuda_stream);

/*
 * Synchronises `cuda_stream`, reads and clears the device status word.
 * MAIZE_OK, MAIZE_ERR_TIMEOUT or MAIZE_ERR_DEVICE_ABORT; replaces the
 * reference's device-side trap (src/main.rs:54,71).
 */
MAIZE_API maize_status_t maize_ctx_poll(maize_ctx_t *ctx, void *cuda_stream);

/* Tunables.  Keys: "timeout_ns" (device wait budget), "force_kernel" (0 = heuristic,
 * see maize_kernel_name), "max_ctas" (cap on the persistent grid, 0 = SM count),
 * "profile" (1 = per-CTA cycle accounting, see maize_ctx_read_profile), "group_rows" (rows of A
 * whose tiles are scheduled together; default 0 = by kernel: 2048, and 4096 for the 256 x 512 tile), "push_threads" (threads per CTA of the copy
 * kernels of the multi-GPU path, default 512), "pdl" (default 1: the GEMM kernels are launched with
 * programmatic stream serialization, so that a kernel's set-up (barriers, tensor memory, descriptor
 * prefetch) runs while the stream's previous kernel drains; the kernel waits for that kernel to complete
 * before it touches A, B or C, so stream order is kept; 0 = ordinary launches), "b_static" (1 = the
 * caller guarantees that no earlier work of the stream writes B, e.g. inference weights; with "pdl" the
 * decode kernel then fetches its first B tiles before waiting for that earlier work, the host-buffer entry
 * point keeps B on the device between calls, and the pitch-aligning pre-pass keeps its copy of B),
 * "serpentine" (default 1: every other group of row-blocks sweeps the column-blocks backwards, so that it
 * starts on the panels of B the previous group left in L2), "tail_split" (default 1: when the last round
 * of 256 x 256 tiles would leave CTA pairs idle, its tiles are split along K over them), "tma_store"
 * (default 1: the CTA-pair kernels write C through shared memory and TMA stores when C's rows are 16-byte
 * aligned), "c_evict_first" (default 1: those stores carry an evict-first L2 hint, C passes through L2 once),
 * "wide_tile" (default 1: GEMMs with long K, rounds of tiles at least 86 % full and 16-byte aligned rows of
 * C use a 256 x 512 tile per CTA pair, which moves a quarter less data from L2 per flop; "wide_max_gflop", default 1000000, is the largest
 * 2MNK / 1e9 that takes it: multi-millisecond GEMMs run back to back for seconds are 1-3 % faster on the 256 x 256
 * tile), "tma_promotion" (L2 promotion of the operand tensor maps: 0 none, 1 64 B, 2 128 B, 3 256 B
 * = default), "chain_streams"
 * (1 to 4, default 2: streams that maize_chain_forward deals its chunks over), "chain_stagger"
 * (default 1: when the source is all there, as on the root, the streams start a fraction of a chunk apart,
 * so that they never publish at the same time and the link never idles), "repack_bytes" (size of an
 * optional scratch, allocated by this call, into which operands whose row pitch is not a multiple of 128
 * bytes are copied with an aligned pitch ahead of a large GEMM; 0 frees it), "debug_flags"
 * (performance diagnostics that make results WRONG: 1 = all loads hit one tile, 2 = no loads; refused
 * unless "profile" is 1, cleared when "profile" returns to 0). */
/* An environment variable MAIZE_<KEY> (upper case, e.g. MAIZE_PDL=0, MAIZE_TMA_STORE=0) presets that tunable in
 * every context created afterwards; maize_ctx_set still overrides it. */
MAIZE_API maize_status_t maize_ctx_set(maize_ctx_t *ctx, const char *key, int64_t value);
/* Reads back any key of maize_ctx_set, plus "sm_count", "device" and "last_kernel" (id, as maize_kernel_name
 * takes it, of the GEMM kernel the context's last call launched; 0 before the first). */
MAIZE_API maize_status_t maize_ctx_get(const maize_ctx_t *ctx, const char *key, int64_t *value);

/* Name of kernel variant `id` (1-based), NULL past the end; id of the variant the
 * heuristic picks for a shape of densely stored, aligned operands.  A call may still run another one: a K x N
 * matrix B, a gated launch, or rows of C that TMA cannot store keep the 256 x 256 tile where the shape alone would
 * take the 256 x 512 one ("last_kernel" tells). */
MAIZE_API const char *maize_kernel_name(int id);
MAIZE_API int maize_pick_kernel(const maize_ctx_t *ctx, uint32_t m, uint32_t n, uint32_t k);

/* Number of kernels this context has launched since creation. */
MAIZE_API uint64_t maize_ctx_launch_count(const maize_ctx_t *ctx);

/*
 * Debugging aid with no counterpart in the reference: after maize_ctx_set(ctx, "profile", 1)
 * every GEMM launch records, per CTA, 8 cycle counters (producer blocked on a free stage, MMA
 * blocked on data, MMA blocked on a free accumulator, epilogue blocked on a finished
 * accumulator, epilogue draining, CTA lifetime, tiles done, spare).  Copies the counters of
 * the last launch (8 * CTAs values) to `out` after synchronising the stream; returns the
 * number of CTAs written (at most max_ctas).
 */
MAIZE_API int maize_ctx_read_profile(maize_ctx_t *ctx, uint64_t *out, int max_ctas, void *cuda_stream);

/*
 * Building blocks of the N-sharded multi-GPU path (the reference has none; they serve the
 * split of B's column panels, crates/maize_tile/src/gmem/col_panel.rs:88-124, across GPUs).
 *
 * maize_mc_push: copy `bytes` from local device memory `src` to EVERY GPU's replica of a
 * symmetric buffer through its NVSwitch multicast address `mc_dst` (multimem.st), then publish
 * `flag_value` in the 32-bit word at multicast address `mc_flag` on every GPU.  16-byte aligned
 * pointers and size.  `ctas` = CTAs of the push kernel (0 = default 16).  One push at a time per
 * context.
 * maize_mc_push_after: the same, but the kernel first waits (bounded) until the local word
 * `wait_flag` has reached `wait_value`: for a source that another GPU is still filling.
 * maize_scatter_push (root): split `bytes` of `src` into `world` equal chunks (16-byte units) and
 * store chunk p into `peer_dst[p]` + its offset (peer-mapped landing buffer of rank p, given at
 * the slab's base), then publish `flag_value` in `peer_flag[p]`; the root's own chunk is skipped.
 * `peer_dst` / `peer_flag` are host arrays of `world` device pointers.
 * maize_flags_wait: enqueue a bounded device-side wait until each of `count` (<= 32) consecutive
 * 32-bit words at `flags` (local memory, written by peers) has reached `value` (values only grow;
 * wrap-around safe).  An expired wait is reported by maize_ctx_poll as MAIZE_ERR_TIMEOUT.
 * maize_flag_store: enqueue a system-scope release store of `value` to `flag`, which may be a
 * peer-mapped address, ordered after the stream's earlier work.
 */
MAIZE_API maize_status_t maize_mc_push(maize_ctx_t *ctx, const void *src, void *mc_dst, uint64_t bytes, void *mc_flag,
                                       uint32_t flag_value, int ctas, void *cuda_stream);
MAIZE_API maize_status_t maize_mc_push_after(maize_ctx_t *ctx, const void *wait_flag, uint32_t wait_value,
                                             const void *src, void *mc_dst, uint64_t bytes, void *mc_flag,
                                             uint32_t flag_value, int ctas, void *cuda_stream);
MAIZE_API maize_status_t maize_scatter_push(maize_ctx_t *ctx, const void *src, void *const *peer_dst,
                                            void *const *peer_flag, uint32_t world, uint32_t root, uint64_t bytes,
                                            uint32_t flag_value, int ctas, void *cuda_stream);
/* Enqueue a device-to-device copy (copy engines; `dst` may be a peer-mapped address: the bytes then cross
 * NVLink without any SM taking part).  Building block of the "chain" transport of the N-sharded path. */
MAIZE_API maize_status_t maize_copy_async(maize_ctx_t *ctx, void *dst, const void *src, uint64_t bytes,
                                          void *cuda_stream);
/* C = A * B^T like maize_gemm_bf16_ld, for an A whose rows are still arriving IN ROW ORDER while the kernel runs
 * (the receiving ranks of the N-sharded multi-GPU path: one launch per step instead of one per row slab).
 * Whoever delivers A counts chunks of `rows_per_count` rows in the 32-bit word `rows_landed` (this GPU's memory, a
 * peer-mapped address or mapped host memory), storing it with release semantics after the chunk's bytes: rows
 * [0, r) of A are read only once (int32)(*rows_landed - landed_base) >= ceil(r / rows_per_count).  Tiles are visited
 * in ascending groups of rows (see "group_rows"), each CTA's loader waits for its tile's rows, and the wait is
 * bounded like every other: if the count does not arrive within "timeout_ns" the kernel ends and
 * maize_ctx_poll returns MAIZE_ERR_TIMEOUT (C is then incomplete).  Decode-shaped problems run on the tiled
 * kernels here.  No reference counterpart (the reference is single-GPU: its GEMM entry point, crates/maize_tile/src/gemm/mod.rs:37-55, takes one
 * device's panels). */
MAIZE_API maize_status_t maize_gemm_bf16_gated(maize_ctx_t *ctx, const void *a, uint64_t lda, const void *b,
                                               uint64_t ldb, void *c, uint64_t ldc, uint32_t m, uint32_t n, uint32_t k,
                                               const void *rows_landed, uint32_t landed_base, uint32_t rows_per_count,
                                               void *cuda_stream);
/* One step of a rank's part in the chain: cut `total_bytes` at `src` into chunks of `chunk_bytes`; for chunk i
 * (i = 0, 1, ...) wait (bounded, if `wait_flag` is not NULL) until the local word `wait_flag` has reached
 * first_value + i, copy the chunk to `dst` + its offset (copy engines; `dst` is the next rank's landing buffer
 * through its peer mapping), then store first_value + i in `dst_flag` (the next rank's "chunks landed" word).
 * Everything is enqueued in one call, on `cuda_stream` and, with "chain_streams" > 1, round robin on helper
 * streams of the context that fork from and join `cuda_stream` (counts are still published in chunk order). */
MAIZE_API maize_status_t maize_chain_forward(maize_ctx_t *ctx, const void *wait_flag, uint32_t first_value, void *dst,
                                             const void *src, uint64_t total_bytes, uint64_t chunk_bytes,
                                             void *dst_flag, void *cuda_stream);
MAIZE_API maize_status_t maize_flags_wait(maize_ctx_t *ctx, const void *flags, uint32_t count, uint32_t value,
                                          void *cuda_stream);
MAIZE_API maize_status_t maize_flag_store(maize_ctx_t *ctx, void *flag, uint32_t value, void *cuda_stream);

/*
 * The N-sharded multi-GPU GEMM for ONE host process that drives several GPUs of a box.  The reference is
 * single-GPU; a caller that binds where its GEMM entry point sits (crates/maize_tile/src/gemm/mod.rs:37-55) gets
 * the split of B's column panels (crates/maize_tile/src/gmem/col_panel.rs:88-124) across GPUs from these.
 *
 * maize_mgpu_create: `devices` lists n distinct CUDA device ordinals (1 <= n <= 16) with peer access between
 * them.  Creates one context, two streams and a small flag buffer per device, enables peer access and starts
 * one host thread per device (each enqueues its own device's part of a call).
 *
 * maize_gemm_bf16_nsharded: C[:, shard g] = A * B[shard g]^T on every device g, A living on device index `root`
 * before the call.  Shard g = rows [first, end) of B as maize_mgpu_shard reports them (near-equal contiguous
 * blocks, the larger ones first).  Arrays are indexed like `devices`:
 *   a_on_root   M x K on device `root`, dense rows
 *   a_local[g]  M x K landing buffer on device g (entry `root` is ignored and may be NULL)
 *   b_shards[g] (end - first) x K on device g, dense rows;  c_shards[g]  M x (end - first) on device g, dense rows
 * A is forwarded along the chain root, root+1, ... (index order, wrapping) in chunks of "chunk_rows" rows with
 * device-to-device copies; the root runs one GEMM launch, every other device one gated launch
 * (maize_gemm_bf16_gated).  The call returns when everything is enqueued on the handle's own streams (it first
 * waits, on the host, for the call before the previous one to have finished, so at most two calls are in flight);
 * maize_mgpu_sync waits for all devices and reports a device-side timeout like maize_ctx_poll.  The buffers of a
 * call must stay untouched until then, except that the next call may follow at once: it orders itself after the
 * previous one (a landing buffer is only overwritten after the device that owns it has finished reading it).
 * By default the forwarding waits for what device `root`'s stream (maize_mgpu_stream) holds when the call is
 * made, so work that produces A may be enqueued there; maize_mgpu_set("a_on_stream", 0) declares that A is
 * complete in memory when the call is made, which lets the forwarding of a call overlap the previous call's GEMMs.
 *
 * maize_gemm_bf16_nsharded_host: the same from HOST buffers (A M x K, B N x K, C M x N dense): copies A to the
 * root and each device's rows of B up, runs the sharded GEMM, copies every device's column block into the dense
 * C and waits.  Device staging is cached in the handle and grows on demand.
 *
 * maize_mgpu_set: "chunk_rows" (multiple of 256, default 2048), "a_on_stream" (default 1); any other key is
 * passed to every device's context (maize_ctx_set).
 */
typedef struct maize_mgpu maize_mgpu_t;
MAIZE_API maize_status_t maize_mgpu_create(int n, const int *devices, maize_mgpu_t **out);
MAIZE_API void maize_mgpu_destroy(maize_mgpu_t *mg);
MAIZE_API const char *maize_mgpu_last_error(const maize_mgpu_t *mg);
MAIZE_API int maize_mgpu_size(const maize_mgpu_t *mg);
/* The stream (a cudaStream_t) on which device `index`'s GEMMs of this handle run. */
MAIZE_API void *maize_mgpu_stream(const maize_mgpu_t *mg, int index);
MAIZE_API maize_status_t maize_mgpu_shard(const maize_mgpu_t *mg, uint32_t n_rows, int index, uint32_t *first,
                                          uint32_t *end);
MAIZE_API maize_status_t maize_mgpu_set(maize_mgpu_t *mg, const char *key, int64_t value);
MAIZE_API maize_status_t maize_gemm_bf16_nsharded(maize_mgpu_t *mg, int root, const void *a_on_root, uint32_t m,
                                                  uint32_t k, void *const *a_local, const void *const *b_shards,
                                                  uint32_t n, void *const *c_shards);
MAIZE_API maize_status_t maize_gemm_bf16_nsharded_host(maize_mgpu_t *mg, int root, const void *a_host, uint32_t m,
                                                       uint32_t k, const void *b_host, uint32_t n, void *c_host);
MAIZE_API maize_status_t maize_mgpu_sync(maize_mgpu_t *mg);

/*
 * Self-test of the bounded-wait machinery: launches one CTA that waits on a
 * barrier nothing will ever complete, with a budget of `budget_ns`.  The kernel
 * returns by itself; the following maize_ctx_poll reports MAIZE_ERR_TIMEOUT.
 */
MAIZE_API maize_status_t maize_debug_wait_expires(maize_ctx_t *ctx, uint64_t budget_ns, void *cuda_stream);

/*
 * Allocation-free form of the skinny (M <= 32) GEMM.  It has no counterpart in the reference.
 *
 * For callers that must not allocate device memory where the GEMM is needed: services with a
 * "no cudaMalloc after start-up" rule (everything reserved up front, so a late allocation can
 * neither fail nor stall the device) and plugins whose host owns all device memory and hands out
 * only the operand buffers.  It takes no context (creating one allocates).  The stream-K scratch of
 * the kernel is a fixed array inside the library image: 8 MiB + 4.25 KiB on EVERY GPU that loads the
 * library, held until the process exits.  It calls no cudaMalloc, cudaFree or allocating library
 * routine.
 *
 * C = A * B^T as in maize_gemm_bf16, dense rows, on the CURRENT device (the one that owns a, b, c and
 * the stream).  Limits: M <= 32; N <= 65536; the split of the work over the SMs must need at most
 * 256 partial-sum slots (for example 16 x 16384 x 4096 needs exactly 256); K % 8 == 0, A and B
 * 16-byte aligned.  Anything beyond is refused with MAIZE_ERR_UNSUPPORTED and a message in `errbuf`
 * that states what was needed and what the scratch holds; use maize_gemm_bf16 with a context then.
 *
 * The FIRST call on each device is a start-up step: it looks up the array's device address, the SM count
 * and the tensor-map encoder and sets the kernel's shared-memory limit, and if the library's GPU code has not
 * been loaded on that device yet, the CUDA runtime loads it then, which is when the driver reserves the array
 * (and may fail for lack of memory).  Make that first call at start-up, before any stream capture; only the
 * calls after it are free of allocation.  K == 0 sets C to zero, as in maize_gemm_bf16.
 * Every call on a device uses the same array and finds what the previous call left there: the
 * counters and the status word are cleared on `cuda_stream` before each launch.  Calls whose kernels
 * could overlap on the GPU (different streams without a dependency) race on the array: order them.
 *
 * `device_status`: optional 16-byte device buffer (4-byte aligned, zero it yourself) that receives
 * MAIZE_ERR_TIMEOUT in its first word if a bounded device wait expires; NULL = not reported.
 * `errbuf` / `errbuf_len`: optional host buffer for the error text.
 */
MAIZE_API maize_status_t maize_gemm_bf16_skinny_static(const void *a, uint32_t a_rows, uint32_t a_cols, const void *b,
                                                       uint32_t b_rows, uint32_t b_cols, void *c, uint32_t c_rows,
                                                       uint32_t c_cols, void *cuda_stream, void *device_status,
                                                       char *errbuf, size_t errbuf_len);

#ifdef __cplusplus
}
#endif
#endif /* MAIZE_GEMM_H */
