/*
 * CPU oracle for the BF16 GEMM hot path.  TEST INFRASTRUCTURE ONLY: nothing in
 * the shipped library or the Python package links, imports or calls this file.
 * It is the checker for the CUDA path and the timed CPU baseline of the bench.
 *
 * PARITY UNPINNED: the reference (averyparr/maize) holds no CPU matmul, no
 * numeric test and no golden vector for this path, and it cannot be built here
 * (Rust + LLVM, neither installed).  This file restates the numeric contract the
 * reference's GEMM is built on, not its (self-declared incorrect) data movement:
 *
 *   - operands are bf16            crates/maize_core/src/ty/raw.rs:23, ty/sized.rs:67
 *   - products accumulate in fp32  crates/maize_tile/src/mma/sm80.rs:136-160
 *                                  (mma.m16n8k16 ... f32.bf16.bf16.f32, CFrag = V<F32,4>)
 *   - the accumulator starts at 0  crates/maize_tile/src/mma/mod.rs:48-50
 *   - the k loop walks tiles in ascending k
 *                                  crates/maize_tile/src/gemm/mod.rs:66-87
 *   - one kernel argument triple (ptr, rows, cols) per matrix
 *                                  src/main.rs:32-39
 *
 *   C[m][n] = bf16_rne( sum_{k ascending} float(A[m][k]) * float(B[n][k]) )
 *
 * with A  M x K row-major, B  N x K row-major (K-major, so C = A * B^T) and
 * C  M x N row-major.  The sum is a plain fp32 running sum in ascending k, one
 * rounding per addition.  A bf16 x bf16 product is exact in fp32 (8+8 significand
 * bits), so fused and unfused multiply-add give the same bits and the result
 * does not depend on how the compiler vectorises across n.
 *
 * The file also holds the seeded input generator shared by every parity test,
 * so that the same bytes reach the oracle and the GPU.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_EXPORT __attribute__((visibility("default")))

/* ---------------------------------------------------------------- bf16 ---- */

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* Round-to-nearest-even fp32 -> bf16; NaN stays a quiet NaN. */
static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)
        return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

ORACLE_EXPORT uint16_t maize_oracle_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
ORACLE_EXPORT float maize_oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* ------------------------------------------------------- seeded inputs ---- */

static inline uint64_t splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* Uniform in (0,1), 53 bits, never 0 or 1. */
static inline double u01(uint64_t key, uint64_t counter)
{
    uint64_t x = splitmix64(key ^ splitmix64(counter));
    return ((double)(x >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}

enum { ORACLE_DIST_NORMAL = 0, ORACLE_DIST_UNIFORM = 1 };

/*
 * Fill out[0..count) with bf16 values of a counter-based stream keyed by
 * (seed, matrix_id): element i depends only on (seed, matrix_id, first + i), so
 * any slice of a matrix can be generated on its own.
 *   dist 0: N(0, scale^2) by Box-Muller;  dist 1: U(-scale, scale).
 */
ORACLE_EXPORT void maize_oracle_fill_bf16(uint64_t seed, uint32_t matrix_id, int dist, double scale,
                                          uint64_t first, uint64_t count, uint16_t *out)
{
    const uint64_t key = splitmix64(seed * 0x100000001B3ull + (uint64_t)matrix_id + 1u);
    const double two_pi = 6.283185307179586476925286766559;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        uint64_t idx = first + (uint64_t)i;
        double v;
        if (dist == ORACLE_DIST_UNIFORM) {
            v = (2.0 * u01(key, 2 * idx) - 1.0) * scale;
        } else {
            double u1 = u01(key, 2 * idx), u2 = u01(key, 2 * idx + 1);
            v = sqrt(-2.0 * log(u1)) * cos(two_pi * u2) * scale;
        }
        out[i] = f32_to_bf16_rne((float)v);
    }
}

/* ---------------------------------------------------------------- GEMM ---- */

#define NB 16 /* columns of C per packed B panel (one 512-bit vector of fp32) */
#define MB 8  /* rows of C per register block */

/*
 * acc[i][j] += a_rows[i][k] * bp[k][j] for k ascending: each (i, j) is an
 * independent strictly sequential fp32 sum; the compiler vectorises across j.
 */
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
static void block_kernel(int mb, uint32_t K, const float *a_rows /* MB x K */, const float *bp /* K x NB */,
                         float *acc /* MB x NB */)
{
    float r[MB][NB];
    for (int i = 0; i < MB; ++i)
        for (int j = 0; j < NB; ++j)
            r[i][j] = 0.0f;
    if (mb == MB) {
        for (uint32_t k = 0; k < K; ++k) {
            const float *b = bp + (size_t)k * NB;
            for (int i = 0; i < MB; ++i) {
                float a = a_rows[(size_t)i * K + k];
#pragma omp simd
                for (int j = 0; j < NB; ++j)
                    r[i][j] += a * b[j];
            }
        }
    } else {
        for (uint32_t k = 0; k < K; ++k) {
            const float *b = bp + (size_t)k * NB;
            for (int i = 0; i < mb; ++i) {
                float a = a_rows[(size_t)i * K + k];
#pragma omp simd
                for (int j = 0; j < NB; ++j)
                    r[i][j] += a * b[j];
            }
        }
    }
    for (int i = 0; i < MB; ++i)
        for (int j = 0; j < NB; ++j)
            acc[i * NB + j] = r[i][j];
}

/*
 * Shared driver.  c_bf16 and/or c_f32 may be NULL; c_f32 receives the fp32 sum
 * before the final rounding (for error analysis in the tests).
 * Leading dimensions are in elements.  Returns 0, or -1 on a bad argument /
 * failed allocation.
 */
static int gemm_driver(const uint16_t *a, uint32_t M, uint32_t K, uint64_t lda, const uint16_t *b, uint32_t N,
                       uint64_t ldb, uint16_t *c_bf16, float *c_f32, uint64_t ldc, int nthreads)
{
    if (M == 0 || N == 0)
        return 0;
    if ((!a || !b) && K > 0)
        return -1;
    if (lda < K || ldb < K || ldc < N)
        return -1;
#ifdef _OPENMP
    if (nthreads <= 0)
        nthreads = omp_get_max_threads();
#else
    nthreads = 1;
#endif
    const uint32_t n_panels = (N + NB - 1) / NB;
    const uint32_t m_blocks = (M + MB - 1) / MB;

    /* A widened to fp32 once (row-major M x K, dense). */
    float *af = (float *)malloc(sizeof(float) * (size_t)M * (K ? K : 1));
    if (!af)
        return -1;
#pragma omp parallel for schedule(static) num_threads(nthreads)
    for (int64_t m = 0; m < (int64_t)M; ++m)
        for (uint32_t k = 0; k < K; ++k)
            af[(size_t)m * K + k] = bf16_to_f32(a[(size_t)m * lda + k]);

    int failed = 0;
#pragma omp parallel num_threads(nthreads)
    {
        float *bp = (float *)malloc(sizeof(float) * (size_t)(K ? K : 1) * NB);
        float acc[MB * NB];
        if (!bp) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t p = 0; p < (int64_t)n_panels; ++p) {
            if (!bp)
                continue;
            const uint32_t n0 = (uint32_t)p * NB;
            const uint32_t nb = (N - n0 < NB) ? (N - n0) : NB;
            /* pack B[n0..n0+nb) x K into K x NB fp32, zero for the ragged tail */
            for (uint32_t k = 0; k < K; ++k)
                for (uint32_t j = 0; j < NB; ++j)
                    bp[(size_t)k * NB + j] = (j < nb) ? bf16_to_f32(b[(size_t)(n0 + j) * ldb + k]) : 0.0f;
            for (uint32_t mblk = 0; mblk < m_blocks; ++mblk) {
                const uint32_t m0 = mblk * MB;
                const int mb = (int)((M - m0 < MB) ? (M - m0) : MB);
                block_kernel(mb, K, af + (size_t)m0 * K, bp, acc);
                for (int i = 0; i < mb; ++i)
                    for (uint32_t j = 0; j < nb; ++j) {
                        float v = acc[i * NB + j];
                        if (c_f32)
                            c_f32[(size_t)(m0 + i) * ldc + n0 + j] = v;
                        if (c_bf16)
                            c_bf16[(size_t)(m0 + i) * ldc + n0 + j] = f32_to_bf16_rne(v);
                    }
            }
        }
        free(bp);
    }
    free(af);
    return failed ? -1 : 0;
}

/* C (bf16) = A * B^T, fp32 ascending-k running sum, one RNE rounding at the end. */
ORACLE_EXPORT int maize_oracle_gemm_bf16(const uint16_t *a, uint32_t a_rows, uint32_t a_cols, const uint16_t *b,
                                         uint32_t b_rows, uint32_t b_cols, uint16_t *c, uint32_t c_rows,
                                         uint32_t c_cols, int nthreads)
{
    if (a_cols != b_cols || c_rows != a_rows || c_cols != b_rows)
        return -1;
    return gemm_driver(a, a_rows, a_cols, a_cols, b, b_rows, b_cols, c, NULL, c_cols, nthreads);
}

/* Same with explicit leading dimensions (elements). */
ORACLE_EXPORT int maize_oracle_gemm_bf16_ld(const uint16_t *a, uint64_t lda, const uint16_t *b, uint64_t ldb,
                                            uint16_t *c, uint64_t ldc, uint32_t M, uint32_t N, uint32_t K,
                                            int nthreads)
{
    return gemm_driver(a, M, K, lda, b, N, ldb, c, NULL, ldc, nthreads);
}

/* The unrounded fp32 sums (dense M x N). */
ORACLE_EXPORT int maize_oracle_gemm_f32out(const uint16_t *a, const uint16_t *b, float *c, uint32_t M, uint32_t N,
                                           uint32_t K, int nthreads)
{
    return gemm_driver(a, M, K, K, b, N, K, NULL, c, N, nthreads);
}

/* Textbook triple loop, no packing, no blocking: pins the blocked driver above. */
ORACLE_EXPORT void maize_oracle_gemm_naive(const uint16_t *a, const uint16_t *b, uint16_t *c, uint32_t M, uint32_t N,
                                           uint32_t K)
{
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t n = 0; n < N; ++n) {
            volatile float s = 0.0f; /* volatile: one rounding per step, no reassociation */
            for (uint32_t k = 0; k < K; ++k) {
                float p = bf16_to_f32(a[(size_t)m * K + k]) * bf16_to_f32(b[(size_t)n * K + k]);
                s = s + p;
            }
            c[(size_t)m * N + n] = f32_to_bf16_rne(s);
        }
}

/*
 * Acceptance check of the path's tolerance:
 *   |c - ref| <= 1e-2 * sqrt(K) * max|a| * max|b|  +  |ref| * 2^-7
 * (the second term is one bf16 ulp for the final rounding).  Writes the largest
 * absolute error, the bound's first term and the count of violations.
 */
ORACLE_EXPORT int maize_oracle_check(const uint16_t *c, uint64_t ldc, const uint16_t *ref, uint64_t ldref, uint32_t M,
                                     uint32_t N, uint32_t K, double max_abs_a, double max_abs_b, double *max_abs_err,
                                     double *bound, uint64_t *violations)
{
    const double base = 1e-2 * sqrt((double)K) * max_abs_a * max_abs_b;
    double worst = 0.0;
    uint64_t bad = 0;
#pragma omp parallel for reduction(max : worst) reduction(+ : bad) schedule(static)
    for (int64_t m = 0; m < (int64_t)M; ++m)
        for (uint32_t n = 0; n < N; ++n) {
            double g = bf16_to_f32(c[(size_t)m * ldc + n]);
            double r = bf16_to_f32(ref[(size_t)m * ldref + n]);
            double e = fabs(g - r);
            if (!(e <= base + fabs(r) * (1.0 / 128.0)))
                ++bad; /* also catches NaN */
            if (e > worst || e != e)
                worst = (e != e) ? INFINITY : e;
        }
    if (max_abs_err)
        *max_abs_err = worst;
    if (bound)
        *bound = base;
    if (violations)
        *violations = bad;
    return bad == 0 ? 0 : 1;
}

ORACLE_EXPORT double maize_oracle_max_abs_bf16(const uint16_t *x, uint64_t count)
{
    double worst = 0.0;
#pragma omp parallel for reduction(max : worst) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        double v = fabs((double)bf16_to_f32(x[i]));
        if (v > worst)
            worst = v;
    }
    return worst;
}

ORACLE_EXPORT int maize_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the thread count of every later parallel region of this library (fill, check, max-abs and the GEMMs
 * called with nthreads <= 0).  A launcher may have exported OMP_NUM_THREADS=1 for its children
 * (torch.distributed.run does); the timed CPU baseline then asks for the cores it may really use. */
ORACLE_EXPORT void maize_oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}
