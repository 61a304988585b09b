/*
 * A compiled-language caller of the C ABI: plain C11, no CUDA headers, no Python.
 * It links libmaize_gemm.so the way a maintainer of the reference would bind it from
 * Rust (the kernel argument list of src/main.rs:32-39 as (ptr, rows, cols) triples),
 * runs C = A * B^T on host buffers through maize_gemm_bf16_host and checks the result
 * against the CPU oracle (test infrastructure, linked here only as the checker).
 *
 *   harness M N K [seed]            exit 0: parity holds; 1: mismatch or error;
 *                                   77: no CUDA device (reported, nothing computed)
 *   harness --mgpu G M N K [seed]   the same through maize_gemm_bf16_nsharded_host on devices 0..G-1,
 *                                   twice with different A (the landing buffers are reused)
 *   harness --selftest              host-only checks that need no device
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "maize_gemm.h"

/* the oracle's exports used here (oracle/cpu_gemm.c) */
void maize_oracle_fill_bf16(uint64_t seed, uint32_t matrix_id, int dist, double scale, uint64_t first, uint64_t count,
                            uint16_t *out);
int maize_oracle_gemm_bf16(const uint16_t *a, uint32_t a_rows, uint32_t a_cols, const uint16_t *b, uint32_t b_rows,
                           uint32_t b_cols, uint16_t *c, uint32_t c_rows, uint32_t c_cols, int nthreads);
int maize_oracle_check(const uint16_t *c, uint64_t ldc, const uint16_t *ref, uint64_t ldref, uint32_t M, uint32_t N,
                       uint32_t K, double max_abs_a, double max_abs_b, double *max_abs_err, double *bound,
                       uint64_t *violations);
double maize_oracle_max_abs_bf16(const uint16_t *x, uint64_t count);

static int selftest(void)
{
    int bad = 0;
    /* no device is needed for any of these */
    if (maize_version() <= 0)
        ++bad;
    if (strcmp(maize_status_string(MAIZE_OK), "ok") != 0)
        ++bad;
    if (maize_kernel_name(0) != NULL || maize_kernel_name(1) == NULL)
        ++bad;
    /* a NULL context must be refused, not dereferenced */
    if (maize_gemm_bf16(NULL, NULL, 1, 8, NULL, 1, 8, NULL, 1, 1, NULL) != MAIZE_ERR_INVALID_ARG)
        ++bad;
    if (maize_ctx_poll(NULL, NULL) != MAIZE_ERR_INVALID_ARG)
        ++bad;
    if (maize_mgpu_sync(NULL) != MAIZE_ERR_INVALID_ARG || maize_mgpu_size(NULL) != 0)
        ++bad;
    /* the kernel chosen for a large square problem and for a decode shape differ */
    const int big = maize_pick_kernel(NULL, 16384, 16384, 16384);
    const int decode = maize_pick_kernel(NULL, 16, 16384, 4096);
    if (big < 1 || decode < 1 || big == decode)
        ++bad;
    printf("selftest: version %d, large -> %s, decode -> %s, %d failure(s)\n", maize_version(), maize_kernel_name(big),
           maize_kernel_name(decode), bad);
    return bad ? 1 : 0;
}

/* C = A * B^T over G devices of one process: B's rows and C's columns are split over the devices, A is forwarded
 * from device 0 along the chain. */
static int run_mgpu(int g, uint32_t m, uint32_t n, uint32_t k, uint64_t seed)
{
    int devices[16];
    if (g < 1 || g > 16)
        return 1;
    for (int i = 0; i < g; ++i)
        devices[i] = i;
    maize_mgpu_t *mg = NULL;
    maize_status_t st = maize_mgpu_create(g, devices, &mg);
    if (st == MAIZE_ERR_NO_DEVICE) {
        printf("no CUDA device: %s; nothing computed (there is no CPU path in the library)\n", maize_status_string(st));
        return 77;
    }
    if (st != MAIZE_OK) {
        fprintf(stderr, "maize_mgpu_create(%d): %s\n", g, maize_status_string(st));
        return 1;
    }
    uint16_t *a = malloc((size_t)m * k * 2 + 2), *b = malloc((size_t)n * k * 2 + 2);
    uint16_t *c = malloc((size_t)m * n * 2 + 2), *ref = malloc((size_t)m * n * 2 + 2);
    if (!a || !b || !c || !ref)
        return 1;
    maize_oracle_fill_bf16(seed, 1, 0, 1.0, 0, (uint64_t)n * k, b);
    int failed = 0;
    for (int step = 0; step < 2 && !failed; ++step) {
        maize_oracle_fill_bf16(seed + 100 * (uint64_t)step, 0, 0, 1.0, 0, (uint64_t)m * k, a);
        memset(c, 0xff, (size_t)m * n * 2);
        st = maize_gemm_bf16_nsharded_host(mg, 0, a, m, k, b, n, c);
        if (st != MAIZE_OK) {
            fprintf(stderr, "sharded GEMM failed: %s: %s\n", maize_status_string(st), maize_mgpu_last_error(mg));
            failed = 1;
            break;
        }
        maize_oracle_gemm_bf16(a, m, k, b, n, k, ref, m, n, 0);
        double err = 0, bound = 0;
        uint64_t bad = 0;
        const int rc = maize_oracle_check(c, n, ref, n, m, n, k, maize_oracle_max_abs_bf16(a, (uint64_t)m * k),
                                          maize_oracle_max_abs_bf16(b, (uint64_t)n * k), &err, &bound, &bad);
        printf("%d device(s), step %d, %u x %u x %u: max |err| %.6g <= %.6g, %llu violation(s)\n", maize_mgpu_size(mg),
               step, m, n, k, err, bound, (unsigned long long)bad);
        failed = rc != 0;
    }
    maize_mgpu_destroy(mg);
    free(a);
    free(b);
    free(c);
    free(ref);
    return failed;
}

int main(int argc, char **argv)
{
    if (argc == 2 && strcmp(argv[1], "--selftest") == 0)
        return selftest();
    if (argc >= 6 && strcmp(argv[1], "--mgpu") == 0)
        return run_mgpu(atoi(argv[2]), (uint32_t)strtoul(argv[3], NULL, 10), (uint32_t)strtoul(argv[4], NULL, 10),
                        (uint32_t)strtoul(argv[5], NULL, 10), argc > 6 ? strtoull(argv[6], NULL, 10) : 0);
    if (argc < 4) {
        fprintf(stderr, "usage: %s M N K [seed] | --selftest\n", argv[0]);
        return 1;
    }
    const uint32_t m = (uint32_t)strtoul(argv[1], NULL, 10);
    const uint32_t n = (uint32_t)strtoul(argv[2], NULL, 10);
    const uint32_t k = (uint32_t)strtoul(argv[3], NULL, 10);
    const uint64_t seed = argc > 4 ? strtoull(argv[4], NULL, 10) : 0;

    maize_ctx_t *ctx = NULL;
    maize_status_t st = maize_ctx_create(0, &ctx);
    if (st == MAIZE_ERR_NO_DEVICE) {
        printf("no CUDA device: %s; nothing computed (there is no CPU path in the library)\n", maize_status_string(st));
        return 77;
    }
    if (st != MAIZE_OK) {
        fprintf(stderr, "maize_ctx_create: %s\n", maize_status_string(st));
        return 1;
    }

    uint16_t *a = malloc((size_t)m * k * 2 + 2), *b = malloc((size_t)n * k * 2 + 2);
    uint16_t *c = malloc((size_t)m * n * 2 + 2), *ref = malloc((size_t)m * n * 2 + 2);
    if (!a || !b || !c || !ref) {
        fprintf(stderr, "out of host memory\n");
        return 1;
    }
    maize_oracle_fill_bf16(seed, 0, 0, 1.0, 0, (uint64_t)m * k, a);
    maize_oracle_fill_bf16(seed, 1, 0, 1.0, 0, (uint64_t)n * k, b);
    memset(c, 0xff, (size_t)m * n * 2); /* NaN pattern: every element must be written */

    /* the reference's call shape: (A, a_rows, a_cols, B, b_rows, b_cols) plus the C triple it lacks */
    st = maize_gemm_bf16_host(ctx, a, m, k, b, n, k, c, m, n, NULL);
    if (st == MAIZE_OK)
        st = maize_ctx_poll(ctx, NULL);
    if (st != MAIZE_OK) {
        fprintf(stderr, "GEMM failed: %s: %s\n", maize_status_string(st), maize_last_error(ctx));
        maize_ctx_destroy(ctx);
        return 1;
    }
    if (maize_oracle_gemm_bf16(a, m, k, b, n, k, ref, m, n, 0) != 0) {
        fprintf(stderr, "oracle failed\n");
        return 1;
    }
    double err = 0, bound = 0;
    uint64_t bad = 0;
    const int rc = maize_oracle_check(c, n, ref, n, m, n, k, maize_oracle_max_abs_bf16(a, (uint64_t)m * k),
                                      maize_oracle_max_abs_bf16(b, (uint64_t)n * k), &err, &bound, &bad);
    printf("%u x %u x %u seed %llu: kernel %s, max |err| %.6g <= %.6g, %llu violation(s), %llu launch(es)\n", m, n, k,
           (unsigned long long)seed, maize_kernel_name(maize_pick_kernel(ctx, m, n, k)), err, bound,
           (unsigned long long)bad, (unsigned long long)maize_ctx_launch_count(ctx));
    maize_ctx_destroy(ctx);
    free(a);
    free(b);
    free(c);
    free(ref);
    return rc == 0 ? 0 : 1;
}
