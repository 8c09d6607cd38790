/*
 * A C host running the quantized Linear over several GPUs with rplb_* calls only
 * (no CUDA headers, no Python): one process per GPU, forked here; rank 0 makes the
 * NCCL id and hands it to the others through a pipe.
 *
 *   sharded_check WORLD
 *
 * The problem is shaped like the large sharded GEMM (rows of A and columns of the
 * output both split over the ranks), at a size plain C loops can check: every
 * rank compares the int8 activation it ends up with, the scale and its column
 * block of the fp32 output with loops written after the reference's statements
 * (src/rpl_quantization.c:79-90, :340-350; src/rpl_core.c:521-527).
 */
#define _POSIX_C_SOURCE 200809L
#include "rpl_b200.h"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#define CHECK(call) do { int rc_ = (call); if (rc_ != 0) { fprintf(stderr, "rank %d: %s failed: %s [%d]\n", g_rank, #call, rplb_last_error(), rc_); return 1; } } while (0)

static int g_rank = 0;

static uint64_t lcg(uint64_t* s) { *s = *s * 6364136223846793005ull + 1442695040888963407ull; return *s >> 33; }
static float unit(uint64_t* s) { return (float)(lcg(s) & 0xFFFFFF) / 8388608.0f - 1.0f; }      /* [-1, 1) */

static int8_t quantize_one(float x, float scale) {
    float v = roundf(x / scale);
    int32_t q = (fabsf(v) < 2147483648.0f) ? (int32_t)v : INT32_MIN;
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

static int run_rank(int rank, int world, const void* nccl_id) {
    g_rank = rank;
    CHECK(rplb_set_device(rank));                            /* one GPU per process */
    const uint64_t M = 1024, K = 512, N = 2048;
    uint64_t seed = 42;
    float* x = malloc(M * K * 4);
    float* w = malloc(N * K * 4);
    for (uint64_t i = 0; i < M * K; i++) x[i] = unit(&seed) * 3.0f;
    for (uint64_t i = 0; i < N * K; i++) w[i] = unit(&seed) * 0.05f;

    /* this rank's columns and rows */
    uint64_t cb, cc, rb, rc;
    CHECK(rplb_shard_range(N, world, rank, 256, &cb, &cc));
    CHECK(rplb_shard_range(M, world, rank, 128, &rb, &rc));

    /* weights: quantize this rank's rows per channel on the device */
    void *w_dev, *wq_dev, *ws_dev, *x_dev, *out_dev;
    CHECK(rplb_malloc(&w_dev, cc * K * 4));
    CHECK(rplb_malloc(&wq_dev, cc * K));
    CHECK(rplb_malloc(&ws_dev, cc * 4));
    CHECK(rplb_copy(w_dev, w + cb * K, cc * K * 4, NULL));
    CHECK(rplb_quantize_per_channel_f32_i8(w_dev, wq_dev, ws_dev, NULL, cc, K, NULL));
    CHECK(rplb_malloc(&x_dev, (rc ? rc : 1) * K * 4));
    CHECK(rplb_copy(x_dev, x + rb * K, rc * K * 4, NULL));
    CHECK(rplb_malloc(&out_dev, M * cc * 4));

    rplb_sharded_linear* layer = NULL;
    CHECK(rplb_sharded_linear_create(&layer, rank, world, world > 1 ? nccl_id : NULL, NULL, M, K, N, wq_dev, ws_dev, NULL));
    uint64_t b2, c2;
    CHECK(rplb_sharded_linear_columns(layer, &b2, &c2));
    if (b2 != cb || c2 != cc) { fprintf(stderr, "rank %d: column block mismatch\n", rank); return 1; }

    int8_t* xq_ref = malloc(M * K);
    int8_t* xq_got = malloc(M * K);
    int8_t* wq = malloc(cc * K);
    float* ws = malloc(cc * 4);
    float* out = malloc(M * cc * 4);
    for (int pass = 0; pass < 2; pass++) {                   /* twice: the shared buffers are reused */
        CHECK(rplb_sharded_linear_forward(layer, x_dev, M, out_dev, cc, 0, NULL));
        CHECK(rplb_stream_sync(NULL));
        if (rplb_kernel_status(1) != 0) { fprintf(stderr, "rank %d: a kernel gave up waiting\n", rank); return 1; }
        const int8_t* xq_dev; const float* scale_dev; float scale;
        CHECK(rplb_sharded_linear_activation(layer, &xq_dev, &scale_dev));
        CHECK(rplb_copy(xq_got, xq_dev, M * K, NULL));
        CHECK(rplb_copy(&scale, scale_dev, 4, NULL));
        CHECK(rplb_copy(wq, wq_dev, cc * K, NULL));
        CHECK(rplb_copy(ws, ws_dev, cc * 4, NULL));
        CHECK(rplb_copy(out, out_dev, M * cc * 4, NULL));
        CHECK(rplb_stream_sync(NULL));

        /* the reference's statements over the WHOLE activation */
        float mn = 3.402823466e38f, mx = -3.402823466e38f;
        for (uint64_t i = 0; i < M * K; i++) { if (x[i] < mn) mn = x[i]; if (x[i] > mx) mx = x[i]; }
        const float want_scale = fmaxf(fabsf(mn), fabsf(mx)) / 127.0f;
        if (memcmp(&scale, &want_scale, 4) != 0) { fprintf(stderr, "rank %d: scale %.9g, expected %.9g\n", rank, scale, want_scale); return 1; }
        for (uint64_t i = 0; i < M * K; i++) xq_ref[i] = quantize_one(x[i], want_scale);
        if (memcmp(xq_ref, xq_got, M * K) != 0) { fprintf(stderr, "rank %d: int8 activation differs\n", rank); return 1; }
        for (uint64_t m = 0; m < M; m++)
            for (uint64_t n = 0; n < cc; n++) {
                int32_t acc = 0;
                for (uint64_t k = 0; k < K; k++) acc += (int32_t)xq_ref[m * K + k] * (int32_t)wq[n * K + k];
                volatile float v = (float)acc * want_scale;
                v = v * ws[n];
                float got = out[m * cc + n], want = v;
                if (memcmp(&got, &want, 4) != 0) {
                    fprintf(stderr, "rank %d: out[%llu,%llu] = %.9g, expected %.9g\n", rank, (unsigned long long)m, (unsigned long long)n, got, want);
                    return 1;
                }
            }
        for (uint64_t i = 0; i < rc * K; i++) x[rb * K + i] *= 0.5f;       /* new data for the second pass */
        for (uint64_t i = 0; i < M * K; i++) if (i < rb * K || i >= (rb + rc) * K) x[i] *= 0.5f;
        CHECK(rplb_copy(x_dev, x + rb * K, rc * K * 4, NULL));
        CHECK(rplb_stream_sync(NULL));
    }
    rplb_sharded_linear_free(layer);
    rplb_free(w_dev); rplb_free(wq_dev); rplb_free(ws_dev); rplb_free(x_dev); rplb_free(out_dev);
    free(x); free(w); free(xq_ref); free(xq_got); free(wq); free(ws); free(out);
    return 0;
}

int main(int argc, char** argv) {
    int world = argc > 1 ? atoi(argv[1]) : 1;
    if (world < 1 || world > 8) { fprintf(stderr, "usage: sharded_check WORLD (1..8)\n"); return 2; }
    if (world == 1) {
        if (rplb_device_count() == 0) { printf("sharded_check: no CUDA device\n"); return 2; }
        int rc = run_rank(0, 1, NULL);
        if (rc == 0) printf("sharded_check: OK (1 rank)\n");
        return rc;
    }
    /* Rank 0 creates the id in its own process (after the fork, so that no CUDA state is inherited). */
    int pipes[8][2];
    pid_t pids[8];
    for (int r = 1; r < world; r++) if (pipe(pipes[r]) != 0) return 3;
    for (int r = 0; r < world; r++) {
        pids[r] = fork();
        if (pids[r] < 0) return 3;
        if (pids[r] == 0) {
            char id[RPLB_NCCL_ID_BYTES];
            g_rank = r;
            if (r == 0) {
                if (rplb_nccl_unique_id(id) != 0) { fprintf(stderr, "rank 0: %s\n", rplb_last_error()); _exit(1); }
                for (int q = 1; q < world; q++)
                    if (write(pipes[q][1], id, sizeof(id)) != (ssize_t)sizeof(id)) _exit(1);
            } else {
                if (read(pipes[r][0], id, sizeof(id)) != (ssize_t)sizeof(id)) _exit(1);
            }
            _exit(run_rank(r, world, id));
        }
    }
    int bad = 0;
    for (int r = 0; r < world; r++) {
        int st = 0;
        waitpid(pids[r], &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) bad++;
    }
    if (!bad) printf("sharded_check: OK (%d ranks)\n", world);
    return bad ? 1 : 0;
}
