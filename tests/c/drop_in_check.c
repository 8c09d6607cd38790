/*
 * A C caller of the INT8 path, written the way examples/c_api_demo.c:112-190 of
 * the reference uses it (min/max -> scale -> tensor_quantize_int8 ->
 * tensor_dequantize_int8, then gemm_int8 on int8 matrices), plus linear_int8
 * and the symmetric / per-channel quantizers.  It checks every result against
 * a plain C loop of the same statements and prints "drop_in_check: OK".
 *
 * Compile against either header:
 *   -DUSE_REFERENCE_HEADER -I<reference>/include   the reference's own rpl.h
 *   (default)                                      include/rpl_b200.h
 * and link with -lrpl from rpl_b200/lib.  Exit code 0 = all checks passed,
 * 2 = the library reported no usable CUDA device, 1 = a mismatch.
 */
#ifdef USE_REFERENCE_HEADER
#include "rpl.h"
#endif
#include "rpl_b200.h"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static unsigned long long rng_state = 0x9E3779B97F4A7C15ull;
static float frand(void) {            /* uniform in [-1, 1) */
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
    return (float)((rng_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}

static int8_t quant_one(float x, float scale, int zp) {
    int q = (int)roundf(x / scale) + zp;
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

int main(void) {
    if (rplb_device_count() == 0) {
        printf("drop_in_check: no CUDA device\n");
        return 2;
    }
    int bad = 0;
    uint32_t shape[2] = {100, 100};
    Tensor* t = tensor_create(2, shape, false);
    for (uint32_t i = 0; i < t->size; i++) t->data[i] = frand() * 3.0f;

    float mn = 0, mx = 0;
    tensor_get_min_max(t, &mn, &mx);
    float lo = t->data[0], hi = t->data[0];
    for (uint32_t i = 1; i < t->size; i++) { if (t->data[i] < lo) lo = t->data[i]; if (t->data[i] > hi) hi = t->data[i]; }
    bad += (mn != lo) + (mx != hi);

    float abs_max = (mx > -mn) ? mx : -mn;
    float scale = abs_max / 127.0f;
    QuantizedTensor* q = tensor_quantize_int8(t, scale, 0);
    if (!q) { printf("tensor_quantize_int8 returned NULL (error %d)\n", rpl_cuda_last_error()); return 1; }
    for (uint32_t i = 0; i < t->size; i++) bad += q->data[i] != quant_one(t->data[i], scale, 0);
    Tensor* back = tensor_dequantize_int8(q);
    for (uint32_t i = 0; i < t->size; i++) bad += back->data[i] != (float)(q->data[i] - q->zero_point) * q->scale;

    QuantizedTensor* qs = tensor_quantize_int8_symmetric(t);
    float s2 = fmaxf(fabsf(lo), fabsf(hi)) / 127.0f;
    bad += qs->scale != s2;
    for (uint32_t i = 0; i < t->size; i++) bad += qs->data[i] != quant_one(t->data[i], s2, 0);

    PerChannelQuantizedTensor* pc = tensor_quantize_per_channel(t, 0);
    bad += (pc->num_channels != 100) + (pc->channel_size != 100);
    for (uint32_t c = 0; c < 100; c++) {
        float l = 3.4e38f, h = -3.4e38f;
        for (uint32_t i = 0; i < 100; i++) { float v = t->data[c * 100 + i]; if (v < l) l = v; if (v > h) h = v; }
        float sc = fmaxf(fabsf(l), fabsf(h)) / 127.0f;
        bad += pc->scales[c] != sc;
        for (uint32_t i = 0; i < 100; i++) bad += pc->data[c * 100 + i] != quant_one(t->data[c * 100 + i], sc, 0);
    }

    /* INT8 GEMM as the reference's example does it: 128^3, scales 0.01 */
    enum { M = 128, N = 128, K = 128 };
    int8_t* A = (int8_t*)rpitorch_aligned_alloc(64, M * K);
    int8_t* B = (int8_t*)rpitorch_aligned_alloc(64, K * N);
    int32_t* C = (int32_t*)rpitorch_aligned_alloc(64, M * N * sizeof(int32_t));
    for (int i = 0; i < M * K; i++) A[i] = (int8_t)(frand() * 127.0f);
    for (int i = 0; i < K * N; i++) B[i] = (int8_t)(frand() * 127.0f);
    gemm_int8(A, B, C, M, N, K, 0.01f, 0.01f, 0.01f, 0, 0);
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            int32_t sum = 0;
            for (int k = 0; k < K; k++) sum += (int32_t)A[i * K + k] * (int32_t)B[k * N + j];
            float r = sum * 0.01f * 0.01f / 0.01f;
            bad += C[i * N + j] != (int32_t)roundf(r);
        }
    /* linear_int8: weights [out, in] */
    QuantizedTensor qa = {A, 1.0f, 0, M * K, 2, {M, K}}, qw = {B, 1.0f, 0, N * K, 2, {N, K}};
    linear_int8(&qa, &qw, NULL, C, M, K, N);
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            int32_t sum = 0;
            for (int k = 0; k < K; k++) sum += (int32_t)A[i * K + k] * (int32_t)B[j * K + k];
            bad += C[i * N + j] != sum;
        }

    per_channel_quantized_tensor_free(pc);
    quantized_tensor_free(qs);
    quantized_tensor_free(q);
    tensor_free(back);
    tensor_free(t);
    rpitorch_aligned_free(A); rpitorch_aligned_free(B); rpitorch_aligned_free(C);
    if (bad || rpl_cuda_last_error()) { printf("drop_in_check: %d mismatches, last error %d\n", bad, rpl_cuda_last_error()); return 1; }
    printf("drop_in_check: OK\n");
    return 0;
}
