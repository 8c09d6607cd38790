/*
 * CPU oracle for the INT8 quantized-inference path of commandant1/rpl.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared with; nothing in the shipped library may call, link or import it.
 *
 * It is a restatement, in plain C with explicit operation order, of what the
 * reference's scalar (non-NEON) branch computes.  Each function names the
 * reference lines it follows.  Parity pin: tests compare every function here
 * with the reference's own code compiled from its sources (oracle/_ref, built
 * by oracle/Makefile) and with committed vectors generated from that build
 * (tests/golden/).  The reference ships no golden vectors of its own for
 * this path.
 *
 * Two behaviours of the reference are undefined in ISO C and are fixed here
 * to what its x86-64 build does, because that build is the parity authority:
 *   - float -> int32 of NaN / out-of-range values gives INT32_MIN
 *     (cvttss2si "integer indefinite");
 *   - int32 additions wrap in two's complement.
 *
 * Compile with -ffp-contract=off so that no multiply-add is fused.
 */
#include <stdint.h>
#include <stddef.h>
#include <math.h>
#include <float.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* (int32_t)v as an x86-64 build performs it. */
static inline int32_t orc_f2i(float v) {
    if (!(fabsf(v) < 2147483648.0f)) return INT32_MIN;
    return (int32_t)v;
}

static inline int32_t orc_wrap_add(int32_t a, int32_t b) {
    return (int32_t)((uint32_t)a + (uint32_t)b);
}

static inline int8_t orc_clamp_i8(int32_t q) {
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    return (int8_t)q;
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* src/ops_extended.c:52-61 (tensor_get_min_max): seed with x[0], strict
 * compares, untouched outputs when n == 0. */
ORC_API void orc_minmax_serial(const float* x, uint64_t n, float* mn, float* mx) {
    if (n == 0) return;
    float lo = x[0], hi = x[0];
    for (uint64_t i = 1; i < n; i++) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
    }
    *mn = lo;
    *mx = hi;
}

/* src/rpl_quantization.c:79-85 (the reduction inside
 * tensor_quantize_int8_symmetric / _asymmetric and calibrator_update :33-49):
 * seeds are +FLT_MAX / -FLT_MAX, strict compares, so NaNs never win. */
ORC_API void orc_minmax_seeded(const float* x, uint64_t n, float* mn, float* mx) {
    float lo = FLT_MAX, hi = -FLT_MAX;
    #pragma omp parallel for reduction(min:lo) reduction(max:hi)
    for (int64_t i = 0; i < (int64_t)n; i++) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
    }
    *mn = lo;
    *mx = hi;
}

/* src/rpl_quantization.c:87-88 and :57-59: symmetric scale. */
ORC_API float orc_scale_symmetric(float mn, float mx) {
    float abs_max = fmaxf(fabsf(mn), fabsf(mx));
    return abs_max / 127.0f;
}

/* src/rpl_quantization.c:102-104 and :62-64: asymmetric scale, zero point. */
ORC_API void orc_params_asymmetric(float mn, float mx, float* scale, int32_t* zp) {
    float range = mx - mn;
    float s = range / 255.0f;
    *scale = s;
    *zp = orc_f2i(roundf(-mn / s));
}

/* src/rpl_core.c:521-527 (tensor_quantize_int8): divide, roundf (ties away
 * from zero), convert, add the zero point, then clamp to [-128,127]. */
ORC_API void orc_quantize_i8(const float* x, int8_t* q, uint64_t n, float scale, int32_t zp) {
    #pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)n; i++) {
        int32_t v = orc_wrap_add(orc_f2i(roundf(x[i] / scale)), zp);
        q[i] = orc_clamp_i8(v);
    }
}

/* src/rpl_quantization.c:77-91 (tensor_quantize_int8_symmetric). */
ORC_API float orc_quantize_symmetric(const float* x, int8_t* q, uint64_t n) {
    float mn, mx;
    orc_minmax_seeded(x, n, &mn, &mx);
    float scale = orc_scale_symmetric(mn, mx);
    orc_quantize_i8(x, q, n, scale, 0);
    return scale;
}

/* src/rpl_quantization.c:93-107 (tensor_quantize_int8_asymmetric). */
ORC_API void orc_quantize_asymmetric(const float* x, int8_t* q, uint64_t n, float* scale, int32_t* zp) {
    float mn, mx;
    orc_minmax_seeded(x, n, &mn, &mx);
    orc_params_asymmetric(mn, mx, scale, zp);
    orc_quantize_i8(x, q, n, *scale, *zp);
}

/* src/rpl_quantization.c:134-157 (tensor_quantize_per_channel): a channel is
 * the contiguous block [c*L, (c+1)*L) whatever channel_axis was; its scale is
 * absmax/127, its zero point 0. */
ORC_API void orc_quantize_per_channel(const float* x, int8_t* q, float* scales, int32_t* zps,
                                      uint64_t num_channels, uint64_t channel_size) {
    #pragma omp parallel for
    for (int64_t c = 0; c < (int64_t)num_channels; c++) {
        const float* row = x + (uint64_t)c * channel_size;
        int8_t* out = q + (uint64_t)c * channel_size;
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (uint64_t i = 0; i < channel_size; i++) {
            if (row[i] < lo) lo = row[i];
            if (row[i] > hi) hi = row[i];
        }
        float s = fmaxf(fabsf(lo), fabsf(hi)) / 127.0f;
        scales[c] = s;
        zps[c] = 0;
        for (uint64_t i = 0; i < channel_size; i++)
            out[i] = orc_clamp_i8(orc_f2i(roundf(row[i] / s)));
    }
}

/* src/ops_extended.c:67-70 (tensor_dequantize_int8): integer subtract, one
 * exact int->float conversion, one fp32 multiply. */
ORC_API void orc_dequantize_i8(const int8_t* q, float* out, uint64_t n, float scale, int32_t zp) {
    #pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)n; i++)
        out[i] = (float)(int32_t)((uint32_t)(int32_t)q[i] - (uint32_t)zp) * scale;   /* int32 subtraction wraps */
}

/* Per-channel form of the same statement (the reference has no per-channel
 * dequantizer; this follows src/ops_extended.c:69 with scales[c], zp 0). */
ORC_API void orc_dequantize_per_channel(const int8_t* q, const float* scales, float* out,
                                        uint64_t num_channels, uint64_t channel_size) {
    #pragma omp parallel for
    for (int64_t c = 0; c < (int64_t)num_channels; c++)
        for (uint64_t i = 0; i < channel_size; i++)
            out[(uint64_t)c * channel_size + i] = (float)(int32_t)q[(uint64_t)c * channel_size + i] * scales[c];
}

/* src/ops_extended.c:114-120 (gemm_int8_fallback, scalar branch):
 *   sum = sum_k (A[i,k]-za) * (B[k,j]-zb)                 int32
 *   C[i,j] = (int32) roundf( (((float)sum * sa) * sb) / sc )
 * A is [M,K] row-major, B is [K,N] row-major, C is [M,N] row-major int32.
 * The loop order differs from the reference (k outside j, so B is read along
 * rows); integer sums do not depend on the order. */
ORC_API void orc_gemm_i8_requant(const int8_t* A, const int8_t* B, int32_t* C,
                                 uint64_t M, uint64_t N, uint64_t K,
                                 float sa, float sb, float sc, int32_t za, int32_t zb) {
    #pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)M; i++) {
        int32_t* acc = C + (uint64_t)i * N;
        for (uint64_t j = 0; j < N; j++) acc[j] = 0;
        for (uint64_t k = 0; k < K; k++) {
            int32_t a = (int32_t)A[(uint64_t)i * K + k] - za;
            const int8_t* brow = B + k * N;
            for (uint64_t j = 0; j < N; j++)
                acc[j] = orc_wrap_add(acc[j], (int32_t)((uint32_t)a * (uint32_t)((int32_t)brow[j] - zb)));
        }
        for (uint64_t j = 0; j < N; j++) {
            float r = (float)acc[j] * sa;
            r = r * sb;
            r = r / sc;
            acc[j] = orc_f2i(roundf(r));
        }
    }
}

/* src/rpl_quantization.c:340-350 (linear_int8, scalar branch):
 *   out[b,o] = sum_i in[b,i] * w[o,i]  (+ (int8) bias[o])      raw int32
 * in is [M,K], w is [N,K] (both K-contiguous), out is [M,N]. */
ORC_API void orc_linear_i8(const int8_t* in, const int8_t* w, const int8_t* bias, int32_t* out,
                           uint64_t M, uint64_t K, uint64_t N) {
    #pragma omp parallel for
    for (int64_t b = 0; b < (int64_t)M; b++) {
        const int8_t* a = in + (uint64_t)b * K;
        for (uint64_t o = 0; o < N; o++) {
            const int8_t* wr = w + o * K;
            int32_t sum = 0;
            for (uint64_t i = 0; i < K; i++) sum += (int32_t)a[i] * (int32_t)wr[i];
            if (bias) sum = orc_wrap_add(sum, (int32_t)bias[o]);
            out[(uint64_t)b * N + o] = sum;
        }
    }
}

/* Fused fp32 epilogue.  The reference has no such function; this composes its
 * primitives in a fixed order:
 *   acc            src/rpl_quantization.c:340-350 (linear_int8, bias NULL)
 *   (float)acc*s   src/ops_extended.c:69 (int -> float, then one multiply)
 *   + bias[n]      src/rpl_nn.c:69-71 with src/rpl_core.c:117-119 (bias
 *                  broadcast over the last dimension)
 *   ReLU           src/rpl_core.c:254-255 (x < 0 -> 0)
 *   out[m,n] = relu?( (((float)acc * a_scale) * w_scales[n]) + bias[n] )
 * out has row stride ldo (>= N) so a column block of a wider matrix can be
 * written in place. */
ORC_API void orc_linear_i8_dequant(const int8_t* in, const int8_t* w, float* out,
                                   uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                   float a_scale, const float* w_scales, const float* bias, int relu) {
    #pragma omp parallel for
    for (int64_t b = 0; b < (int64_t)M; b++) {
        const int8_t* a = in + (uint64_t)b * K;
        for (uint64_t o = 0; o < N; o++) {
            const int8_t* wr = w + o * K;
            int32_t sum = 0;
            for (uint64_t i = 0; i < K; i++) sum += (int32_t)a[i] * (int32_t)wr[i];
            float v = (float)sum * a_scale;
            v = v * w_scales[o];
            if (bias) v = v + bias[o];
            if (relu && v < 0.0f) v = 0.0f;
            out[(uint64_t)b * ldo + o] = v;
        }
    }
}

/* src/rpl_core.c:254-255 (tensor_relu_inplace, scalar branch). */
ORC_API void orc_relu_inplace(float* x, uint64_t n) {
    #pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)n; i++)
        if (x[i] < 0.0f) x[i] = 0.0f;
}
