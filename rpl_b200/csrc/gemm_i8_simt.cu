// INT8 x INT8 -> INT32 contraction on the integer dot-product units (dp4a).
//
// This kernel takes every shape, layout and alignment the entry points accept
// (ragged M/N/K, B as [N,K] or [K,N], zero points), and is the cross-check of
// the tensor-core kernel at sizes a CPU cannot reach.  64x64 output tile per
// CTA, 64-byte K steps staged in shared memory as 32-bit words, 4x4 outputs
// per thread.
#include "gemm_common.cuh"

namespace rplb {

constexpr int BM = 64, BN = 64, BKW = 16;     // tile: 64 x 64 outputs, 16 words (64 int8) of K per step
constexpr int LDW = BKW + 1;                  // word stride of a tile row (odd: no bank conflicts)
constexpr int SIMT_THREADS = 256;

// Four consecutive K bytes of row `r` starting at byte k of a [rows, K]
// row-major matrix, zero beyond the edges.
__device__ __forceinline__ uint32_t load_word_rowmajor(const int8_t* __restrict__ base, uint64_t rows, uint64_t K,
                                                       uint64_t r, uint64_t k, bool aligned) {
    if (r >= rows || k >= K) return 0;
    const int8_t* p = base + r * K + k;
    if (aligned && k + 4 <= K) return __ldg(reinterpret_cast<const uint32_t*>(p));
    uint32_t w = 0;
    #pragma unroll
    for (int b = 0; b < 4; b++)
        if (k + b < K) w |= (uint32_t)(uint8_t)__ldg(p + b) << (8 * b);
    return w;
}

template <bool ZERO_POINTS>
__global__ void __launch_bounds__(SIMT_THREADS)
gemm_i8_simt_kernel(GemmProblem p) {
    __shared__ uint32_t As[BM * LDW];
    __shared__ uint32_t Bs[BN * LDW];
    const int t = threadIdx.x;
    const int tx = t & 15, ty = t >> 4;
    const uint64_t m0 = (uint64_t)blockIdx.x * BM, n0 = (uint64_t)blockIdx.y * BN;      // x spans M: it may be large
    const bool a_aligned = (((uintptr_t)p.A & 3) == 0) && (p.K % 4 == 0);
    const bool b_aligned = (((uintptr_t)p.B & 3) == 0) && (p.K % 4 == 0);

    int32_t acc[4][4];
    int32_t rowsum[4] = {0, 0, 0, 0}, colsum[4] = {0, 0, 0, 0};
    #pragma unroll
    for (int i = 0; i < 4; i++)
        #pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0;

    for (uint64_t k0 = 0; k0 < p.K; k0 += BKW * 4) {
        // Stage A: 64 rows x 16 words, four words per thread.
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            int w = t + SIMT_THREADS * j;
            int r = w / BKW, kw = w % BKW;
            As[r * LDW + kw] = load_word_rowmajor(p.A, p.M, p.K, m0 + r, k0 + kw * 4, a_aligned);
        }
        if (!p.b_is_kn) {
            #pragma unroll
            for (int j = 0; j < 4; j++) {
                int w = t + SIMT_THREADS * j;
                int r = w / BKW, kw = w % BKW;
                Bs[r * LDW + kw] = load_word_rowmajor(p.B, p.N, p.K, n0 + r, k0 + kw * 4, b_aligned);
            }
        } else {
            // B is [K,N]: consecutive threads read consecutive n of one k row.
            const int n = t & 63, kg = t >> 6;          // kg: which 16-byte K group
            #pragma unroll
            for (int kw = 0; kw < 4; kw++) {
                uint32_t w = 0;
                #pragma unroll
                for (int b = 0; b < 4; b++) {
                    uint64_t k = k0 + (uint64_t)(kg * 16 + kw * 4 + b);
                    if (k < p.K && n0 + n < p.N) w |= (uint32_t)(uint8_t)__ldg(p.B + k * p.N + n0 + n) << (8 * b);
                }
                Bs[n * LDW + kg * 4 + kw] = w;
            }
        }
        __syncthreads();
        #pragma unroll
        for (int kw = 0; kw < BKW; kw++) {
            uint32_t a[4], b[4];
            #pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[(ty * 4 + i) * LDW + kw];
            #pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[(tx + 16 * j) * LDW + kw];
            #pragma unroll
            for (int i = 0; i < 4; i++)
                #pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __dp4a((int)a[i], (int)b[j], acc[i][j]);
            if (ZERO_POINTS) {
                #pragma unroll
                for (int i = 0; i < 4; i++) rowsum[i] = __dp4a((int)a[i], 0x01010101, rowsum[i]);
                #pragma unroll
                for (int j = 0; j < 4; j++) colsum[j] = __dp4a((int)b[j], 0x01010101, colsum[j]);
            }
        }
        __syncthreads();
    }

    const bool fp_mode = p.mode == EPI_DEQUANT_F32 || p.mode == EPI_DEQUANT_I8;
    const float a_scale = fp_mode ? __ldg(p.a_scale) : 0.0f;
    const QuantConsts oq = make_quant_consts(p.mode == EPI_DEQUANT_I8 ? __ldg(p.out_scale) : 1.0f, p.out_zp);
    float absmax = 0.0f;
    #pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint64_t m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint64_t n = n0 + tx + 16 * j;
            if (n >= p.N) continue;
            int32_t sum = acc[i][j];
            if (ZERO_POINTS) sum = apply_zero_points(sum, rowsum[i], colsum[j], p.za, p.zb, (uint32_t)p.K);
            const uint64_t o = m * p.ldo + n;
            if (p.mode == EPI_RAW_I32) {
                if (p.bias_i8) sum = (int32_t)((uint32_t)sum + (uint32_t)(int32_t)__ldg(p.bias_i8 + n));
                static_cast<int32_t*>(p.out)[o] = sum;
            } else if (p.mode == EPI_REQUANT_I32) {
                static_cast<int32_t*>(p.out)[o] = requant_i32(sum, p.sa, p.sb, p.sc);
            } else {
                const float v = dequant_f32(sum, a_scale, __ldg(p.w_scales + n), p.bias_f32 != nullptr,
                                            p.bias_f32 ? __ldg(p.bias_f32 + n) : 0.0f, p.relu != 0);
                if (p.absmax_out) absmax_fold(absmax, v);
                if (p.mode == EPI_DEQUANT_F32) static_cast<float*>(p.out)[o] = v;
                else static_cast<int8_t*>(p.out)[o] = (int8_t)quantize_one(v, oq.scale, oq.zp);
            }
        }
    }
    if (fp_mode && p.absmax_out) absmax_publish(p.absmax_out, absmax);
}

// ---------------------------------------------------------------------------
// Quantize fused into a layer with very few output features (the last layer of
// the quantized MLP: 128 -> 10): out[m,n] = relu?(((float)acc * sA) * sW[n] + bias[n])
// with acc = sum_k q(x[m,k]) * w[n,k] and q = tensor_quantize_int8's statement
// (src/rpl_core.c:523-526) with the scale *a_scale.  The fp32 activation is read
// once, coalesced (a warp takes 32 rows; lane l loads quad l of each row), quantized
// in registers and transposed through a 32 x 33-word shared-memory tile, after
// which lane l owns row l and accumulates its N dot products with dp4a against the
// weight words held in shared memory (every lane reads the same word: a broadcast).
// Neither the int8 activation nor a 128- or 256-column tensor-core tile is
// materialised for a handful of outputs.
constexpr int SMALL_N_MAX = 16;
constexpr int SMALL_K_MAX = 512;
constexpr int SMALL_WARPS = 8;

template <int NT>                      // the number of output features, known at compile time: the inner loop has no tests
__global__ void __launch_bounds__(SMALL_WARPS * 32, 2)
quantize_linear_small_kernel(const float* __restrict__ x, const GemmProblem p) {
    constexpr uint32_t N = NT, NP = (NT + 3) & ~3;                       // N padded to whole 16-byte pieces
    __shared__ __align__(16) uint32_t w_words[SMALL_N_MAX * SMALL_K_MAX / 4];   // [K/4][NP]: word t of every output feature side by side
    __shared__ uint32_t tiles[SMALL_WARPS][32 * 33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t K = (uint32_t)p.K, kw = K / 4;
    for (uint32_t i = threadIdx.x; i < NP * kw; i += blockDim.x) {
        const uint32_t n = i / kw, t = i % kw;
        w_words[t * NP + n] = n < N ? __ldg(reinterpret_cast<const uint32_t*>(p.B) + (size_t)n * kw + t) : 0u;
    }
    __syncthreads();
    const QuantConsts qc = make_quant_consts(__ldg(p.a_scale), 0);
    const float a_scale = qc.scale;
    const bool has_bias = p.bias_f32 != nullptr, relu = p.relu != 0;
    uint32_t* tile = tiles[warp];
    float absmax = 0.0f;
    const uint64_t groups = (p.M + 31) / 32;
    for (uint64_t g = (uint64_t)blockIdx.x * SMALL_WARPS + warp; g < groups; g += (uint64_t)gridDim.x * SMALL_WARPS) {
        const uint64_t m0 = g * 32;
        int32_t acc[NT];
        #pragma unroll
        for (int n = 0; n < NT; n++) acc[n] = 0;
        for (uint32_t c0 = 0; c0 < kw; c0 += 32) {                      // 32 words = 128 k per pass
            const uint32_t j = c0 + lane;                                // this lane's word of every row
            __syncwarp();                                                // the previous pass has been read out of the tile
            #pragma unroll 1
            for (int half = 0; half < 2; half++) {                       // sixteen rows at a time: 16 loads in flight per lane
                float4 v[16];
                #pragma unroll
                for (int r = 0; r < 16; r++) {
                    const uint64_t m = m0 + half * 16 + r;
                    v[r] = (j < kw && m < p.M) ? __ldcs(reinterpret_cast<const float4*>(x + m * K) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                #pragma unroll
                for (int r = 0; r < 16; r++)
                    tile[(half * 16 + r) * 33 + lane] = (j < kw && m0 + half * 16 + r < p.M) ? quantize_quad_packed(v[r], qc) : 0u;
            }
            __syncwarp();
            const uint32_t words = min(32u, kw - c0);
            for (uint32_t t = 0; t < words; t++) {
                const int a = (int)tile[lane * 33 + t];                  // row `lane`, word c0 + t
                const uint4* wt = reinterpret_cast<const uint4*>(w_words + (size_t)(c0 + t) * NP);   // the same words for every lane
                uint32_t wv[NP];
                #pragma unroll
                for (uint32_t q = 0; q < NP / 4; q++) {
                    const uint4 u = wt[q];
                    wv[4 * q] = u.x; wv[4 * q + 1] = u.y; wv[4 * q + 2] = u.z; wv[4 * q + 3] = u.w;
                }
                #pragma unroll
                for (int n = 0; n < NT; n++) acc[n] = __dp4a(a, (int)wv[n], acc[n]);
            }
        }
        const uint64_t m = m0 + lane;
        if (m < p.M) {
            float* row = static_cast<float*>(p.out) + m * p.ldo;
            #pragma unroll
            for (int n = 0; n < NT; n++) {
                const float o = dequant_f32(acc[n], a_scale, __ldg(p.w_scales + n), has_bias, has_bias ? __ldg(p.bias_f32 + n) : 0.0f, relu);
                if (p.absmax_out) absmax_fold(absmax, o);
                row[n] = o;
            }
        }
    }
    if (p.absmax_out) absmax_publish(p.absmax_out, absmax);
}

bool quantize_linear_small_supports(const float* x, const GemmProblem& p) {
    return p.mode == EPI_DEQUANT_F32 && !p.b_is_kn && !p.n_peers && !p.a_ready && p.M && p.N && p.K &&
           p.N <= (uint64_t)SMALL_N_MAX && p.K <= (uint64_t)SMALL_K_MAX && p.K % 4 == 0 &&
           (((uintptr_t)x & 15) == 0) && (((uintptr_t)p.B & 3) == 0);
}

int quantize_linear_small(const float* x, const GemmProblem& p, cudaStream_t st) {
    if (!quantize_linear_small_supports(x, p))
        return fail(RPLB_E_UNSUPPORTED, "fused quantize + small linear needs N <= %d, K <= %d, K %% 4 == 0, aligned x and w", SMALL_N_MAX, SMALL_K_MAX);
    const uint64_t groups = (p.M + 31) / 32;
    uint64_t want = (groups + SMALL_WARPS - 1) / SMALL_WARPS;
    uint64_t cap = (uint64_t)sm_count() * 4;
    if (cap == 0) cap = 148 * 4;
    const unsigned int grid = (unsigned int)(want < cap ? want : cap);
    switch (p.N) {
#define RPLB_SMALL_N(NT) case NT: quantize_linear_small_kernel<NT><<<grid, SMALL_WARPS * 32, 0, st>>>(x, p); break;
        RPLB_SMALL_N(1) RPLB_SMALL_N(2) RPLB_SMALL_N(3) RPLB_SMALL_N(4) RPLB_SMALL_N(5) RPLB_SMALL_N(6) RPLB_SMALL_N(7) RPLB_SMALL_N(8)
        RPLB_SMALL_N(9) RPLB_SMALL_N(10) RPLB_SMALL_N(11) RPLB_SMALL_N(12) RPLB_SMALL_N(13) RPLB_SMALL_N(14) RPLB_SMALL_N(15) RPLB_SMALL_N(16)
#undef RPLB_SMALL_N
        default: return fail(RPLB_E_UNSUPPORTED, "fused quantize + small linear: N = %llu", (unsigned long long)p.N);
    }
    return launched("quantize_linear_small_kernel");
}

int gemm_simt(const GemmProblem& p, cudaStream_t st) {
    if (p.M == 0 || p.N == 0) return 0;
    uint64_t gx = (p.M + BM - 1) / BM, gy = (p.N + BN - 1) / BN;
    if (gy > 65535 || gx > 0x7fffffffull)
        return fail(RPLB_E_TOO_LARGE, "dp4a GEMM: N = %llu exceeds 65535*64 columns (or M beyond 2^37 rows)", (unsigned long long)p.N);
    dim3 grid((unsigned int)gx, (unsigned int)gy);
    if (p.mode == EPI_REQUANT_I32 && (p.za != 0 || p.zb != 0))
        gemm_i8_simt_kernel<true><<<grid, SIMT_THREADS, 0, st>>>(p);
    else
        gemm_i8_simt_kernel<false><<<grid, SIMT_THREADS, 0, st>>>(p);
    return launched("gemm_i8_simt_kernel");
}

}  // namespace rplb
