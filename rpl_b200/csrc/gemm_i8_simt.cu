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
