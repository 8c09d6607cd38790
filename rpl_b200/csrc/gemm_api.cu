// C ABI of the INT8 contraction: argument checks, choice of kernel, and the
// [K,N] -> [N,K] transpose that lets gemm_int8's B layout reach the
// tensor-core kernel.
#include "gemm_common.cuh"
#include <atomic>

namespace rplb {

int gemm_tcgen05_status(bool clear);     // gemm_i8_tcgen05.cu

static std::atomic<int> g_backend{0};    // 0 auto, 1 dp4a, 2 tcgen05, 3 tcgen05 single-CTA, 4 tcgen05 CTA pair

// Below this many multiply-accumulates the persistent tensor-core kernel has
// no advantage over the dp4a kernel (one tile is 128 x 256 outputs).
constexpr uint64_t kTcMinMacs = 1ull << 24;

// B [K,N] row-major -> Bt [N,K] row-major through a 32x33-byte shared tile.
__global__ void transpose_i8_kernel(const int8_t* __restrict__ B, int8_t* __restrict__ Bt, uint64_t K, uint64_t N) {
    __shared__ int8_t tile[32][33];
    const uint64_t n0 = (uint64_t)blockIdx.x * 32, k0 = (uint64_t)blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        uint64_t k = k0 + r, n = n0 + threadIdx.x;
        if (k < K && n < N) tile[r][threadIdx.x] = B[k * N + n];
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        uint64_t n = n0 + r, k = k0 + threadIdx.x;
        if (k < K && n < N) Bt[n * K + k] = tile[threadIdx.x][r];
    }
}

static int run_gemm(GemmProblem p, cudaStream_t st) {
    if (p.M == 0 || p.N == 0) return 0;
    if (!p.A || !p.B || !p.out) return fail(RPLB_E_BAD_ARG, "INT8 GEMM: null pointer");
    if (p.ldo < p.N) return fail(RPLB_E_BAD_ARG, "INT8 GEMM: output row stride %llu < N %llu",
                                 (unsigned long long)p.ldo, (unsigned long long)p.N);
    const int backend = g_backend.load(std::memory_order_relaxed);
    if (backend == 1) return gemm_simt(p, st);

    GemmProblem q = p;
    const bool big = p.M * p.N * (p.K ? p.K : 1) >= kTcMinMacs;
    if (p.b_is_kn && (backend >= 2 || big) && p.K % 16 == 0 && p.K && !(p.mode == EPI_REQUANT_I32 && (p.za || p.zb))) {
        // Reorder B once into the K-contiguous layout the tensor-core kernel reads.
        const uint64_t gy = (p.K + 31) / 32;
        if (gy <= 65535) {
            Scratch sc;
            if (int rc = scratch_for(st, (size_t)(p.K * p.N), &sc)) return rc;
            dim3 grid((unsigned int)((p.N + 31) / 32), (unsigned int)gy), block(32, 8);
            transpose_i8_kernel<<<grid, block, 0, st>>>(p.B, static_cast<int8_t*>(sc.data), p.K, p.N);
            if (int rc = launched("transpose_i8_kernel")) return rc;
            q.B = static_cast<const int8_t*>(sc.data);
            q.b_is_kn = 0;
        }
    }
    if (backend >= 2) return gemm_tcgen05(q, st, backend - 2);
    if (big && gemm_tcgen05_supports(q)) return gemm_tcgen05(q, st);
    return gemm_simt(p, st);
}

}  // namespace rplb

using namespace rplb;

extern "C" {

int rplb_gemm_backend(int which) {
    if (which < 0 || which > 4) return g_backend.load();
    return g_backend.exchange(which);
}

int rplb_kernel_status(int clear) { return gemm_tcgen05_status(clear != 0); }

int rplb_linear_i8_i32(const int8_t* x, const int8_t* w, const int8_t* bias, int32_t* out,
                       uint64_t M, uint64_t K, uint64_t N, void* stream) {
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = N;
    p.b_is_kn = 0; p.mode = EPI_RAW_I32; p.bias_i8 = bias;
    return run_gemm(p, as_stream(stream));
}

int rplb_gemm_i8_requant_i32(const int8_t* A, const int8_t* B, int32_t* C, uint64_t M, uint64_t N, uint64_t K,
                             float sa, float sb, float sc, int32_t za, int32_t zb, void* stream) {
    GemmProblem p = {};
    p.A = A; p.B = B; p.out = C; p.M = M; p.N = N; p.K = K; p.ldo = N;
    p.b_is_kn = 1; p.mode = EPI_REQUANT_I32;
    p.sa = sa; p.sb = sb; p.sc = sc; p.za = za; p.zb = zb;
    return run_gemm(p, as_stream(stream));
}

int rplb_linear_i8_dequant_f32(const int8_t* x, const int8_t* w, float* out, uint64_t M, uint64_t K, uint64_t N,
                               uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                               int relu, void* stream) {
    if (!a_scale || !w_scales) return fail(RPLB_E_BAD_ARG, "rplb_linear_i8_dequant_f32: null scale pointer");
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu;
    return run_gemm(p, as_stream(stream));
}

}  // extern "C"
