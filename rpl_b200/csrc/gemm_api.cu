// C ABI of the INT8 contraction: argument checks, choice of kernel, and the
// [K,N] -> [N,K] transpose that lets gemm_int8's B layout reach the
// tensor-core kernel.
#include "gemm_common.cuh"
#include <atomic>

namespace rplb {

int gemm_tcgen05_status(bool clear);     // gemm_i8_tcgen05.cu
int bounded_wait_selftest(cudaStream_t st);
int bounded_wait_leave_status(cudaStream_t st);

// Per host thread: 0 auto, 1 dp4a, 2 tcgen05, 3 tcgen05 128x256 tiles, 4 tcgen05 CTA pair, 5 tcgen05 256x256 tiles per CTA,
// 6 tcgen05 kernel for few output features
static thread_local int t_backend = 0;
int thread_gemm_backend(int which) {
    const int prev = t_backend;
    if (which >= 0 && which <= 6) t_backend = which;
    return prev;
}

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

// sums[r] = sum_k X[r,k] of a row-major [rows, K] int8 matrix: one warp per row,
// 16-byte loads when the row allows it, dp4a against a word of ones.
__global__ void row_sums_i8_kernel(const int8_t* __restrict__ X, int32_t* __restrict__ sums, uint64_t rows, uint64_t K) {
    const uint64_t row = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int8_t* x = X + row * K;
    int32_t acc = 0;
    if ((((uintptr_t)x & 15) == 0) && (K % 16 == 0)) {
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        for (uint64_t i = lane; i < K / 16; i += 32) {
            uint4 v = __ldg(x4 + i);
            acc = __dp4a((int)v.x, 0x01010101, acc);
            acc = __dp4a((int)v.y, 0x01010101, acc);
            acc = __dp4a((int)v.z, 0x01010101, acc);
            acc = __dp4a((int)v.w, 0x01010101, acc);
        }
    } else {
        for (uint64_t i = lane; i < K; i += 32) acc += (int32_t)x[i];
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) sums[row] = acc;
}

// sums[n] = sum_k B[k,n] of a row-major [K, N] int8 matrix: 32 consecutive columns per
// CTA (coalesced along N), 8 K-slices per CTA folded through shared memory.
__global__ void col_sums_i8_kernel(const int8_t* __restrict__ B, int32_t* __restrict__ sums, uint64_t K, uint64_t N) {
    __shared__ int32_t part[8][33];
    const uint64_t n = (uint64_t)blockIdx.x * 32 + threadIdx.x;
    int32_t acc = 0;
    if (n < N)
        for (uint64_t k = threadIdx.y; k < K; k += 8) acc += (int32_t)__ldg(B + k * N + n);
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && n < N) {
        #pragma unroll
        for (int j = 1; j < 8; j++) acc += part[j][threadIdx.x];
        sums[n] = acc;
    }
}

// scale = absmax / 127.0f (src/rpl_quantization.c:87-88) from the value the GEMM epilogue accumulated.
__global__ void absmax_to_scale_kernel(const float* __restrict__ absmax, float* __restrict__ scale) {
    *scale = __fdiv_rn(*absmax, 127.0f);
}

static int launch_row_sums(const int8_t* X, int32_t* sums, uint64_t rows, uint64_t K, cudaStream_t st) {
    const unsigned int warps = 8;
    row_sums_i8_kernel<<<(unsigned int)((rows + warps - 1) / warps), warps * 32, 0, st>>>(X, sums, rows, K);
    return launched("row_sums_i8_kernel");
}

int run_gemm(GemmProblem p, cudaStream_t st) {
    if (p.M == 0 || p.N == 0) return 0;
    // An operand with no elements (K = 0) may legitimately be a null pointer.
    if ((!p.A || !p.B) && p.K) return fail(RPLB_E_BAD_ARG, "INT8 GEMM: null input pointer");
    if (!p.out) return fail(RPLB_E_BAD_ARG, "INT8 GEMM: null output pointer");
    if (p.ldo < p.N) return fail(RPLB_E_BAD_ARG, "INT8 GEMM: output row stride %llu < N %llu",
                                 (unsigned long long)p.ldo, (unsigned long long)p.N);
    const int backend = t_backend;
    if (backend == 1) return gemm_simt(p, st);

    GemmProblem q = p;
    const bool big = (double)p.M * (double)p.N * (double)(p.K ? p.K : 1) >= (double)kTcMinMacs;
    // What the tensor-core kernel will need once B is K-contiguous: K % 16 == 0 and
    // 16-byte aligned operands (the transposed copy in scratch is aligned by construction).
    const bool want_tc = (backend >= 2 || big) && p.K && p.K % 16 == 0 && (((uintptr_t)p.A & 15) == 0) &&
                         (p.b_is_kn || (((uintptr_t)p.B & 15) == 0));
    const bool zero_points = p.mode == EPI_REQUANT_I32 && (p.za || p.zb);
    // gemm_int8's B[K,N] goes to the tensor cores as it lies (MN-major operand) when its rows are
    // 16-byte multiples; backends 4 and 5 get a transposed, K-contiguous copy instead.
    const bool b_in_place = p.b_is_kn && p.N % 16 == 0 && (((uintptr_t)p.B & 15) == 0) &&
                            (backend == 0 || backend == 2 || backend == 3);
    if (backend == 6 && (p.b_is_kn || zero_points)) return fail(RPLB_E_UNSUPPORTED, "the kernel for few output features takes W as [N,K] and no zero points");
    if (want_tc && b_in_place && zero_points) {
        // Row sums of A and column sums of B, both taken from the operands as they lie.
        const size_t rs_bytes = ((size_t)p.M * 4 + 255) & ~(size_t)255;
        Scratch sc;
        if (int rc = scratch_for(st, rs_bytes + (size_t)p.N * 4, &sc)) return rc;
        int32_t* rs = reinterpret_cast<int32_t*>(sc.data);
        int32_t* cs = reinterpret_cast<int32_t*>(static_cast<char*>(sc.data) + rs_bytes);
        if (int rc = launch_row_sums(p.A, rs, p.M, p.K, st)) return rc;
        col_sums_i8_kernel<<<(unsigned int)((p.N + 31) / 32), dim3(32, 8), 0, st>>>(p.B, cs, p.K, p.N);
        if (int rc = launched("col_sums_i8_kernel")) return rc;
        q.a_row_sums = rs;
        q.b_col_sums = cs;
    }
    if (want_tc && !b_in_place && (p.b_is_kn || zero_points) && (p.K + 31) / 32 <= 65535) {
        // Library scratch: [ B as [N,K] | row sums of A | column sums of B ].
        const size_t bt_bytes = p.b_is_kn ? (((size_t)(p.K * p.N) + 255) & ~(size_t)255) : 0;
        const size_t rs_bytes = zero_points ? (((size_t)p.M * 4 + 255) & ~(size_t)255) : 0;
        const size_t cs_bytes = zero_points ? (size_t)p.N * 4 : 0;
        Scratch sc;
        if (int rc = scratch_for(st, bt_bytes + rs_bytes + cs_bytes, &sc)) return rc;
        char* base = static_cast<char*>(sc.data);
        if (p.b_is_kn) {
            // Reorder B once into the K-contiguous layout the tensor-core kernel reads.
            dim3 grid((unsigned int)((p.N + 31) / 32), (unsigned int)((p.K + 31) / 32)), block(32, 8);
            transpose_i8_kernel<<<grid, block, 0, st>>>(p.B, reinterpret_cast<int8_t*>(base), p.K, p.N);
            if (int rc = launched("transpose_i8_kernel")) return rc;
            q.B = reinterpret_cast<const int8_t*>(base);
            q.b_is_kn = 0;
        }
        if (zero_points && !q.b_is_kn) {
            int32_t* rs = reinterpret_cast<int32_t*>(base + bt_bytes);
            int32_t* cs = reinterpret_cast<int32_t*>(base + bt_bytes + rs_bytes);
            if (int rc = launch_row_sums(q.A, rs, p.M, p.K, st)) return rc;
            if (int rc = launch_row_sums(q.B, cs, p.N, p.K, st)) return rc;      // rows of [N,K] = columns of B
            q.a_row_sums = rs;
            q.b_col_sums = cs;
        }
    }
    if (backend >= 2) return gemm_tcgen05(q, st, backend - 2);
    if (big && gemm_tcgen05_supports(q)) return gemm_tcgen05(q, st);
    return gemm_simt(p, st);
}

}  // namespace rplb

using namespace rplb;

extern "C" {

int rplb_gemm_backend(int which) { return thread_gemm_backend(which); }

int rplb_gemm_epilogue(int which) { return thread_gemm_epilogue(which); }

int rplb_selftest_bounded_wait_keep(void* stream) { return bounded_wait_leave_status(as_stream(stream)); }

int rplb_kernel_status(int clear) { return gemm_tcgen05_status(clear != 0); }

int rplb_selftest_bounded_wait(void* stream) { return bounded_wait_selftest(as_stream(stream)); }

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

int rplb_linear_i8_dequant_f32_absmax(const int8_t* x, const int8_t* w, float* out, uint64_t M, uint64_t K, uint64_t N,
                                      uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                                      int relu, float* absmax, float* next_scale, void* stream) {
    if (!a_scale || !w_scales || !absmax) return fail(RPLB_E_BAD_ARG, "rplb_linear_i8_dequant_f32_absmax: null pointer");
    cudaStream_t st = as_stream(stream);
    if (int rc = cuda_ok(cudaMemsetAsync(absmax, 0, sizeof(float), st), "cudaMemsetAsync(absmax)")) return rc;
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu; p.absmax_out = absmax;
    int folded = 0;
    p.next_scale = next_scale; p.next_scale_done = &folded;
    if (int rc = run_gemm(p, st)) return rc;
    if (next_scale && !folded) {
        absmax_to_scale_kernel<<<1, 1, 0, st>>>(absmax, next_scale);
        return launched("absmax_to_scale_kernel");
    }
    return 0;
}

int rplb_linear_i8_dequant_f32_peers(const int8_t* x, const int8_t* w, float* out, uint64_t M, uint64_t K, uint64_t N,
                                     uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                                     int relu, float* const* peer_out, int n_peers, void* stream) {
    const char* who = "rplb_linear_i8_dequant_f32_peers";
    if (!a_scale || !w_scales) return fail(RPLB_E_BAD_ARG, "%s: null scale pointer", who);
    if (n_peers < 0 || n_peers > kMaxPeers) return fail(RPLB_E_BAD_ARG, "%s: %d peers (at most %d)", who, n_peers, kMaxPeers);
    if (n_peers > 0 && !peer_out) return fail(RPLB_E_BAD_ARG, "%s: null peer list", who);
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu;
    for (int i = 0; i < n_peers; i++) {
        if (!peer_out[i]) return fail(RPLB_E_BAD_ARG, "%s: peer destination %d is null", who, i);
        p.peer_out[i] = peer_out[i];
    }
    p.n_peers = n_peers;
    if (n_peers == 0) return run_gemm(p, as_stream(stream));
    if (M == 0 || N == 0) return 0;
    if (!x || !w || !out) return fail(RPLB_E_BAD_ARG, "%s: null pointer", who);
    if (ldo < N) return fail(RPLB_E_BAD_ARG, "%s: output row stride %llu < N %llu", who, (unsigned long long)ldo, (unsigned long long)N);
    // Only the tensor-core kernel stores to peer destinations; there is no other route.
    if (!gemm_tcgen05_supports(p))
        return fail(RPLB_E_UNSUPPORTED, "%s: needs K %% 16 == 0 and 16-byte aligned x and w", who);
    return gemm_tcgen05(p, as_stream(stream), 1);
}

int rplb_quantize_linear_dequant_f32(const float* x, const int8_t* w, float* out, uint64_t M, uint64_t K, uint64_t N,
                                     uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                                     int relu, float* absmax, float* next_scale, void* stream) {
    const char* who = "rplb_quantize_linear_dequant_f32";
    if (!a_scale || !w_scales) return fail(RPLB_E_BAD_ARG, "%s: null scale pointer", who);
    if (next_scale && !absmax) return fail(RPLB_E_BAD_ARG, "%s: next_scale needs absmax", who);
    if (M == 0 || N == 0) return 0;
    if (!x || !w || !out) return fail(RPLB_E_BAD_ARG, "%s: null pointer", who);
    if (ldo < N) return fail(RPLB_E_BAD_ARG, "%s: output row stride %llu < N %llu", who, (unsigned long long)ldo, (unsigned long long)N);
    cudaStream_t st = as_stream(stream);
    GemmProblem p = {};
    p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu; p.absmax_out = absmax;
    const bool small = quantize_linear_small_supports(x, p), tc = gemm_fused_quant_supports(x, p);
    if (!small && !tc)
        return fail(RPLB_E_UNSUPPORTED, "%s: needs N <= 128 with K <= 896 and K %% 16 == 0, or N <= 16 with K <= 512 and K %% 4 == 0; "
                    "quantize into a buffer and call rplb_linear_i8_dequant_f32 instead", who);
    if (absmax) if (int rc = cuda_ok(cudaMemsetAsync(absmax, 0, sizeof(float), st), "cudaMemsetAsync(absmax)")) return rc;
    int folded = 0;
    p.next_scale = next_scale; p.next_scale_done = &folded;
    if (int rc = small ? quantize_linear_small(x, p, st) : gemm_fused_quant(x, p, st)) return rc;
    if (next_scale && !folded) {
        absmax_to_scale_kernel<<<1, 1, 0, st>>>(absmax, next_scale);
        return launched("absmax_to_scale_kernel");
    }
    return 0;
}

int rplb_linear_i8_dequant_f32_arriving(const int8_t* x, const int8_t* w, float* out, uint64_t M, uint64_t K, uint64_t N,
                                        uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                                        int relu, const uint32_t* row_block_ready, uint32_t epoch,
                                        uint32_t local_first_block, uint32_t local_blocks, void* stream) {
    const char* who = "rplb_linear_i8_dequant_f32_arriving";
    if (!a_scale || !w_scales) return fail(RPLB_E_BAD_ARG, "%s: null scale pointer", who);
    if (M == 0 || N == 0) return 0;
    if (!x || !w || !out) return fail(RPLB_E_BAD_ARG, "%s: null pointer", who);
    if (!row_block_ready) return fail(RPLB_E_BAD_ARG, "%s: null arrival words", who);
    if (ldo < N) return fail(RPLB_E_BAD_ARG, "%s: output row stride %llu < N %llu", who, (unsigned long long)ldo, (unsigned long long)N);
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu;
    p.a_ready = row_block_ready; p.a_epoch = epoch; p.a_local_first = local_first_block; p.a_local_count = local_blocks;
    // Only the tensor-core kernel waits for arriving rows; there is no other route.
    if (!gemm_tcgen05_supports(p))
        return fail(RPLB_E_UNSUPPORTED, "%s: needs K %% 16 == 0 and 16-byte aligned x and w", who);
    const int asked = t_backend;         // 5: the 256 x 256 kernel, 3: the 128 x 256 kernel, else the library's choice of the two
    return gemm_tcgen05(p, as_stream(stream), asked == 3 ? 1 : asked == 5 ? 3 : 0);
}

int rplb_linear_i8_requant_i8(const int8_t* x, const int8_t* w, int8_t* out, uint64_t M, uint64_t K, uint64_t N,
                              uint64_t ldo, const float* a_scale, const float* w_scales, const float* bias,
                              int relu, const float* out_scale, int32_t out_zero_point, void* stream) {
    if (!a_scale || !w_scales || !out_scale) return fail(RPLB_E_BAD_ARG, "rplb_linear_i8_requant_i8: null scale pointer");
    GemmProblem p = {};
    p.A = x; p.B = w; p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_I8;
    p.a_scale = a_scale; p.w_scales = w_scales; p.bias_f32 = bias; p.relu = relu;
    p.out_scale = out_scale; p.out_zp = out_zero_point;
    return run_gemm(p, as_stream(stream));
}

}  // extern "C"
