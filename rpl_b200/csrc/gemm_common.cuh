// What the two contraction kernels (dp4a and tcgen05) share: the description of
// a problem and the three epilogues of the path.
#pragma once
#include "common.cuh"

namespace rplb {

enum EpilogueMode : int {
    EPI_RAW_I32 = 0,      // linear_int8: raw accumulator (+ int8 bias)      src/rpl_quantization.c:346-350
    EPI_REQUANT_I32 = 1,  // gemm_int8: roundf(sum*sa*sb/sc) as int32        src/ops_extended.c:119-120
    EPI_DEQUANT_F32 = 2,  // fused fp32: ((float)acc*sA)*sW[n] + bias[n], optional ReLU
    EPI_DEQUANT_I8 = 3,   // the same fp32 value quantized straight to int8 with a given output scale / zero point
};

constexpr int kMaxPeers = 7;          // a node of 8 GPUs: this rank and seven others

struct GemmProblem {
    const int8_t* A;      // [M,K] row-major
    const int8_t* B;      // b_is_kn ? [K,N] row-major : [N,K] row-major
    void* out;            // int32 or float, [M, ldo]
    uint64_t M, N, K, ldo;
    int b_is_kn;
    int mode;
    // EPI_RAW_I32
    const int8_t* bias_i8;
    // EPI_REQUANT_I32
    float sa, sb, sc;
    int32_t za, zb;
    const int32_t* a_row_sums;   // sum_k A[m,k], needed by kernels that cannot subtract zero points in the loop
    const int32_t* b_col_sums;   // sum_k B[k,n]
    // EPI_DEQUANT_F32
    const float* a_scale;     // one float on the device
    const float* w_scales;    // N floats
    const float* bias_f32;    // N floats or null
    int relu;
    float* absmax_out;        // optional: max |out| over the call is folded in here (bits of a non-negative float)
    // Optional, with absmax_out: the next layer's activation scale, *absmax_out / 127 (src/rpl_quantization.c:87-88).
    // A launcher whose kernel writes it (its last warp through, counted on `ticket`, a device word that is zero at
    // rest) sets *next_scale_done, a host flag; otherwise the caller launches the one-thread kernel that divides.
    float* next_scale;
    unsigned int* ticket;
    int* next_scale_done;
    // EPI_DEQUANT_I8
    const float* out_scale;   // one float on the device
    int32_t out_zp;
    // EPI_DEQUANT_F32 only: further [M, ldo] destinations that receive the same
    // values as `out` (buffers of other GPUs mapped into this process).
    int n_peers;
    float* peer_out[kMaxPeers];
    // Rows of A that other GPUs deliver while the kernel runs (tensor-core kernel
    // with 128-row tiles only).  a_ready[t] belongs to rows [128 t, 128 t + 128):
    // the block is in place once (int32)(a_ready[t] - a_epoch) >= 0.  Blocks
    // [a_local_first, a_local_first + a_local_count) are in place at launch; the
    // kernel starts with them and takes the others in ascending order, wrapping
    // round.  a_ready == nullptr: all of A is in place at launch.
    const uint32_t* a_ready;
    uint32_t a_epoch;
    uint32_t a_local_first, a_local_count;
};

#ifdef __CUDACC__
// Requantize as the scalar branch of gemm_int8_fallback does: three fp32
// operations left to right, then roundf and the x86 float->int conversion.
__device__ __forceinline__ int32_t requant_i32(int32_t sum, float sa, float sb, float sc) {
    float r = __fmul_rn(__int2float_rn(sum), sa);
    r = __fmul_rn(r, sb);
    r = __fdiv_rn(r, sc);
    return round_to_i32_x86(r);
}

// One output value of the fused fp32 epilogue; each step is rounded on its own
// (no fused multiply-add), in the order the CPU restatement uses.
__device__ __forceinline__ float dequant_f32(int32_t acc, float a_scale, float w_scale, bool has_bias,
                                             float bias, bool relu) {
    float v = __fmul_rn(__int2float_rn(acc), a_scale);
    v = __fmul_rn(v, w_scale);
    if (has_bias) v = __fadd_rn(v, bias);
    if (relu && v < 0.0f) v = 0.0f;
    return v;
}
#endif

#ifdef __CUDACC__
// sum_k (a-za)(b-zb) from the plain product and the row / column sums, mod 2^32.
__device__ __forceinline__ int32_t apply_zero_points(int32_t sum, int32_t row_sum, int32_t col_sum, int32_t za, int32_t zb, uint32_t K) {
    uint32_t s = (uint32_t)sum;
    s -= (uint32_t)zb * (uint32_t)row_sum;
    s -= (uint32_t)za * (uint32_t)col_sum;
    s += K * (uint32_t)za * (uint32_t)zb;
    return (int32_t)s;
}

// Folds |v| into a running maximum kept as the bit pattern of a non-negative
// float (such patterns order like unsigned integers).  NaN is skipped, as the
// reference's min/max compares skip it.
__device__ __forceinline__ void absmax_fold(float& running, float v) {
    running = fmaxf(running, fabsf(v));         // fmaxf returns the other operand for a NaN
}
__device__ __forceinline__ void absmax_publish(float* dst, float running) {
    running = warp_max(running);
    if ((threadIdx.x & 31) == 0 && running > 0.0f) atomicMax(reinterpret_cast<unsigned int*>(dst), __float_as_uint(running));
}
#endif

// Implemented in gemm_i8_simt.cu / gemm_i8_tcgen05.cu.
int gemm_simt(const GemmProblem& p, cudaStream_t st);
// variant: 0 = choose, 1 = one CTA per 128 x 256 tile, 2 = a CTA pair (two SMs) per 256 x 256 tile,
// 3 = one CTA per 256 x 256 tile.
int gemm_tcgen05(const GemmProblem& p, cudaStream_t st, int variant = 0);
// Which contraction kernel and which store path this host thread's calls use (rplb_gemm_backend, rplb_gemm_epilogue).
int thread_gemm_backend(int which);
int thread_gemm_epilogue(int which);
// Quantize fused into the contraction's A side: x is fp32 [M,K] and is quantized with *p.a_scale on its way
// in (p.A is not used).  gemm_fused_quant: tensor cores, N <= 128 and K <= 896; quantize_linear_small: dp4a,
// N <= 16 and K <= 512.  Both: fp32 epilogue only.
bool gemm_fused_quant_supports(const float* x, const GemmProblem& p);
int gemm_fused_quant(const float* x, const GemmProblem& p, cudaStream_t st);
// The same kernel for an activation that is int8 already: the contraction for few output features (whole weight
// matrix resident in shared memory, 128-column accumulators, fp32 epilogue only).
bool gemm_narrow_supports(const GemmProblem& p);
int gemm_narrow(const GemmProblem& p, cudaStream_t st);
bool quantize_linear_small_supports(const float* x, const GemmProblem& p);
int quantize_linear_small(const float* x, const GemmProblem& p, cudaStream_t st);
// Argument checks and choice of kernel for one contraction (gemm_api.cu).
int run_gemm(GemmProblem p, cudaStream_t st);
// True when the tensor-core kernel can take the problem as it stands.
bool gemm_tcgen05_supports(const GemmProblem& p);

}  // namespace rplb
