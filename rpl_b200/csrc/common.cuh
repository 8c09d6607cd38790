// Shared plumbing of the CUDA side of librpl.so: error reporting, launch
// counting, per-stream scratch memory and the scalar arithmetic that must
// match the reference's x86-64 build bit for bit.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <float.h>
#include <limits.h>
#include "rpl_b200.h"

namespace rplb {

// Records `code` with a printf-style text for rplb_last_error() and returns it.
int fail(int code, const char* fmt, ...);
// cudaSuccess -> 0; otherwise records the CUDA error text and returns the code.
int cuda_ok(cudaError_t e, const char* what);
// Checks the launch that was just issued and counts it.
int launched(const char* kernel);

// Scratch memory owned by the library, one block per (device, stream),
// allocated with cudaMalloc on first use and grown when a call needs more.
// Contents: [0, 64) control words kept zero between calls (ticket counters),
// then `bytes` of uninitialised space.  Calls on the same stream are ordered
// by the stream, so they can share it.
struct Scratch {
    unsigned int* control;   // 16 words, zero at kernel entry, kernels restore zero
    void* data;              // at least the requested size, 256-byte aligned
};
int scratch_for(cudaStream_t stream, size_t bytes, Scratch* out);

int sm_count();              // SMs of the current device (cached per device)

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ---------------------------------------------------------------------------
// Device arithmetic with the reference's x86-64 semantics.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
// (int32_t)v as cvttss2si does it: NaN and anything outside int32 give INT_MIN
// (src/rpl_core.c:523 compiled for x86-64).
__device__ __forceinline__ int32_t f2i_x86(float v) {
    int32_t i = __float2int_rz(v);
    return (fabsf(v) < 2147483648.0f) ? i : INT_MIN;
}

// roundf(v): ties away from zero.  truncf(v + copysignf(0.49999997f, v))
// equals roundf(v) for every non-NaN float (checked exhaustively on the
// host: all 2^32 bit patterns); NaN stays NaN.
__device__ __forceinline__ float round_half_away(float v) {
    return truncf(__fadd_rn(v, copysignf(0.49999997f, v)));
}

// (int32_t)roundf(v) with both of the above in one conversion.
__device__ __forceinline__ int32_t round_to_i32_x86(float v) {
    float s = __fadd_rn(v, copysignf(0.49999997f, v));
    int32_t i = __float2int_rz(s);
    return (fabsf(s) < 2147483648.0f) ? i : INT_MIN;
}

// clamp((int32)roundf(x / scale) + zp, -128, 127)   src/rpl_core.c:523-526
// The division is IEEE round-to-nearest; the zero point is added with
// two's-complement wrap before the clamp.
__device__ __forceinline__ int32_t quantize_one(float x, float scale, int32_t zp) {
    int32_t q = round_to_i32_x86(__fdiv_rn(x, scale));
    q = (int32_t)((uint32_t)q + (uint32_t)zp);
    return max(-128, min(127, q));
}

__device__ __forceinline__ uint32_t pack4_i8(int32_t a, int32_t b, int32_t c, int32_t d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)d << 24);
}

__device__ __forceinline__ float warp_min(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
#endif  // __CUDACC__

}  // namespace rplb
