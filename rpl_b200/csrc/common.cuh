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

// Scratch memory owned by the library, one block per (device, stream, host
// thread), allocated with cudaMalloc on first use and grown when a call needs
// more.  Contents: [0, 64) control words kept zero between calls (ticket
// counters), then `bytes` of uninitialised space.  One thread's calls on one
// stream are ordered by the stream, so they can share it; another thread's
// kernels may be queued between two kernels of a call, so it gets its own.
struct Scratch {
    unsigned int* control;   // 16 words, zero at kernel entry, kernels restore zero
    void* data;              // at least the requested size, 256-byte aligned
};
int scratch_for(cudaStream_t stream, size_t bytes, Scratch* out);

int sm_count();              // SMs of the current device (cached per device)

// The device allocator in use (cudaMalloc / cudaFree, or what rplb_set_allocator installed).
int device_alloc(void** p, size_t bytes, const char* what);
int device_free(void* p);

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

// Four int32 -> four int8 with saturation to [-128,127], a in the lowest byte.
__device__ __forceinline__ uint32_t pack4_sat_i8(int32_t a, int32_t b, int32_t c, int32_t d) {
    uint32_t hi, w;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(b), "r"(a), "r"(hi));
    return w;
}

// Per-tensor (or per-channel) constants of the quantize fast path.
struct QuantConsts {
    float scale;
    float rcp;          // correctly rounded 1/scale
    int32_t zp;
    bool fast;          // scale and 1/scale are normal numbers
};
__device__ __forceinline__ QuantConsts make_quant_consts(float scale, int32_t zp) {
    QuantConsts c;
    c.scale = scale;
    c.zp = zp;
    c.rcp = __frcp_rn(scale);
    const float as = fabsf(scale), ar = fabsf(c.rcp);
    c.fast = (as >= 1.17549435e-38f) && (as < INFINITY) && (ar >= 1.17549435e-38f) && (ar < INFINITY);
    return c;
}

// (int32)roundf(x / scale) without a division or a float->int conversion per
// element.  v = x * (1/scale) differs from the correctly rounded quotient
// RN(x/scale) by less than |v| * 2^-22 (two roundings of 2^-24 each, with
// margin), so both round to the same integer whenever v is farther than that
// from the nearest half-integer; `slow` is raised otherwise (and for NaN or
// |v| >= 2^22) and the caller recomputes with the exact path.
//   t = v + 1.5*2^23          the add rounds v to the nearest integer (ties to even)
//   bits(t) - 0x4B400000      that integer, two's complement
//   f = t - 1.5*2^23          the same integer as a float, exact
//   d = v - f                 in [-0.5, 0.5]; |d| = 0.5 exactly at a tie
// Away from ties, nearest-even and roundf's ties-away agree; ties are sent to
// the exact path by the same test that guards the reciprocal.
__device__ __forceinline__ int32_t quotient_round_fast(float x, float rcp, bool& slow) {
    const float v = __fmul_rn(x, rcp);
    const float t = __fadd_rn(v, 12582912.0f);
    const float d = __fsub_rn(v, __fsub_rn(t, 12582912.0f));
    const float e = __fmaf_rn(fabsf(v), 2.384185791015625e-07f, fabsf(d));     // |v| * 2^-22 + |d|
    slow = slow || !(e < 0.5f);
    return __float_as_int(t) - 0x4B400000;
}

// Four elements at once: fast path, exact path for the whole quad when any
// element needs it.  Same value as four quantize_one() calls, packed.
__device__ __forceinline__ uint32_t quantize_quad_packed(float4 v, const QuantConsts& c) {
    if (c.fast) {
        bool slow = false;
        const int32_t q0 = quotient_round_fast(v.x, c.rcp, slow);
        const int32_t q1 = quotient_round_fast(v.y, c.rcp, slow);
        const int32_t q2 = quotient_round_fast(v.z, c.rcp, slow);
        const int32_t q3 = quotient_round_fast(v.w, c.rcp, slow);
        // |q| < 2^22 here, so adding a zero point cannot wrap unless |zp| is
        // within 2^22 of the int32 limits; that case takes the exact path.
        if (!slow && ((uint32_t)c.zp + 0x40000000u) < 0x80000000u)
            return pack4_sat_i8(q0 + c.zp, q1 + c.zp, q2 + c.zp, q3 + c.zp);
    }
    return pack4_i8(quantize_one(v.x, c.scale, c.zp), quantize_one(v.y, c.scale, c.zp),
                    quantize_one(v.z, c.scale, c.zp), quantize_one(v.w, c.scale, c.zp));
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
