// Memory-bound kernels of the path: min/max reduction, fp32 -> int8 quantize
// (per tensor and per channel) and int8 -> fp32 dequantize.
//
// Data layout: tensors are flat, contiguous, row-major.  The vector paths view
// them as "quads": one float4 (16 B) in, one packed int8x4 word (4 B) out, or
// the reverse.  A warp touches 32 consecutive quads per instruction, so every
// load is 512 contiguous bytes and every store 128 (quantize) or the other way
// round (dequantize).  Buffers whose base address does not allow that
// (fp32 side not 16-byte aligned, int8 side not 4-byte aligned) take the
// scalar kernels, which compute the same values.
#include "common.cuh"
#include <atomic>
#include <mutex>

namespace rplb {

int* kernel_status_word_device();   // gemm_i8_tcgen05.cu: the calling host thread's status word, as the device sees it

constexpr int kThreads = 256;       // threads per CTA in the streaming kernels
constexpr int kUnroll = 4;          // quads per thread per grid-stride step
constexpr int kCtasPerSm = 8;       // 2048 resident threads per SM

static inline unsigned int stream_grid(uint64_t work_items, uint64_t items_per_cta) {
    uint64_t need = (work_items + items_per_cta - 1) / items_per_cta;
    uint64_t cap = (uint64_t)sm_count() * kCtasPerSm;
    if (cap == 0) cap = 148 * kCtasPerSm;
    if (need < 1) need = 1;
    return (unsigned int)(need < cap ? need : cap);
}

// One CTA per `items_per_cta` items (the kernels' grid-stride loops then run once).
static inline unsigned int one_shot_grid(uint64_t work_items, uint64_t items_per_cta) {
    uint64_t need = (work_items + items_per_cta - 1) / items_per_cta;
    if (need < 1) need = 1;
    return (unsigned int)(need < 0x7fffffffull ? need : 0x7fffffffull);
}

// ---------------------------------------------------------------------------
// min/max  (src/ops_extended.c:52-61, src/rpl_quantization.c:79-85)
// ---------------------------------------------------------------------------
// Every CTA reduces a grid-stride slice to one (min,max) pair in scratch, takes
// a ticket, and the CTA that draws the last ticket folds the pairs and writes
// the derived parameters.  fminf/fmaxf return the other operand when one is
// NaN, which is what the reference's strict compares amount to (a NaN never
// replaces the running value).
__device__ __forceinline__ void finalize_params(float lo, float hi, float first, rplb_qparams* p) {
    p->true_min = lo;
    p->true_max = hi;
    p->first = first;
    // Seeds of src/rpl_quantization.c:79: a tensor with no element below
    // FLT_MAX keeps the seed.
    float mn = fminf(lo, FLT_MAX);
    float mx = fmaxf(hi, -FLT_MAX);
    p->min_val = mn;
    p->max_val = mx;
    p->scale_sym = __fdiv_rn(fmaxf(fabsf(mn), fabsf(mx)), 127.0f);
    float range = __fsub_rn(mx, mn);
    float sa = __fdiv_rn(range, 255.0f);
    p->scale_asym = sa;
    p->zp_asym = round_to_i32_x86(__fdiv_rn(-mn, sa));
}

__global__ void __launch_bounds__(kThreads)
minmax_kernel(const float* __restrict__ x, uint64_t n, uint64_t head, uint64_t nquads,
              float2* __restrict__ partials, unsigned int* __restrict__ ticket,
              rplb_qparams* __restrict__ params) {
    float lo = INFINITY, hi = -INFINITY;
    const float4* xq = reinterpret_cast<const float4*>(x + head);
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
    // Main body: kUnroll independent 16-byte loads in flight per thread.
    for (; i + (kUnroll - 1) * stride < nquads; i += kUnroll * stride) {
        float4 v[kUnroll];
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) v[u] = __ldg(xq + i + u * stride);
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            lo = fminf(fminf(lo, v[u].x), fminf(v[u].y, fminf(v[u].z, v[u].w)));
            hi = fmaxf(fmaxf(hi, v[u].x), fmaxf(v[u].y, fmaxf(v[u].z, v[u].w)));
        }
    }
    for (; i < nquads; i += stride) {
        float4 v = __ldg(xq + i);
        lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));
        hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
    }
    // Unaligned head and the tail that does not fill a quad.
    if (blockIdx.x == 0) {
        uint64_t tail0 = head + nquads * 4;
        for (uint64_t j = threadIdx.x; j < head; j += kThreads) { float v = x[j]; lo = fminf(lo, v); hi = fmaxf(hi, v); }
        for (uint64_t j = tail0 + threadIdx.x; j < n; j += kThreads) { float v = x[j]; lo = fminf(lo, v); hi = fmaxf(hi, v); }
    }

    __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
    __shared__ bool s_last;
    lo = warp_min(lo);
    hi = warp_max(hi);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
    __syncthreads();
    if (warp == 0) {
        lo = lane < kThreads / 32 ? s_lo[lane] : INFINITY;
        hi = lane < kThreads / 32 ? s_hi[lane] : -INFINITY;
        lo = warp_min(lo);
        hi = warp_max(hi);
        if (lane == 0) {
            partials[blockIdx.x] = make_float2(lo, hi);
            __threadfence();
            unsigned int t = atomicAdd(ticket, 1u);
            s_last = (t == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    lo = INFINITY; hi = -INFINITY;
    for (unsigned int j = threadIdx.x; j < gridDim.x; j += kThreads) {
        float2 p = __ldcg(partials + j);
        lo = fminf(lo, p.x);
        hi = fmaxf(hi, p.y);
    }
    lo = warp_min(lo);
    hi = warp_max(hi);
    if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kThreads / 32; w++) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
        finalize_params(lo, hi, n ? x[0] : 0.0f, params);
        *ticket = 0;                 // leave the control word as it was found
    }
}

// A tensor whose rows are spread over several GPUs: each reduces its rows, the
// pairs (-min, max) are combined with one max-reduction across the GPUs, and
// the parameters are then derived from the combined pair by the very statements
// the single-GPU reduction ends with (IEEE division included).
__global__ void qparams_to_pair_kernel(const rplb_qparams* __restrict__ params, float* __restrict__ pair) {
    pair[0] = -params->true_min;
    pair[1] = params->true_max;
}
__global__ void qparams_from_pair_kernel(const float* __restrict__ pair, rplb_qparams* __restrict__ params) {
    finalize_params(-pair[0], pair[1], params->first, params);
}

// ---------------------------------------------------------------------------
// quantize  (src/rpl_core.c:521-527)
// ---------------------------------------------------------------------------

// REVERSE walks the tensor from its end: after a forward min/max pass the end
// of the tensor is what the L2 cache still holds.
template <bool REVERSE>
__global__ void __launch_bounds__(kThreads)
quantize_quads_kernel(const float4* __restrict__ x, uint32_t* __restrict__ q, uint64_t nquads,
                      float scale_imm, int32_t zp_imm,
                      const float* __restrict__ scale_dev, const int32_t* __restrict__ zp_dev) {
    const QuantConsts qc = make_quant_consts(scale_dev ? __ldg(scale_dev) : scale_imm, zp_dev ? __ldg(zp_dev) : zp_imm);
    // A CTA step covers kThreads*kUnroll consecutive quads; within it thread t
    // takes quads t, t+kThreads, ... so each warp instruction is contiguous.
    const uint64_t step = (uint64_t)kThreads * kUnroll;
    const uint64_t nsteps = (nquads + step - 1) / step;
    for (uint64_t s = blockIdx.x; s < nsteps; s += gridDim.x) {
        const uint64_t base = (REVERSE ? (nsteps - 1 - s) : s) * step + threadIdx.x;
        float4 v[kUnroll];
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nquads) v[u] = __ldcs(x + i);
        }
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nquads) __stcs(q + i, quantize_quad_packed(v[u], qc));
        }
    }
}

__global__ void __launch_bounds__(kThreads)
quantize_scalar_kernel(const float* __restrict__ x, int8_t* __restrict__ q, uint64_t begin, uint64_t n,
                       float scale_imm, int32_t zp_imm,
                       const float* __restrict__ scale_dev, const int32_t* __restrict__ zp_dev) {
    const float scale = scale_dev ? __ldg(scale_dev) : scale_imm;
    const int32_t zp = zp_dev ? __ldg(zp_dev) : zp_imm;
    for (uint64_t i = begin + (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kThreads)
        q[i] = (int8_t)quantize_one(x[i], scale, zp);
}

// ---------------------------------------------------------------------------
// Per-tensor quantize in one launch, for tensors that fit in the registers of
// one resident grid (up to a few million elements): tensor_quantize_int8_symmetric
// / _asymmetric (src/rpl_quantization.c:77-107) read the tensor twice because the
// scale depends on every element; here every thread keeps its quads in registers
// across a grid-wide barrier, so the tensor is read once (5 B/element instead of
// 9) and one launch replaces two.  The kernel is launched cooperatively (all CTAs
// resident, guaranteed by the driver); the barrier is a counter in the library's
// control words with a bounded wait, and the last CTA through puts the counters
// back to zero.
__device__ __forceinline__ void block_minmax(float& lo, float& hi, float* s_lo, float* s_hi);    // defined with the per-channel kernels

constexpr int kOnePassQuads = 8;                       // quads per thread kept in registers
constexpr uint64_t kOnePassCtaQuads = (uint64_t)kThreads * kOnePassQuads;

__global__ void __launch_bounds__(kThreads)
quantize_onepass_kernel(const float* __restrict__ x, int8_t* __restrict__ q, uint64_t n, uint64_t nquads, int asymmetric,
                        float2* __restrict__ partials, unsigned int* __restrict__ counters, rplb_qparams* __restrict__ params,
                        int* __restrict__ status) {
    __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
    __shared__ int s_abort;
    const float4* xq = reinterpret_cast<const float4*>(x);
    const uint64_t base = (uint64_t)blockIdx.x * kOnePassCtaQuads + threadIdx.x;
    float4 v[kOnePassQuads];
    float lo = INFINITY, hi = -INFINITY;
    #pragma unroll
    for (int u = 0; u < kOnePassQuads; u++) {
        const uint64_t i = base + (uint64_t)u * kThreads;
        if (i < nquads) v[u] = __ldcs(xq + i);
    }
    #pragma unroll
    for (int u = 0; u < kOnePassQuads; u++) {
        const uint64_t i = base + (uint64_t)u * kThreads;
        if (i < nquads) {
            lo = fminf(fminf(lo, v[u].x), fminf(v[u].y, fminf(v[u].z, v[u].w)));
            hi = fmaxf(fmaxf(hi, v[u].x), fmaxf(v[u].y, fmaxf(v[u].z, v[u].w)));
        }
    }
    // The up to three elements that do not fill a quad: thread t of CTA 0 takes element 4 nquads + t.
    float tail = 0.0f;
    const bool has_tail = blockIdx.x == 0 && nquads * 4 + threadIdx.x < n;
    if (has_tail) { tail = x[nquads * 4 + threadIdx.x]; lo = fminf(lo, tail); hi = fmaxf(hi, tail); }
    if (threadIdx.x == 0) s_abort = 0;
    block_minmax(lo, hi, s_lo, s_hi);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = make_float2(lo, hi);
        __threadfence();
        atomicAdd(&counters[0], 1u);
        // Grid-wide barrier: every CTA is resident (cooperative launch), so this ends; bounded all the same.
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile unsigned int*>(&counters[0]) < gridDim.x) {
            if (clock64() - t0 > 2000000000LL) { s_abort = 1; atomicCAS(status, 0, 7); break; }
            __nanosleep(64);
        }
        __threadfence();
    }
    __syncthreads();
    if (s_abort) return;
    lo = INFINITY; hi = -INFINITY;
    for (unsigned int j = threadIdx.x; j < gridDim.x; j += kThreads) {
        const float2 p = __ldcg(partials + j);
        lo = fminf(lo, p.x);
        hi = fmaxf(hi, p.y);
    }
    __syncthreads();                                   // s_lo / s_hi are reused
    block_minmax(lo, hi, s_lo, s_hi);
    // Every CTA derives the same parameters from the same pairs; CTA 0 also writes them out.
    __shared__ rplb_qparams s_params;
    if (threadIdx.x == 0) {
        finalize_params(lo, hi, n ? x[0] : 0.0f, &s_params);
        if (blockIdx.x == 0) *params = s_params;
        // Leave the counters as they were found: the last CTA to get here resets them.
        if (atomicAdd(&counters[1], 1u) == gridDim.x - 1) { counters[0] = 0; counters[1] = 0; }
    }
    __syncthreads();
    const QuantConsts qc = make_quant_consts(asymmetric ? s_params.scale_asym : s_params.scale_sym, asymmetric ? s_params.zp_asym : 0);
    uint32_t* out = reinterpret_cast<uint32_t*>(q);
    #pragma unroll
    for (int u = 0; u < kOnePassQuads; u++) {
        const uint64_t i = base + (uint64_t)u * kThreads;
        if (i < nquads) __stcs(out + i, quantize_quad_packed(v[u], qc));
    }
    if (has_tail) q[nquads * 4 + threadIdx.x] = (int8_t)quantize_one(tail, qc.scale, qc.zp);
}

// How many CTAs of the kernel above can be resident on the current device (0 = cooperative launches unsupported).
static unsigned int onepass_capacity() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64 && cached[dev].load() != 0) return (unsigned int)(cached[dev].load() > 0 ? cached[dev].load() : 0);
    int coop = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) coop = 0;
    if (coop && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_onepass_kernel, kThreads, 0) != cudaSuccess) per_sm = 0;
    cudaGetLastError();
    const int cap = coop ? per_sm * sm_count() : 0;
    if (dev >= 0 && dev < 64) cached[dev].store(cap > 0 ? cap : -1);
    return cap > 0 ? (unsigned int)cap : 0;
}

// 1 = the one-launch path may be taken (per host thread; rplb_quantize_onepass switches it off for measurements).
static thread_local int t_onepass = 1;

// Tries the one-launch path; *done = false when the tensor does not qualify (too large, unaligned).
static int launch_quantize_onepass(const float* x, int8_t* q, uint64_t n, rplb_qparams* params, int asymmetric, cudaStream_t st, bool* done) {
    *done = false;
    if (!t_onepass || n < 4 || !x || !q || !params) return 0;
    if (((uintptr_t)x & 15) || ((uintptr_t)q & 3)) return 0;
    const uint64_t nquads = n / 4;
    const uint64_t ctas = (nquads + kOnePassCtaQuads - 1) / kOnePassCtaQuads;
    const unsigned int cap = onepass_capacity();
    if (cap == 0 || ctas > cap) return 0;
    Scratch sc;
    if (int rc = scratch_for(st, (size_t)ctas * sizeof(float2), &sc)) return rc;
    int* status_dev = kernel_status_word_device();
    if (!status_dev) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
    float2* partials = static_cast<float2*>(sc.data);
    unsigned int* counters = sc.control + 2;            // words 2 and 3 of the control block (zero at rest)
    uint64_t n_arg = n, nq_arg = nquads;
    void* args[] = {(void*)&x, (void*)&q, (void*)&n_arg, (void*)&nq_arg, (void*)&asymmetric, (void*)&partials, (void*)&counters,
                    (void*)&params, (void*)&status_dev};
    if (int rc = cuda_ok(cudaLaunchCooperativeKernel((const void*)quantize_onepass_kernel, dim3((unsigned int)ctas), dim3(kThreads), args, 0, st),
                         "cudaLaunchCooperativeKernel(quantize_onepass_kernel)")) return rc;
    *done = true;
    return launched("quantize_onepass_kernel");
}

static int launch_quantize(const float* x, int8_t* q, uint64_t n, float scale, int32_t zp,
                           const float* scale_dev, const int32_t* zp_dev, bool reverse, cudaStream_t st) {
    if (n == 0) return 0;
    if (!x || !q) return fail(RPLB_E_BAD_ARG, "quantize: null pointer");
    if ((uintptr_t)x & 3) return fail(RPLB_E_BAD_ARG, "quantize: fp32 input not 4-byte aligned");
    const bool vec = (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 3) == 0);
    uint64_t nquads = vec ? n / 4 : 0;
    if (nquads) {
        // One CTA per step rather than a resident grid striding over the tensor: measured
        // 3-4 % faster for the forward walk (6531 vs 6302 GB/s at 2^26 elements, 6853 vs 6581 at 2^30).
        // The reversed walk after a min/max pass keeps the resident grid while the tensor is within a
        // few L2 sizes, where it re-uses more of what that pass left in L2 (6307 vs 6114 GB/s at 2^26).
        unsigned int grid = one_shot_grid(nquads, (uint64_t)kThreads * kUnroll);
        if (reverse && nquads * 16 <= (1ull << 30)) grid = stream_grid(nquads, (uint64_t)kThreads * kUnroll);
        if (reverse)
            quantize_quads_kernel<true><<<grid, kThreads, 0, st>>>((const float4*)x, (uint32_t*)q, nquads, scale, zp, scale_dev, zp_dev);
        else
            quantize_quads_kernel<false><<<grid, kThreads, 0, st>>>((const float4*)x, (uint32_t*)q, nquads, scale, zp, scale_dev, zp_dev);
        if (int rc = launched("quantize_quads_kernel")) return rc;
    }
    if (nquads * 4 < n) {
        uint64_t rest = n - nquads * 4;
        unsigned int grid = stream_grid(rest, kThreads);
        quantize_scalar_kernel<<<grid, kThreads, 0, st>>>(x, q, nquads * 4, n, scale, zp, scale_dev, zp_dev);
        if (int rc = launched("quantize_scalar_kernel")) return rc;
    }
    return 0;
}

static int launch_minmax(const float* x, uint64_t n, rplb_qparams* params, cudaStream_t st) {
    if (!params) return fail(RPLB_E_BAD_ARG, "minmax: null params pointer");
    if (n && !x) return fail(RPLB_E_BAD_ARG, "minmax: null input");
    if ((uintptr_t)x & 3) return fail(RPLB_E_BAD_ARG, "minmax: fp32 input not 4-byte aligned");
    uint64_t head = (16 - ((uintptr_t)x & 15)) & 15;
    head /= 4;
    if (head > n) head = n;
    uint64_t nquads = (n - head) / 4;
    // One CTA per 65536 elements (16 unrolled steps each) rather than a resident grid:
    // measured 6172 vs 5974 GB/s at 2^26 elements, 7345 vs 7079 at 2^30.
    unsigned int grid = one_shot_grid(nquads, (uint64_t)kThreads * kUnroll * 16);
    Scratch sc;
    if (int rc = scratch_for(st, (size_t)grid * sizeof(float2), &sc)) return rc;
    minmax_kernel<<<grid, kThreads, 0, st>>>(x, n, head, nquads, (float2*)sc.data, sc.control, params);
    return launched("minmax_kernel");
}


// ---------------------------------------------------------------------------
// per-channel quantize  (src/rpl_quantization.c:134-157)
// ---------------------------------------------------------------------------
// One CTA per channel (a contiguous run of channel_size floats).  Rows of up to
// kThreads*4*kRowQuads floats are held in registers between the absmax
// reduction and the quantize step, so HBM sees each element once; longer rows
// are read a second time (from L2 when the row fits there).
constexpr int kRowQuads = 8;       // float4 per thread kept in registers -> rows up to 8192 floats

__device__ __forceinline__ void block_minmax(float& lo, float& hi, float* s_lo, float* s_hi) {
    lo = warp_min(lo);
    hi = warp_max(hi);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
    __syncthreads();
    lo = s_lo[0]; hi = s_hi[0];
    #pragma unroll
    for (int w = 1; w < kThreads / 32; w++) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
}

// Scale of one channel from its min/max, as src/rpl_quantization.c:136-147.
__device__ __forceinline__ float channel_scale(float lo, float hi) {
    float mn = fminf(lo, FLT_MAX), mx = fmaxf(hi, -FLT_MAX);
    return __fdiv_rn(fmaxf(fabsf(mn), fabsf(mx)), 127.0f);
}

template <int QUADS>
__global__ void __launch_bounds__(kThreads)
per_channel_regs_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                        int32_t* __restrict__ zps, uint64_t num_channels, uint32_t row_quads) {
    __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
    for (uint64_t c = blockIdx.x; c < num_channels; c += gridDim.x) {
        const float4* row = reinterpret_cast<const float4*>(x) + c * row_quads;
        uint32_t* out = reinterpret_cast<uint32_t*>(q) + c * row_quads;
        float4 v[QUADS];
        float lo = INFINITY, hi = -INFINITY;
        #pragma unroll
        for (int u = 0; u < QUADS; u++) {
            uint32_t i = threadIdx.x + u * kThreads;
            if (i < row_quads) v[u] = __ldcs(row + i);
        }
        #pragma unroll
        for (int u = 0; u < QUADS; u++) {
            uint32_t i = threadIdx.x + u * kThreads;
            if (i < row_quads) {
                lo = fminf(fminf(lo, v[u].x), fminf(v[u].y, fminf(v[u].z, v[u].w)));
                hi = fmaxf(fmaxf(hi, v[u].x), fmaxf(v[u].y, fmaxf(v[u].z, v[u].w)));
            }
        }
        block_minmax(lo, hi, s_lo, s_hi);
        const float scale = channel_scale(lo, hi);
        const QuantConsts qc = make_quant_consts(scale, 0);
        if (threadIdx.x == 0) { scales[c] = scale; if (zps) zps[c] = 0; }
        #pragma unroll
        for (int u = 0; u < QUADS; u++) {
            uint32_t i = threadIdx.x + u * kThreads;
            if (i < row_quads) __stcs(out + i, quantize_quad_packed(v[u], qc));
        }
        __syncthreads();      // s_lo/s_hi are reused by the next channel
    }
}

// Rows too long for the registers alone: the first kRowQuads quads per thread of a
// row are held in registers as above, the rest of the row is brought into shared
// memory by bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier) that run while the register part is being loaded.  Both parts are
// reduced and then quantized where they lie, so HBM sees each element once here
// too.  Splitting the row between registers and shared memory lets four CTAs
// share an SM for 64 KiB rows (three if the whole row were staged), and it is the
// overlap between CTAs in different phases that keeps the memory system busy
// (measured at 4096 rows of 16384 floats: 5748 GB/s against 4831 for two passes;
// a whole-row ring in one persistent CTA per SM reached 4240).
constexpr uint32_t kBulkPiece = 16384;               // bytes per bulk copy
constexpr size_t kStagedSmemBytes = 216 * 1024;      // shared memory the co-resident CTAs may use together
constexpr size_t kStagedRowMaxBytes = 232 * 1024;    // longer rows take the two-pass kernel
constexpr uint32_t kRegQuads = kThreads * kRowQuads; // quads of a row kept in registers

__device__ __forceinline__ uint32_t smem_addr_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(kThreads, 4)
per_channel_staged_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                          int32_t* __restrict__ zps, uint64_t num_channels, uint32_t row_quads, int* __restrict__ gave_up) {
    extern __shared__ __align__(128) uint8_t staged[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
    __shared__ int s_abort;
    const uint32_t bar_addr = smem_addr_u32(&bar);
    const uint32_t tail_quads = row_quads - kRegQuads;            // the part that goes through shared memory (> 0)
    const uint32_t tail_bytes = tail_quads * 16;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    __syncthreads();
    uint32_t phase = 0;
    for (uint64_t c = blockIdx.x; c < num_channels; c += gridDim.x) {
        const float4* row = reinterpret_cast<const float4*>(x) + c * (uint64_t)row_quads;
        if (threadIdx.x == 0) {
            // The previous row's tail was read with ordinary loads; the copies below write through the async proxy.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(tail_bytes) : "memory");
            const uint8_t* src = reinterpret_cast<const uint8_t*>(row + kRegQuads);
            for (uint32_t off = 0; off < tail_bytes; off += kBulkPiece) {
                const uint32_t n = min(kBulkPiece, tail_bytes - off);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_addr_u32(staged + off)), "l"(src + off), "r"(n), "r"(bar_addr) : "memory");
            }
        }
        float4 v[kRowQuads];
        #pragma unroll
        for (int u = 0; u < kRowQuads; u++) v[u] = __ldcs(row + threadIdx.x + u * kThreads);
        float lo = INFINITY, hi = -INFINITY;
        #pragma unroll
        for (int u = 0; u < kRowQuads; u++) {
            lo = fminf(fminf(lo, v[u].x), fminf(v[u].y, fminf(v[u].z, v[u].w)));
            hi = fmaxf(fmaxf(hi, v[u].x), fmaxf(v[u].y, fmaxf(v[u].z, v[u].w)));
        }
        // Wait for the tail (bounded: a copy that never completes ends the kernel with a flag, not a hang).
        {
            uint32_t done = 0, tries = 0;
            while (!done) {
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
                if (!done && ++tries > (1u << 22)) { s_abort = 1; break; }
            }
        }
        phase ^= 1;
        const float4* tail = reinterpret_cast<const float4*>(staged);
        for (uint32_t i = threadIdx.x; i < tail_quads; i += kThreads) {
            const float4 t = tail[i];
            lo = fminf(fminf(lo, t.x), fminf(t.y, fminf(t.z, t.w)));
            hi = fmaxf(fmaxf(hi, t.x), fmaxf(t.y, fmaxf(t.z, t.w)));
        }
        block_minmax(lo, hi, s_lo, s_hi);                 // contains the barrier that also publishes s_abort
        if (s_abort) {
            if (threadIdx.x == 0) atomicCAS(gave_up, 0, 6);       // status code 6: a bulk copy of a channel did not complete
            return;
        }
        const float scale = channel_scale(lo, hi);
        const QuantConsts qc = make_quant_consts(scale, 0);
        if (threadIdx.x == 0) { scales[c] = scale; if (zps) zps[c] = 0; }
        uint32_t* out = reinterpret_cast<uint32_t*>(q) + c * (uint64_t)row_quads;
        #pragma unroll
        for (int u = 0; u < kRowQuads; u++) __stcs(out + threadIdx.x + u * kThreads, quantize_quad_packed(v[u], qc));
        for (uint32_t i = threadIdx.x; i < tail_quads; i += kThreads) __stcs(out + kRegQuads + i, quantize_quad_packed(tail[i], qc));
        __syncthreads();      // every thread is done with the staged tail (and with s_lo / s_hi)
    }
}

// Any row length and alignment: two passes over the row, scalar accesses.
__global__ void __launch_bounds__(kThreads)
per_channel_stream_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                          int32_t* __restrict__ zps, uint64_t num_channels, uint64_t channel_size, int vec) {
    __shared__ float s_lo[kThreads / 32], s_hi[kThreads / 32];
    for (uint64_t c = blockIdx.x; c < num_channels; c += gridDim.x) {
        const float* row = x + c * channel_size;
        int8_t* out = q + c * channel_size;
        float lo = INFINITY, hi = -INFINITY;
        if (vec) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            const uint64_t nq = channel_size / 4;
            for (uint64_t i = threadIdx.x; i < nq; i += kThreads) {
                float4 v = __ldg(r4 + i);
                lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));
                hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
            }
        } else {
            for (uint64_t i = threadIdx.x; i < channel_size; i += kThreads) {
                float v = row[i];
                lo = fminf(lo, v);
                hi = fmaxf(hi, v);
            }
        }
        block_minmax(lo, hi, s_lo, s_hi);
        const float scale = channel_scale(lo, hi);
        const QuantConsts qc = make_quant_consts(scale, 0);
        if (threadIdx.x == 0) { scales[c] = scale; if (zps) zps[c] = 0; }
        if (vec) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            uint32_t* o4 = reinterpret_cast<uint32_t*>(out);
            const uint64_t nq = channel_size / 4;
            // Walk back from the end of the row: the most recently read part
            // is the most likely to be in cache still.
            for (uint64_t k = threadIdx.x; k < nq; k += kThreads) {
                uint64_t i = nq - 1 - k;
                __stcs(o4 + i, quantize_quad_packed(__ldcs(r4 + i), qc));
            }
        } else {
            for (uint64_t i = threadIdx.x; i < channel_size; i += kThreads)
                out[i] = (int8_t)quantize_one(row[i], scale, 0);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// dequantize  (src/ops_extended.c:67-70)
// ---------------------------------------------------------------------------
// (float)(q - zp) for |q - zp| < 2^22 without an int->float conversion:
// 0x4B400000 is the bit pattern of 1.5 * 2^23, whose low mantissa bits count
// in units of 1, so adding the integer to the pattern and subtracting
// 1.5 * 2^23 as a float gives the integer's value exactly.
__device__ __forceinline__ float int_to_float_small(int32_t i) {
    return __fsub_rn(__int_as_float(0x4B400000 + i), 12582912.0f);
}

template <bool SMALL_ZP>
__device__ __forceinline__ float4 dequant_quad(uint32_t w, float scale, int32_t zp) {
    const int32_t q0 = (int32_t)(int8_t)(w & 0xff), q1 = (int32_t)(int8_t)((w >> 8) & 0xff);
    const int32_t q2 = (int32_t)(int8_t)((w >> 16) & 0xff), q3 = (int32_t)(int8_t)(w >> 24);
    float4 r;
    if (SMALL_ZP) {
        r.x = __fmul_rn(int_to_float_small(q0 - zp), scale);
        r.y = __fmul_rn(int_to_float_small(q1 - zp), scale);
        r.z = __fmul_rn(int_to_float_small(q2 - zp), scale);
        r.w = __fmul_rn(int_to_float_small(q3 - zp), scale);
    } else {
        // int32 subtraction wraps, as the reference's compiled code does
        r.x = __fmul_rn(__int2float_rn((int32_t)((uint32_t)q0 - (uint32_t)zp)), scale);
        r.y = __fmul_rn(__int2float_rn((int32_t)((uint32_t)q1 - (uint32_t)zp)), scale);
        r.z = __fmul_rn(__int2float_rn((int32_t)((uint32_t)q2 - (uint32_t)zp)), scale);
        r.w = __fmul_rn(__int2float_rn((int32_t)((uint32_t)q3 - (uint32_t)zp)), scale);
    }
    return r;
}

// Eight elements per thread: one 8-byte load, one 256-bit store (a whole 32-byte
// sector per thread, 1 KiB contiguous per warp instruction).
__device__ __forceinline__ void store_f32x8(float* p, float4 a, float4 b) {
    asm volatile("st.global.v8.f32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                 :: "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x), "f"(b.y), "f"(b.z), "f"(b.w), "l"(p) : "memory");
}

template <int UNROLL, bool STREAM_LOADS>
__global__ void __launch_bounds__(kThreads)
dequantize_octs_kernel(const uint2* __restrict__ q, float* __restrict__ out, uint64_t nocts, float scale, int32_t zp) {
    const uint64_t step = (uint64_t)kThreads * UNROLL;
    const uint64_t nsteps = (nocts + step - 1) / step;
    for (uint64_t s = blockIdx.x; s < nsteps; s += gridDim.x) {
        const uint64_t base = s * step + threadIdx.x;
        uint2 w[UNROLL];
        #pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nocts) w[u] = STREAM_LOADS ? __ldcs(q + i) : __ldg(q + i);
        }
        #pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nocts) store_f32x8(out + i * 8, dequant_quad<true>(w[u].x, scale, zp), dequant_quad<true>(w[u].y, scale, zp));
        }
    }
}

template <bool SMALL_ZP>
__global__ void __launch_bounds__(kThreads)
dequantize_quads_kernel(const uint32_t* __restrict__ q, float4* __restrict__ out, uint64_t nquads,
                        float scale, int32_t zp) {
    const uint64_t step = (uint64_t)kThreads * kUnroll;
    const uint64_t nsteps = (nquads + step - 1) / step;
    for (uint64_t s = blockIdx.x; s < nsteps; s += gridDim.x) {
        const uint64_t base = s * step + threadIdx.x;
        uint32_t w[kUnroll];
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nquads) w[u] = __ldcs(q + i);
        }
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            // Plain (write-back) stores: measured 5 % faster here than st.global.cs,
            // which pushes every line to DRAM as soon as it is written.
            if (i < nquads) out[i] = dequant_quad<SMALL_ZP>(w[u], scale, zp);
        }
    }
}

__global__ void __launch_bounds__(kThreads)
dequantize_scalar_kernel(const int8_t* __restrict__ q, float* __restrict__ out, uint64_t begin, uint64_t n,
                         float scale, int32_t zp) {
    for (uint64_t i = begin + (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kThreads)
        out[i] = __fmul_rn((float)((int32_t)q[i] - zp), scale);
}

// Per-channel: quads never straddle a channel when channel_size % 4 == 0.
__global__ void __launch_bounds__(kThreads)
dequantize_pc_quads_kernel(const uint32_t* __restrict__ q, const float* __restrict__ scales,
                           float4* __restrict__ out, uint64_t nquads, uint64_t row_quads) {
    const uint64_t step = (uint64_t)kThreads * kUnroll;
    const uint64_t nsteps = (nquads + step - 1) / step;
    for (uint64_t s = blockIdx.x; s < nsteps; s += gridDim.x) {
        const uint64_t base = s * step + threadIdx.x;
        #pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            uint64_t i = base + (uint64_t)u * kThreads;
            if (i < nquads) out[i] = dequant_quad<true>(__ldcs(q + i), __ldg(scales + i / row_quads), 0);
        }
    }
}

__global__ void __launch_bounds__(kThreads)
dequantize_pc_scalar_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                            float* __restrict__ out, uint64_t n, uint64_t channel_size) {
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kThreads)
        out[i] = __fmul_rn((float)(int32_t)q[i], scales[i / channel_size]);
}

}  // namespace rplb

namespace rplb {
// ReLU between quantized layers (src/rpl_core.c:254-255): x < 0 -> 0, in place.
__global__ void __launch_bounds__(kThreads)
relu_kernel(float* __restrict__ x, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kThreads) {
        float v = x[i];
        if (v < 0.0f) x[i] = 0.0f;
    }
}
}  // namespace rplb

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using namespace rplb;

// Per host thread: 1 = rows between 32 and 232 KiB are split between registers and shared memory (one HBM pass), 0 = two passes.
static thread_local int t_per_channel_smem = 1;

extern "C" {

int rplb_minmax_f32(const float* x, uint64_t n, rplb_qparams* params, void* stream) {
    return launch_minmax(x, n, params, as_stream(stream));
}

int rplb_qparams_to_pair(const rplb_qparams* params, float* pair, void* stream) {
    if (!params || !pair) return fail(RPLB_E_BAD_ARG, "rplb_qparams_to_pair: null pointer");
    qparams_to_pair_kernel<<<1, 1, 0, as_stream(stream)>>>(params, pair);
    return launched("qparams_to_pair_kernel");
}

int rplb_qparams_from_pair(const float* pair, rplb_qparams* params, void* stream) {
    if (!params || !pair) return fail(RPLB_E_BAD_ARG, "rplb_qparams_from_pair: null pointer");
    qparams_from_pair_kernel<<<1, 1, 0, as_stream(stream)>>>(pair, params);
    return launched("qparams_from_pair_kernel");
}

int rplb_quantize_f32_i8(const float* x, int8_t* q, uint64_t n, float scale, int32_t zero_point, void* stream) {
    return launch_quantize(x, q, n, scale, zero_point, nullptr, nullptr, false, as_stream(stream));
}

int rplb_quantize_f32_i8_dev(const float* x, int8_t* q, uint64_t n, const float* scale_dev,
                             const int32_t* zp_dev, void* stream) {
    if (!scale_dev) return fail(RPLB_E_BAD_ARG, "rplb_quantize_f32_i8_dev: null scale pointer");
    return launch_quantize(x, q, n, 0.0f, 0, scale_dev, zp_dev, false, as_stream(stream));
}

int rplb_quantize_onepass(int which) {
    const int prev = t_onepass;
    if (which == 0 || which == 1) t_onepass = which;
    return prev;
}

int rplb_quantize_symmetric_f32_i8(const float* x, int8_t* q, uint64_t n, rplb_qparams* params, void* stream) {
    bool done = false;
    if (int rc = launch_quantize_onepass(x, q, n, params, 0, as_stream(stream), &done)) return rc;
    if (done) return 0;
    if (int rc = launch_minmax(x, n, params, as_stream(stream))) return rc;
    return launch_quantize(x, q, n, 0.0f, 0, &params->scale_sym, nullptr, true, as_stream(stream));
}

int rplb_quantize_asymmetric_f32_i8(const float* x, int8_t* q, uint64_t n, rplb_qparams* params, void* stream) {
    bool done = false;
    if (int rc = launch_quantize_onepass(x, q, n, params, 1, as_stream(stream), &done)) return rc;
    if (done) return 0;
    if (int rc = launch_minmax(x, n, params, as_stream(stream))) return rc;
    return launch_quantize(x, q, n, 0.0f, 0, &params->scale_asym, &params->zp_asym, true, as_stream(stream));
}

int rplb_quantize_per_channel_f32_i8(const float* x, int8_t* q, float* scales, int32_t* zero_points,
                                     uint64_t num_channels, uint64_t channel_size, void* stream) {
    if (num_channels == 0) return 0;
    if (!x || !q || !scales) return fail(RPLB_E_BAD_ARG, "per-channel quantize: null pointer");
    if ((uintptr_t)x & 3) return fail(RPLB_E_BAD_ARG, "per-channel quantize: fp32 input not 4-byte aligned");
    cudaStream_t st = as_stream(stream);
    const bool vec = (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 3) == 0) && (channel_size % 4 == 0) && channel_size;
    uint64_t cap = (uint64_t)sm_count() * kCtasPerSm * 4;
    if (cap == 0) cap = 4096;
    unsigned int grid = (unsigned int)(num_channels < cap ? num_channels : cap);
    const uint64_t row_quads = channel_size / 4;
    if (vec && row_quads <= (uint64_t)kThreads * kRowQuads) {
        const uint32_t rq = (uint32_t)row_quads;
        if (rq <= kThreads * 1)      per_channel_regs_kernel<1><<<grid, kThreads, 0, st>>>(x, q, scales, zero_points, num_channels, rq);
        else if (rq <= kThreads * 2) per_channel_regs_kernel<2><<<grid, kThreads, 0, st>>>(x, q, scales, zero_points, num_channels, rq);
        else if (rq <= kThreads * 4) per_channel_regs_kernel<4><<<grid, kThreads, 0, st>>>(x, q, scales, zero_points, num_channels, rq);
        else                         per_channel_regs_kernel<kRowQuads><<<grid, kThreads, 0, st>>>(x, q, scales, zero_points, num_channels, rq);
        return launched("per_channel_regs_kernel");
    }
    const size_t row_bytes = (size_t)channel_size * 4;
    if (vec && row_bytes <= kStagedRowMaxBytes && t_per_channel_smem) {
        // Part of the row in registers, the rest staged in shared memory; up to four CTAs per SM.
        static std::atomic<uint64_t> attr_done{0};
        int dev = 0;
        if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
        if (dev >= 64 || !((attr_done.load() >> dev) & 1ull)) {
            if (int rc = cuda_ok(cudaFuncSetAttribute(per_channel_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      (int)(kStagedRowMaxBytes - (size_t)kRegQuads * 16)),
                                 "cudaFuncSetAttribute(per_channel_staged_kernel)")) return rc;
            if (dev < 64) attr_done.fetch_or(1ull << dev);
        }
        const size_t tail_bytes = row_bytes - (size_t)kRegQuads * 16;
        uint64_t per = kStagedSmemBytes / (tail_bytes + 1024);
        if (per > 4) per = 4;
        if (per < 1) per = 1;
        uint64_t cap2 = (uint64_t)sm_count() * per;
        if (cap2 == 0) cap2 = 148 * per;
        // A wait that runs out is reported through the calling thread's kernel status word (rplb_kernel_status).
        int* status_dev = kernel_status_word_device();
        if (!status_dev) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
        const unsigned int g2 = (unsigned int)(num_channels < cap2 ? num_channels : cap2);
        per_channel_staged_kernel<<<g2, kThreads, tail_bytes, st>>>(x, q, scales, zero_points, num_channels, (uint32_t)row_quads,
                                                                    status_dev);
        return launched("per_channel_staged_kernel");
    }
    per_channel_stream_kernel<<<grid, kThreads, 0, st>>>(x, q, scales, zero_points, num_channels, channel_size, vec ? 1 : 0);
    return launched("per_channel_stream_kernel");
}

int rplb_per_channel_staging(int which) {
    const int prev = t_per_channel_smem;
    if (which == 0 || which == 1) t_per_channel_smem = which;
    return prev;
}

int rplb_dequantize_i8_f32(const int8_t* q, float* out, uint64_t n, float scale, int32_t zero_point, void* stream) {
    if (n == 0) return 0;
    if (!q || !out) return fail(RPLB_E_BAD_ARG, "dequantize: null pointer");
    if ((uintptr_t)out & 3) return fail(RPLB_E_BAD_ARG, "dequantize: fp32 output not 4-byte aligned");
    cudaStream_t st = as_stream(stream);
    const bool vec = (((uintptr_t)out & 15) == 0) && (((uintptr_t)q & 3) == 0);
    uint64_t nquads = vec ? n / 4 : 0;
    if ((((uintptr_t)out & 31) == 0) && (((uintptr_t)q & 7) == 0) && n >= 8 &&
        zero_point > -(1 << 21) && zero_point < (1 << 21)) {
        const uint64_t nocts = n / 8;
        // One CTA per step: for this write-heavy kernel a resident, striding grid was 13 % slower
        // (5473 vs 6246 GB/s at 2^26 elements, 5759 vs 6771 at 2^30).
        unsigned int grid = one_shot_grid(nocts, (uint64_t)kThreads * kUnroll);
        dequantize_octs_kernel<kUnroll, true><<<grid, kThreads, 0, st>>>((const uint2*)q, out, nocts, scale, zero_point);
        if (int rc = launched("dequantize_octs_kernel")) return rc;
        nquads = nocts * 2;                 // the scalar kernel below takes what is left
    } else if (nquads) {
        unsigned int grid = one_shot_grid(nquads, (uint64_t)kThreads * kUnroll);
        if (zero_point > -(1 << 21) && zero_point < (1 << 21))
            dequantize_quads_kernel<true><<<grid, kThreads, 0, st>>>((const uint32_t*)q, (float4*)out, nquads, scale, zero_point);
        else
            dequantize_quads_kernel<false><<<grid, kThreads, 0, st>>>((const uint32_t*)q, (float4*)out, nquads, scale, zero_point);
        if (int rc = launched("dequantize_quads_kernel")) return rc;
    }
    if (nquads * 4 < n) {
        unsigned int grid = stream_grid(n - nquads * 4, kThreads);
        dequantize_scalar_kernel<<<grid, kThreads, 0, st>>>(q, out, nquads * 4, n, scale, zero_point);
        if (int rc = launched("dequantize_scalar_kernel")) return rc;
    }
    return 0;
}

int rplb_dequantize_per_channel_i8_f32(const int8_t* q, const float* scales, float* out,
                                       uint64_t num_channels, uint64_t channel_size, void* stream) {
    const uint64_t n = num_channels * channel_size;
    if (n == 0) return 0;
    if (!q || !out || !scales) return fail(RPLB_E_BAD_ARG, "per-channel dequantize: null pointer");
    if ((uintptr_t)out & 3) return fail(RPLB_E_BAD_ARG, "per-channel dequantize: fp32 output not 4-byte aligned");
    cudaStream_t st = as_stream(stream);
    const bool vec = (((uintptr_t)out & 15) == 0) && (((uintptr_t)q & 3) == 0) && (channel_size % 4 == 0);
    if (vec) {
        unsigned int grid = one_shot_grid(n / 4, (uint64_t)kThreads * kUnroll);
        dequantize_pc_quads_kernel<<<grid, kThreads, 0, st>>>((const uint32_t*)q, scales, (float4*)out, n / 4, channel_size / 4);
        return launched("dequantize_pc_quads_kernel");
    }
    unsigned int grid = stream_grid(n, kThreads);
    dequantize_pc_scalar_kernel<<<grid, kThreads, 0, st>>>(q, scales, out, n, channel_size);
    return launched("dequantize_pc_scalar_kernel");
}

int rplb_relu_f32_inplace(float* x, uint64_t n, void* stream) {
    if (n == 0) return 0;
    if (!x) return fail(RPLB_E_BAD_ARG, "relu: null pointer");
    relu_kernel<<<stream_grid(n, kThreads * 4), kThreads, 0, as_stream(stream)>>>(x, n);
    return launched("relu_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free min/max
// ---------------------------------------------------------------------------
// Same kernel as rplb_minmax_f32, with the per-CTA partial results and the
// ticket counter in a fixed array that is part of the loaded library image
// instead of a cudaMalloc'ed block.
namespace rplb {

constexpr unsigned int kStaticMaxCtas = RPLB_STATIC_MINMAX_MAX_CTAS;

struct StaticMinmaxScratch {
    unsigned int ticket;                 // must be zero when the kernel starts
    unsigned int pad[63];
    float2 partials[kStaticMaxCtas];     // one (min, max) pair per CTA
};

// Lives in every device that loads the library, from load to exit (8.25 KiB).
static __device__ __align__(256) StaticMinmaxScratch g_static_minmax;

// Device address of the array above, per device ordinal.  In host code the
// symbol's name is only a handle: the address a kernel can use has to be asked
// for, with the device in question current.  The answer is kept for the life of
// the process: a cudaDeviceReset() unloads the library's device image, after
// which the library as a whole (not only this cache) must not be used.
constexpr int kMaxDevices = 64;
static StaticMinmaxScratch* g_static_minmax_addr[kMaxDevices];
static std::mutex g_static_minmax_mu;

static int static_minmax_address(StaticMinmaxScratch** out) {
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= kMaxDevices) return fail(RPLB_E_BAD_ARG, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_minmax_mu);
    if (!g_static_minmax_addr[dev]) {
        void* p = nullptr;
        if (int rc = cuda_ok(cudaGetSymbolAddress(&p, g_static_minmax), "cudaGetSymbolAddress(g_static_minmax)")) return rc;
        g_static_minmax_addr[dev] = static_cast<StaticMinmaxScratch*>(p);
    }
    *out = g_static_minmax_addr[dev];
    return 0;
}

}  // namespace rplb

extern "C" int rplb_minmax_f32_static(const float* x, uint64_t n, rplb_qparams* params, void* stream) {
    using namespace rplb;
    if (n > RPLB_STATIC_MINMAX_MAX_ELEMENTS)
        return fail(RPLB_E_TOO_LARGE, "rplb_minmax_f32_static: %llu elements exceed the limit of %llu; use rplb_minmax_f32",
                    (unsigned long long)n, (unsigned long long)RPLB_STATIC_MINMAX_MAX_ELEMENTS);
    if (!params) return fail(RPLB_E_BAD_ARG, "rplb_minmax_f32_static: null params pointer");
    if (n && !x) return fail(RPLB_E_BAD_ARG, "rplb_minmax_f32_static: null input");
    if ((uintptr_t)x & 3) return fail(RPLB_E_BAD_ARG, "rplb_minmax_f32_static: fp32 input not 4-byte aligned");
    cudaStream_t st = as_stream(stream);
    StaticMinmaxScratch* sc = nullptr;
    if (int rc = static_minmax_address(&sc)) return rc;
    uint64_t head = ((16 - ((uintptr_t)x & 15)) & 15) / 4;
    if (head > n) head = n;
    const uint64_t nquads = (n - head) / 4;
    unsigned int grid = stream_grid(nquads, (uint64_t)kThreads * kUnroll);
    if (grid > kStaticMaxCtas) grid = kStaticMaxCtas;       // the kernel strides over the rest
    // Every call shares the array and it keeps what the last call left there:
    // the ticket has to start at zero, the partials are overwritten before use.
    if (int rc = cuda_ok(cudaMemsetAsync(&sc->ticket, 0, sizeof(unsigned int), st), "cudaMemsetAsync(ticket)")) return rc;
    minmax_kernel<<<grid, kThreads, 0, st>>>(x, n, head, nquads, sc->partials, &sc->ticket, params);
    return launched("minmax_kernel(static scratch)");
}
