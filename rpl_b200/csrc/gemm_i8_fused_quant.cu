// Quantize fused into the A side of the INT8 contraction, for layers with few
// output features and a short reduction (the first layer of the quantized MLP:
// 784 -> 128 over a large batch).
//
//   out[m,n] = relu?( ((float)acc * sA) * sW[n] + bias[n] ),
//   acc = sum_k q(x[m,k]) * w[n,k],   q(v) = clamp((int32)roundf(v / sA), -128, 127)
//
// i.e. tensor_quantize_int8 (src/rpl_core.c:521-527) with a scale that is already
// known, linear_int8 (src/rpl_quantization.c:340-350) and the fused fp32 epilogue
// in one kernel.  Such a layer is bound by HBM, not by the tensor cores: done in
// two kernels, the int8 copy of x is written once and read once (a quarter of the
// fp32 bytes each way) for nothing.  Here the fp32 activation travels from HBM into
// a ring of shared-memory slots by TMA (so the bytes in flight do not depend on
// registers), converter warps quantize each slot into the 128-byte-swizzled
// K-major int8 tile that tcgen05.mma reads, and the int8 activation never exists
// in memory.
//
// One persistent CTA per SM, 704 threads:
//   warp 0        loads the whole weight matrix once (TMA, N <= 128 rows x K <= 896
//                 bytes, resident in shared memory for the life of the CTA), then
//                 issues the MMAs: tcgen05.mma.kind::i8, 128 x 128 x 32, into one of
//                 four 128-column TMEM accumulators.
//   warp 1        TMA producer of the activation: boxes of 32 rows x 128 floats
//                 (16 KiB, 512 contiguous bytes per row, no swizzle) into a ring of slots.
//   warps 2-5     epilogue, 16 columns at a time to stay within the register budget of
//                 so large a CTA (tcgen05.ld, dequantize + bias + ReLU, optional
//                 max |out|, row stores), overlapped with the following tiles.
//   warps 6-21    converters: a thread takes 16-byte pieces (four floats) of a slot,
//                 quantizes them to one packed word and stores it at its swizzled
//                 place of the int8 stage; after the last slice of a K block each warp
//                 fences towards the async proxy and arrives on the stage's barrier.
//                 The conversion costs some 70 instructions per piece, so it takes
//                 sixteen warps to keep up with the 44 GB/s of HBM an SM is due
//                 (eight reached 29 % of DRAM bandwidth at 37 % issue utilisation).
// Columns of K beyond the matrix are zero in the weight tile (TMA fill), so whatever
// the activation's padding quantizes to contributes nothing.  Every wait is bounded
// as in the other tensor-core kernels.
#include "gemm_tc_common.cuh"
#include <atomic>
#include <cstring>

namespace rplb {

constexpr int FQ_N = 128;                 // accumulator columns; weight rows beyond N are zero-filled by TMA
constexpr int FQ_MAX_KB = 7;              // 128-byte K blocks: K <= 896
constexpr int FQ_STAGES = 3;              // int8 A stages of 16 KiB when the activation arrives as fp32 ...
constexpr int FQ_SLOTS = 4;               // ... through this many fp32 slots of 16 KiB
constexpr int FQ_STAGES_I8 = FQ_STAGES + FQ_SLOTS - 1;   // int8 activation: the same shared memory is stages, but for the
                                                         // last 16 KiB, which stage the epilogue's TMA stores
constexpr int FQ_ACC = 4;                 // 4 x 128 columns: all of TMEM
constexpr int FQ_CONVERTER_WARPS = 16;
constexpr int FQ_EPILOGUE_WARP0 = 2;
constexpr int FQ_CONVERTER_WARP0 = 6;
constexpr int FQ_THREADS = (2 + 4 + FQ_CONVERTER_WARPS) * 32;
constexpr uint32_t FQ_TILE_BYTES = 128 * TILE_K;          // 16 KiB: an A stage, one K block of W, or one fp32 slot

// 32 lanes x 16 consecutive 32-bit columns of the accumulator.
__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

struct __align__(16) FqShared {
    uint64_t w_full;                  // the weight matrix is in shared memory
    uint64_t slot_full[FQ_SLOTS];     // TMA -> converters
    uint64_t slot_empty[FQ_SLOTS];    // converters -> TMA (one arrival per converter warp)
    uint64_t full[FQ_STAGES_I8];      // converters (one arrival per warp) or TMA -> MMA: stage written
    uint64_t empty[FQ_STAGES_I8];     // MMA -> converters or TMA: stage consumed
    uint64_t acc_full[FQ_ACC];        // MMA -> epilogue
    uint64_t acc_empty[FQ_ACC];       // epilogue -> MMA (one arrival per epilogue warp)
    uint32_t tmem_base;
    volatile int abort_flag;
    float w_scales[FQ_N];
    float bias[FQ_N];
};

constexpr uint32_t kIdescI8N128 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FQ_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);

static size_t fq_smem_bytes(uint32_t num_kb) {
    return 1024 + (size_t)num_kb * FQ_TILE_BYTES + (size_t)(FQ_STAGES + FQ_SLOTS) * FQ_TILE_BYTES + sizeof(FqShared);
}

// 32-byte slices of K that block kb holds (4, or fewer in the last block).
__device__ __forceinline__ uint32_t slices_of_block(uint32_t K, uint32_t kb) {
    const uint32_t k_left = K - kb * TILE_K;
    return k_left >= (uint32_t)TILE_K ? TILE_K / MMA_K : (k_left + MMA_K - 1) / MMA_K;
}

// QUANT = true: x is fp32 and is quantized on the way in (map_x: plain boxes of 32 rows x 128 floats).
// QUANT = false: x is int8 already (map_x: swizzled boxes of 128 rows x 128 bytes, loaded straight into the
// stages); the kernel is then the contraction for few output features -- whole weight matrix resident,
// 128-column accumulators in four TMEM buffers, seven activation stages -- and is launched without the
// converter warps.
template <bool QUANT>
__global__ void __launch_bounds__(QUANT ? FQ_THREADS : FQ_CONVERTER_WARP0 * 32, 1)
gemm_i8_fused_quant_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const __grid_constant__ CUtensorMap map_out, const GemmProblem p, uint32_t tiles_m, uint32_t num_kb,
                           int tma_out, int* status) {
    constexpr int kNumStages = QUANT ? FQ_STAGES : FQ_STAGES_I8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;                                             // [num_kb][128 rows x 128 bytes]
    uint8_t* a_stages = w_tiles + (size_t)num_kb * FQ_TILE_BYTES;        // [FQ_STAGES][128 rows x 128 bytes]
    uint8_t* slots = a_stages + (size_t)FQ_STAGES * FQ_TILE_BYTES;       // [FQ_SLOTS][128 rows x 32 floats]
    FqShared* sh = reinterpret_cast<FqShared*>(slots + (size_t)FQ_SLOTS * FQ_TILE_BYTES);
    uint8_t* epi_tiles = slots + (size_t)(FQ_SLOTS - 1) * FQ_TILE_BYTES;                  // int8 mode only: four 4 KiB staging tiles
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t K = (uint32_t)p.K;

    if (threadIdx.x == 0) {
        mbar_init(&sh->w_full, 1);
        for (int s = 0; s < FQ_SLOTS; s++) { mbar_init(&sh->slot_full[s], 1); mbar_init(&sh->slot_empty[s], FQ_CONVERTER_WARPS); }
        for (int s = 0; s < kNumStages; s++) { mbar_init(&sh->full[s], QUANT ? FQ_CONVERTER_WARPS : 1); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < FQ_ACC; a++) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 4); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(FQ_ACC * FQ_N) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Per-column epilogue inputs: the same for every tile.
    for (int n = threadIdx.x; n < FQ_N; n += blockDim.x) {
        sh->w_scales[n] = (uint64_t)n < p.N ? __ldg(p.w_scales + n) : 0.0f;
        sh->bias[n] = (p.bias_f32 && (uint64_t)n < p.N) ? __ldg(p.bias_f32 + n) : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------- weights once, then the MMAs
        if (lane == 0) {
            mbar_expect_tx(&sh->w_full, num_kb * FQ_TILE_BYTES);
            for (uint32_t kb = 0; kb < num_kb; kb++)
                tma_load_2d(w_tiles + (size_t)kb * FQ_TILE_BYTES, &map_w, &sh->w_full, (int32_t)(kb * TILE_K), 0);
            bool ok = mbar_wait_bounded(&sh->w_full, 0, &sh->abort_flag, status, TC_WAIT_FULL);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            for (uint32_t tile = blockIdx.x; ok && tile < tiles_m; tile += gridDim.x) {
                if (!mbar_wait_bounded(&sh->acc_empty[acc], acc_phase ^ 1, &sh->abort_flag, status, TC_WAIT_ACC_EMPTY)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * FQ_N;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->full[stage], phase, &sh->abort_flag, status, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(a_stages + (size_t)stage * FQ_TILE_BYTES));
                    const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(w_tiles + (size_t)kb * FQ_TILE_BYTES));
                    const uint32_t slices = slices_of_block(K, kb);          // only the slices that carry data
                    for (uint32_t k = 0; k < slices; k++)
                        tc_mma_i8(d_tmem, a_desc + (uint64_t)(k * (MMA_K >> 4)), b_desc + (uint64_t)(k * (MMA_K >> 4)),
                                  kIdescI8N128, (kb | k) != 0 ? 1u : 0u);
                    tc_commit(&sh->empty[stage]);
                    if (++stage == kNumStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(&sh->acc_full[acc]);
                if (++acc == FQ_ACC) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- TMA producer of the activation
        if (lane == 0 && QUANT) {
            uint32_t slot = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < tiles_m; tile += gridDim.x) {
                for (uint32_t kb = 0; ok && kb < num_kb; kb++) {
                    for (uint32_t rq = 0; rq < 4; rq++) {                   // 32 rows x 128 floats: 512 contiguous bytes per row
                        if (!mbar_wait_bounded(&sh->slot_empty[slot], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY)) { ok = false; break; }
                        mbar_expect_tx(&sh->slot_full[slot], FQ_TILE_BYTES);
                        tma_load_2d(slots + (size_t)slot * FQ_TILE_BYTES, &map_x, &sh->slot_full[slot],
                                    (int32_t)(kb * TILE_K), (int32_t)(tile * TILE_M + rq * 32));
                        if (++slot == FQ_SLOTS) { slot = 0; phase ^= 1; }
                    }
                }
            }
        } else if (lane == 0) {
            // int8 activation: 128 rows x 128 bytes straight into a stage (the fp32 slots' memory serves as stages too)
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < tiles_m; tile += gridDim.x) {
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->empty[stage], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(&sh->full[stage], FQ_TILE_BYTES);
                    tma_load_2d(a_stages + (size_t)stage * FQ_TILE_BYTES, &map_x, &sh->full[stage], (int32_t)(kb * TILE_K), (int32_t)(tile * TILE_M));
                    if (++stage == kNumStages) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp < FQ_CONVERTER_WARP0) {
        // ------------------------------------------------------------- epilogue
        const uint32_t quarter = (uint32_t)warp & 3u;        // TMEM lanes this warp may read
        const float a_scale = __ldg(p.a_scale);
        const bool has_bias = p.bias_f32 != nullptr, relu = p.relu != 0;
        const bool tma = !QUANT && tma_out != 0;
        uint8_t* my_tile = epi_tiles + (warp - FQ_EPILOGUE_WARP0) * EPI_TILE_BYTES;
        const QuantConsts oq = make_quant_consts(1.0f, 0);
        float absmax = 0.0f;
        uint32_t acc = 0, acc_phase = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles_m; tile += gridDim.x) {
            const uint64_t m_base = (uint64_t)tile * TILE_M + quarter * 32;
            bool ok = mbar_wait_bounded(&sh->acc_full[acc], acc_phase, &sh->abort_flag, status, TC_WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (!QUANT) {
                // Few threads, many registers: 32 columns at a time, results leave through TMA tensor stores.
                #pragma unroll 1
                for (int chunk = 0; chunk < FQ_N / 32; chunk++) {
                    const uint64_t n_first = (uint64_t)chunk * 32;
                    if (n_first >= p.N) break;
                    uint32_t r[32];
                    tc_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * FQ_N + (uint32_t)chunk * 32u, r);
                    tc_wait_ld();
                    epilogue_chunk<EPI_DEQUANT_F32, false>(p, &map_out, tma, my_tile, r, m_base, lane, n_first, a_scale,
                                                           sh->w_scales + chunk * 32, sh->bias + chunk * 32, oq, 0, absmax);
                }
            } else {
            const uint64_t m = m_base + (uint64_t)lane;
            #pragma unroll 1
            for (int chunk = 0; chunk < FQ_N / 16; chunk++) {
                const uint64_t n_first = (uint64_t)chunk * 16;
                if (n_first >= p.N) break;
                uint32_t r[16];
                tc_ld_32x16(tmem_base + ((quarter * 32u) << 16) + acc * FQ_N + (uint32_t)chunk * 16u, r);
                tc_wait_ld();
                const uint64_t n_left = p.N - n_first;
                float v[16];
                #pragma unroll
                for (int c = 0; c < 16; c++)
                    v[c] = dequant_f32((int32_t)r[c], a_scale, sh->w_scales[chunk * 16 + c], has_bias, sh->bias[chunk * 16 + c], relu);
                if (m < p.M) {
                    if (p.absmax_out) {
                        #pragma unroll
                        for (int c = 0; c < 16; c++)
                            if ((uint64_t)c < n_left) absmax_fold(absmax, v[c]);
                    }
                    float* row = static_cast<float*>(p.out) + m * p.ldo + n_first;
                    if (n_left >= 16 && (((uintptr_t)row & 15) == 0)) {
                        #pragma unroll
                        for (int c = 0; c < 16; c += 4) *reinterpret_cast<float4*>(row + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    } else {
                        #pragma unroll
                        for (int c = 0; c < 16; c++)
                            if ((uint64_t)c < n_left) row[c] = v[c];
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
            if (++acc == FQ_ACC) { acc = 0; acc_phase ^= 1; }
        }
        if (tma && lane == 0) bulk_wait_all();
        if (p.absmax_out) absmax_publish(p.absmax_out, absmax);
        if (p.next_scale && lane == 0) {
            // The last epilogue warp of the grid turns the maximum into the next layer's scale.
            __threadfence();
            if (atomicAdd(p.ticket, 1u) == gridDim.x * (uint32_t)(FQ_CONVERTER_WARP0 - FQ_EPILOGUE_WARP0) - 1u) {
                __threadfence();
                const float top = __uint_as_float(atomicOr(reinterpret_cast<unsigned int*>(p.absmax_out), 0u));
                *p.next_scale = __fdiv_rn(top, 127.0f);
                *p.ticket = 0;                  // leave the control word as it was found
            }
        }
    } else if (QUANT) {
        // ------------------------------------------------------------- converters: fp32 slot -> int8 rows of the stage
        const int cw = warp - FQ_CONVERTER_WARP0;
        const QuantConsts qc = make_quant_consts(__ldg(p.a_scale), 0);
        // A slot holds 32 rows of 128 floats (512 bytes, no swizzle): 1024 pieces of 16 bytes, two per thread.
        // A warp takes a whole row at a time: 512 contiguous bytes in, 128 contiguous bytes out.
        uint32_t slot = 0, slot_phase = 0, stage = 0, phase = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < tiles_m; tile += gridDim.x) {
            for (uint32_t kb = 0; ok && kb < num_kb; kb++) {
                bool got = true;
                if (lane == 0) got = mbar_wait_bounded(&sh->empty[stage], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY);
                if (!__shfl_sync(0xffffffffu, got ? 1 : 0, 0)) { ok = false; break; }
                uint8_t* dst = a_stages + (size_t)stage * FQ_TILE_BYTES;
                for (uint32_t rq = 0; rq < 4; rq++) {
                    if (lane == 0) got = mbar_wait_bounded(&sh->slot_full[slot], slot_phase, &sh->abort_flag, status, TC_WAIT_FULL);
                    if (!__shfl_sync(0xffffffffu, got ? 1 : 0, 0)) { ok = false; break; }
                    const uint8_t* src = slots + (size_t)slot * FQ_TILE_BYTES;
                    #pragma unroll
                    for (int it = 0; it < 32 / FQ_CONVERTER_WARPS; it++) {
                        const int row = cw * (32 / FQ_CONVERTER_WARPS) + it;                 // row of the slot
                        const float4 v = *reinterpret_cast<const float4*>(src + row * 512 + lane * 16);
                        const uint32_t word = quantize_quad_packed(v, qc);
                        const uint32_t R = rq * 32 + (uint32_t)row;                          // row of the stage
                        // bytes [4 lane, +4) of the row's 128: 16-byte piece lane / 4, word lane % 4
                        *reinterpret_cast<uint32_t*>(dst + R * 128 + ((((uint32_t)lane >> 2) ^ (R & 7)) << 4) + (lane & 3) * 4) = word;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->slot_empty[slot]);
                    if (++slot == FQ_SLOTS) { slot = 0; slot_phase ^= 1; }
                }
                if (!ok) break;
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->full[stage]);
                if (++stage == kNumStages) { stage = 0; phase ^= 1; }
            }
        }
    }

    // ----------------------------------------------------------------- teardown
    if (sh->abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FQ_ACC * FQ_N) : "memory");
    }
}

static bool narrow_shape_ok(const GemmProblem& p) {
    if (p.mode != EPI_DEQUANT_F32 || p.b_is_kn || p.n_peers || p.a_ready) return false;
    if (p.M == 0 || p.N == 0 || p.K == 0 || p.N > (uint64_t)FQ_N || p.K > (uint64_t)FQ_MAX_KB * TILE_K) return false;
    if (p.K % 16 != 0) return false;                                  // TMA row strides; whole quads of x
    return (((uintptr_t)p.B & 15) == 0) && p.M <= 0x7fffffffull * 64;
}

bool gemm_fused_quant_supports(const float* x, const GemmProblem& p) { return narrow_shape_ok(p) && (((uintptr_t)x & 15) == 0); }
bool gemm_narrow_supports(const GemmProblem& p) { return narrow_shape_ok(p) && (((uintptr_t)p.A & 15) == 0); }

template <bool QUANT>
static int launch_narrow(const void* x, const GemmProblem& p, cudaStream_t st) {
    if (int prev = gemm_tcgen05_status(true))
        return fail(RPLB_E_KERNEL, "an earlier tcgen05 GEMM of this thread gave up waiting (code %d)", prev);
    int* status_dev = kernel_status_word_device();
    if (!status_dev) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
    const uint32_t num_kb = (uint32_t)((p.K + TILE_K - 1) / TILE_K);
    const uint32_t tiles_m = (uint32_t)((p.M + TILE_M - 1) / TILE_M);
    CUtensorMap mw, mx, mo;
    int tma_out = 0;
    memset(&mo, 0, sizeof(mo));
    if (!QUANT && thread_gemm_epilogue(-1) == 0 && (((uintptr_t)p.out & 15) == 0) && p.ldo % 4 == 0) {
        if (int rc = make_map_2d(&mo, p.out, 4, p.N, p.M, p.ldo * 4, 32, 32, "output")) return rc;
        tma_out = 1;
    }
    if (int rc = make_map_2d(&mw, p.B, 1, p.K, p.N, p.K, (uint32_t)TILE_K, 128, "weights [N,K]")) return rc;
    if (QUANT) {
        if (int rc = make_map_2d(&mx, x, 5, p.K, p.M, p.K * 4, 128, 32, "fp32 activation [M,K]")) return rc;
    } else {
        if (int rc = make_map_2d(&mx, x, 1, p.K, p.M, p.K, (uint32_t)TILE_K, 128, "int8 activation [M,K]")) return rc;
    }
    const size_t smem = fq_smem_bytes(FQ_MAX_KB);
    static std::atomic<uint64_t> attr_done{0};
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev >= 64 || !((attr_done.load() >> dev) & 1ull)) {
        if (int rc = cuda_ok(cudaFuncSetAttribute(gemm_i8_fused_quant_kernel<QUANT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                             "cudaFuncSetAttribute(gemm_i8_fused_quant_kernel)")) return rc;
        if (dev < 64) attr_done.fetch_or(1ull << dev);
    }
    unsigned int sms = (unsigned int)sm_count();
    if (sms == 0) sms = 148;
    const unsigned int grid = tiles_m < sms ? tiles_m : sms;
    GemmProblem q = p;
    q.ticket = nullptr;
    if (q.next_scale && q.absmax_out) {
        // The counter of finished warps lives in the stream's scratch block (control word 8, zero at rest).
        Scratch sc;
        if (scratch_for(st, 0, &sc) == 0) q.ticket = sc.control + 8;
    }
    if (!q.ticket) q.next_scale = nullptr;
    gemm_i8_fused_quant_kernel<QUANT><<<grid, QUANT ? FQ_THREADS : FQ_CONVERTER_WARP0 * 32, fq_smem_bytes(num_kb), st>>>(
        mw, mx, mo, q, tiles_m, num_kb, tma_out, status_dev);
    if (q.next_scale && p.next_scale_done) *p.next_scale_done = 1;
    return launched(QUANT ? "gemm_i8_fused_quant_kernel<quantize>" : "gemm_i8_fused_quant_kernel<int8>");
}

int gemm_fused_quant(const float* x, const GemmProblem& p, cudaStream_t st) {
    if (!gemm_fused_quant_supports(x, p))
        return fail(RPLB_E_UNSUPPORTED, "fused quantize + GEMM needs N <= %d, K <= %d, K %% 16 == 0, 16-byte aligned x and w", FQ_N,
                    FQ_MAX_KB * TILE_K);
    return launch_narrow<true>(x, p, st);
}

int gemm_narrow(const GemmProblem& p, cudaStream_t st) {
    if (!gemm_narrow_supports(p))
        return fail(RPLB_E_UNSUPPORTED, "narrow GEMM needs the fp32 epilogue, N <= %d, K <= %d, K %% 16 == 0, 16-byte aligned x and w", FQ_N,
                    FQ_MAX_KB * TILE_K);
    return launch_narrow<false>(p.A, p, st);
}

}  // namespace rplb
