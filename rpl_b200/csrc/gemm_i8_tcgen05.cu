// INT8 x INT8 -> INT32 contraction on the 5th-generation tensor cores.
//
// C[m,n] = sum_k A[m,k] * W[n,k], A [M,K] and W [N,K] both K-contiguous
// (the layout of linear_int8, src/rpl_quantization.c:340-343), followed by one
// of the epilogues of the path: raw int32 (+ int8 bias), gemm_int8's
// requantization (with zero-point correction from row / column sums), the fused
// fp32 dequantize + bias + ReLU (optionally reporting max |out|), or that value
// quantized straight to int8.
//
// Three kernels share the helpers in this file and differ in how a tile is
// spread over SMs: gemm_i8_tc_kernel (one CTA, 128 x 256 tile, described below;
// the default for long GEMMs), gemm_i8_tc_pair_kernel (two CTAs of a cluster on
// a 256 x 256 tile with cta_group::2; the default for short GEMMs) and
// gemm_i8_tc_wide_kernel (one CTA, 256 x 256 tile in two accumulators).
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads of a 128 x 128-byte
//               A tile and a 256 x 128-byte W tile per stage, 128-byte swizzle,
//               no multicast; kStages-deep ring of shared-memory stages.
//   warp 1      MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::i8
//               (128 x 256 x 32 per instruction, four per stage) into one of two
//               256-column TMEM accumulators, and tcgen05.commit to hand stages
//               back to the producer and finished accumulators to the epilogue.
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, apply the
//               epilogue in registers, then hand the 32 x 32 chunk of four-byte
//               results to the TMA unit through a swizzled shared-memory tile
//               (cp.async.bulk.tensor store: whole 128-byte row segments leave the
//               SM, ragged edges are clipped by the tensor map); outputs whose
//               base or row stride is not a multiple of 16 bytes, and int8
//               outputs, are stored from registers instead.  While the epilogue
//               drains one accumulator the MMA warp fills the other.
//
// Rows of A may still be on their way from other GPUs when the kernel starts
// (GemmProblem::a_ready): the producer then begins with the 128-row blocks that
// are in place and, before the first load of any other block, waits (bounded)
// until that block's arrival word carries the call's epoch.
//
// Every wait on an mbarrier is bounded: when the limit passes the waiter writes
// a code to a status word in global memory and raises a CTA-wide abort flag,
// all roles leave their loops, TMEM is released and the kernel returns; the
// host turns the status word into RPLB_E_KERNEL.
#include "gemm_tc_common.cuh"
#include <atomic>
#include <cstring>
#include <mutex>

namespace rplb {

constexpr int kStages = 4;
constexpr int kAccBuffers = 2;
constexpr int kTmemCols = 512;       // 2 x 256 int32 columns: all of TMEM
constexpr int TC_THREADS = 192;
constexpr int kEpilogueWarp0 = 2;
constexpr int kEpilogueThreads = 128;
constexpr uint32_t A_STAGE_BYTES = TILE_M * TILE_K;      // 16 KiB
constexpr uint32_t B_STAGE_BYTES = TILE_N * TILE_K;      // 32 KiB
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int PAIR_GROUP_M = 16;     // 256-row m-tiles per group (CTA-pair kernel): the same 4096 rows of A

// Dynamic shared memory, after alignment to 1024 bytes:
//   [kStages][A tile | W tile]   then the block below.
struct __align__(16) TcShared {
    uint64_t full[kStages];          // producer -> MMA: stage loaded
    uint64_t empty[kStages];         // MMA -> producer: stage consumed
    uint64_t acc_full[kAccBuffers];  // MMA -> epilogue: accumulator complete
    uint64_t acc_empty[kAccBuffers]; // epilogue -> MMA: accumulator drained
    uint32_t tmem_base;
    volatile int abort_flag;
    float w_scales[4 * TILE_N];      // per-tile copies for the fp32 epilogue, one per epilogue warp
    float bias[4 * TILE_N];
};
constexpr size_t TC_SMEM_BYTES = 1024 + (size_t)kStages * STAGE_BYTES + EPI_STAGE_BYTES + sizeof(TcShared);

// --------------------------------------------------------------------------- the kernel
template <int MODE, bool PEERS = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_out, const GemmProblem p, uint32_t tiles_m, uint32_t tiles_n,
                  uint32_t num_kb, int tma_out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_tiles = smem + (size_t)kStages * STAGE_BYTES;
    TcShared* sh = reinterpret_cast<TcShared*>(epi_tiles + EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t total_tiles = tiles_m * tiles_n;
    // Walk the m-tiles starting at the first block of A that is in place at launch.
    const uint32_t rotate = p.a_ready ? p.a_local_first : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < kAccBuffers; a++) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], kEpilogueThreads / 32); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                uint32_t tm, tn;
                tile_coords(tile, tiles_m, tiles_n, tm, tn, GROUP_M, rotate);
                if (p.a_ready && !(tm - p.a_local_first < p.a_local_count)) {
                    // These rows come from another GPU: wait until they have landed.
                    if (!wait_rows_ready(p.a_ready + tm, p.a_epoch, &sh->abort_flag, status)) break;
                }
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->empty[stage], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY)) { ok = false; break; }
                    uint8_t* a_dst = smem + (size_t)stage * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_STAGE_BYTES;
                    mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, &sh->full[stage], (int32_t)(kb * TILE_K), (int32_t)(tm * TILE_M));
                    if (!p.b_is_kn) {
                        tma_load_2d(b_dst, &map_w, &sh->full[stage], (int32_t)(kb * TILE_K), (int32_t)(tn * TILE_N));
                    } else {
                        // B[K,N]: two boxes of 128 K-rows x 128 N-bytes, one per half of the 256 columns.
                        tma_load_2d(b_dst, &map_w, &sh->full[stage], (int32_t)(tn * TILE_N), (int32_t)(kb * TILE_K));
                        tma_load_2d(b_dst + B_STAGE_BYTES / 2, &map_w, &sh->full[stage], (int32_t)(tn * TILE_N + 128), (int32_t)(kb * TILE_K));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                if (!mbar_wait_bounded(&sh->acc_empty[acc], acc_phase ^ 1, &sh->abort_flag, status, TC_WAIT_ACC_EMPTY)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * TILE_N;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->full[stage], phase, &sh->abort_flag, status, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
                    if (!p.b_is_kn) {
                        const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + A_STAGE_BYTES);
                        #pragma unroll
                        for (int k = 0; k < TILE_K / MMA_K; k++) {
                            // Inside a 128-byte swizzle row the next K slice starts 32 bytes on: +2 in units of 16 bytes.
                            tc_mma_i8(d_tmem, a_desc + (uint64_t)(k * (MMA_K >> 4)), b_desc + (uint64_t)(k * (MMA_K >> 4)),
                                      kIdescI8, (kb | (uint32_t)k) != 0 ? 1u : 0u);
                        }
                    } else {
                        const uint64_t b_desc = make_mnmajor_sw128_desc(a_addr + A_STAGE_BYTES, B_STAGE_BYTES / 2);
                        #pragma unroll
                        for (int k = 0; k < TILE_K / MMA_K; k++) {
                            // The next K slice of an MN-major tile is 32 rows of 128 bytes further on.
                            tc_mma_i8(d_tmem, a_desc + (uint64_t)(k * (MMA_K >> 4)), b_desc + (uint64_t)(k * ((MMA_K * 128) >> 4)),
                                      kIdescI8BMn, (kb | (uint32_t)k) != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit(&sh->empty[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(&sh->acc_full[acc]);
                if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------- epilogue
        const uint32_t quarter = (uint32_t)warp & 3u;        // TMEM lanes this warp may read
        const int ew = warp - kEpilogueWarp0;
        float* s_scales = sh->w_scales + ew * TILE_N;
        float* s_bias = sh->bias + ew * TILE_N;
        uint8_t* my_tile = epi_tiles + ew * EPI_TILE_BYTES;
        const bool tma = tma_out != 0;
        const float a_scale = (MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) ? __ldg(p.a_scale) : 0.0f;
        const QuantConsts oq = make_quant_consts(MODE == EPI_DEQUANT_I8 ? __ldg(p.out_scale) : 1.0f, p.out_zp);
        float absmax = 0.0f;
        uint64_t staged_n0 = ~0ull;          // column block whose scales / bias / sums are in shared memory
        uint32_t acc = 0, acc_phase = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            uint32_t tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn, GROUP_M, rotate);
            const uint64_t n0 = (uint64_t)tn * TILE_N;
            const uint64_t m_base = (uint64_t)tm * TILE_M + quarter * 32;
            const uint64_t m = m_base + lane;
            if (n0 != staged_n0) { stage_columns<MODE>(p, n0, lane, s_scales, s_bias); staged_n0 = n0; }
            const int32_t row_sum = (MODE == EPI_REQUANT_I32 && p.a_row_sums && m < p.M) ? __ldg(p.a_row_sums + m) : 0;
            bool ok = mbar_wait_bounded(&sh->acc_full[acc], acc_phase, &sh->abort_flag, status, TC_WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            #pragma unroll 1
            for (int chunk = 0; chunk < TILE_N / 32; chunk++) {
                const uint64_t n_first = n0 + (uint64_t)chunk * 32;
                if (n_first >= p.N) break;
                uint32_t r[32];
                tc_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * TILE_N + (uint32_t)chunk * 32u, r);
                tc_wait_ld();
                epilogue_chunk<MODE, PEERS>(p, &map_out, tma, my_tile, r, m_base, lane, n_first, a_scale,
                                            s_scales + chunk * 32, s_bias + chunk * 32, oq, row_sum, absmax);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
            if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1; }
        }
        if (tma && lane == 0) bulk_wait_all();           // the last stores have left shared memory and are complete
        if ((MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) && p.absmax_out) absmax_publish(p.absmax_out, absmax);
    }

    // ----------------------------------------------------------------- teardown
    if (sh->abort_flag) {
        // Something gave up: let copies and MMAs already in flight land before
        // shared memory and TMEM are given back.
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// --------------------------------------------------------------------------- the CTA-pair kernel
// Two CTAs of a cluster (two SMs) work on one 256 x 256 output tile.  Each CTA
// loads 128 rows of A and 128 rows of W per stage (32 KiB instead of 48), the
// leader CTA's MMA thread issues tcgen05.mma.cta_group::2 (M = 256: the
// instruction reads both CTAs' shared memory at the same offsets, so each W
// half is fetched from shared memory once for both SMs), and each CTA's TMEM
// receives its own 128 rows of the accumulator, drained by its own epilogue
// warps.  Per SM this halves the W traffic through shared memory, which is what
// bounds the single-CTA kernel.  No TMA multicast: each CTA loads its own halves.
//
// Barriers: full[] lives in the leader (both CTAs' TMA loads signal it; the
// leader's producer arms it for the bytes of both); empty[] and acc_full[] are
// signalled in both CTAs by a multicast tcgen05.commit; acc_empty[] lives in
// the leader and collects the epilogue warps of both CTAs.
constexpr int PAIR_TILE_M = 256;
constexpr int kPairStages = 6;
constexpr uint32_t PAIR_A_BYTES = 128 * TILE_K;           // 16 KiB: this CTA's 128 rows of A
constexpr uint32_t PAIR_B_BYTES = 128 * TILE_K;           // 16 KiB: this CTA's 128 rows of W
constexpr uint32_t PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;

struct __align__(16) PairShared {
    uint64_t full[kPairStages];
    uint64_t empty[kPairStages];
    uint64_t acc_full[kAccBuffers];
    uint64_t acc_empty[kAccBuffers];
    uint32_t tmem_base;
    volatile int abort_flag;
    float w_scales[4 * TILE_N];
    float bias[4 * TILE_N];
};
constexpr size_t PAIR_SMEM_BYTES = 1024 + (size_t)kPairStages * PAIR_STAGE_BYTES + EPI_STAGE_BYTES + sizeof(PairShared);

constexpr uint32_t kIdescI8Pair = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(PAIR_TILE_M >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion is counted on an mbarrier that may live in the
// other CTA of the pair (bar_cluster_addr is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_i8_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_out, const GemmProblem p, uint32_t tiles_m, uint32_t tiles_n,
                       uint32_t num_kb, int tma_out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_tiles = smem + (size_t)kPairStages * PAIR_STAGE_BYTES;
    PairShared* sh = reinterpret_cast<PairShared*>(epi_tiles + EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_cta_rank();             // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t total_tiles = tiles_m * tiles_n;      // tiles of 256 x 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; s++) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < kAccBuffers; a++) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 2 * (kEpilogueThreads / 32)); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // the peer's barriers are initialised too
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = pair; ok && tile < total_tiles; tile += num_pairs) {
                uint32_t tm, tn;
                tile_coords(tile, tiles_m, tiles_n, tm, tn, PAIR_GROUP_M);
                const int32_t a_row = (int32_t)(tm * PAIR_TILE_M + cta * 128);
                const int32_t w_row = (int32_t)(tn * TILE_N + cta * 128);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->empty[stage], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY)) { ok = false; break; }
                    uint8_t* a_dst = smem + (size_t)stage * PAIR_STAGE_BYTES;
                    uint8_t* b_dst = a_dst + PAIR_A_BYTES;
                    const uint32_t leader_full = map_to_cta(smem_u32(&sh->full[stage]), 0);
                    if (cta == 0) mbar_expect_tx(&sh->full[stage], 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &map_a, leader_full, (int32_t)(kb * TILE_K), a_row);
                    tma_load_2d_pair(b_dst, &map_w, leader_full, (int32_t)(kb * TILE_K), w_row);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && cta == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t tile = pair; ok && tile < total_tiles; tile += num_pairs) {
                if (!mbar_wait_bounded(&sh->acc_empty[acc], acc_phase ^ 1, &sh->abort_flag, status, TC_WAIT_ACC_EMPTY)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * TILE_N;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->full[stage], phase, &sh->abort_flag, status, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)stage * PAIR_STAGE_BYTES);
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
                    const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + PAIR_A_BYTES);
                    #pragma unroll
                    for (int k = 0; k < TILE_K / MMA_K; k++) {
                        tc_mma_i8_pair(d_tmem, a_desc + (uint64_t)(k * (MMA_K >> 4)), b_desc + (uint64_t)(k * (MMA_K >> 4)),
                                       kIdescI8Pair, (kb | (uint32_t)k) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair(&sh->empty[stage]);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit_pair(&sh->acc_full[acc]);
                if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        const uint32_t quarter = (uint32_t)warp & 3u;
        const int ew = warp - kEpilogueWarp0;
        float* s_scales = sh->w_scales + ew * TILE_N;
        float* s_bias = sh->bias + ew * TILE_N;
        uint8_t* my_tile = epi_tiles + ew * EPI_TILE_BYTES;
        const bool tma = tma_out != 0;
        const float a_scale = (MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) ? __ldg(p.a_scale) : 0.0f;
        const QuantConsts oq = make_quant_consts(MODE == EPI_DEQUANT_I8 ? __ldg(p.out_scale) : 1.0f, p.out_zp);
        float absmax = 0.0f;
        uint64_t staged_n0 = ~0ull;          // column block whose scales / bias / sums are in shared memory
        uint32_t acc = 0, acc_phase = 0;
        for (uint32_t tile = pair; tile < total_tiles; tile += num_pairs) {
            uint32_t tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn, PAIR_GROUP_M);
            const uint64_t n0 = (uint64_t)tn * TILE_N;
            const uint64_t m_base = (uint64_t)tm * PAIR_TILE_M + cta * 128 + quarter * 32;
            const uint64_t m = m_base + lane;
            if (n0 != staged_n0) { stage_columns<MODE>(p, n0, lane, s_scales, s_bias); staged_n0 = n0; }
            const int32_t row_sum = (MODE == EPI_REQUANT_I32 && p.a_row_sums && m < p.M) ? __ldg(p.a_row_sums + m) : 0;
            bool ok = mbar_wait_bounded(&sh->acc_full[acc], acc_phase, &sh->abort_flag, status, TC_WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            #pragma unroll 1
            for (int chunk = 0; chunk < TILE_N / 32; chunk++) {
                const uint64_t n_first = n0 + (uint64_t)chunk * 32;
                if (n_first >= p.N) break;
                uint32_t r[32];
                tc_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * TILE_N + (uint32_t)chunk * 32u, r);
                tc_wait_ld();
                epilogue_chunk<MODE, false>(p, &map_out, tma, my_tile, r, m_base, lane, n_first, a_scale,
                                            s_scales + chunk * 32, s_bias + chunk * 32, oq, row_sum, absmax);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->acc_empty[acc]), 0));
            if (++acc == kAccBuffers) { acc = 0; acc_phase ^= 1; }
        }
        if (tma && lane == 0) bulk_wait_all();
        if ((MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) && p.absmax_out) absmax_publish(p.absmax_out, absmax);
    }

    // ----------------------------------------------------------------- teardown
    if (sh->abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves while the other may still touch its barriers or shared memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// --------------------------------------------------------------------------- the wide single-CTA kernel
// One CTA computes a 256 x 256 output tile as two 128 x 256 accumulators that
// share every W stage: per K step the CTA loads 256 rows of A and 256 rows of W
// (64 KiB, three stages) and issues the MMAs of the upper and the lower half
// against the same W tile.  Against the 128 x 256 kernel this moves a third
// less data from L2 to the SM per output (512 instead of 768 rows per 256 x 256
// outputs); the price is that both accumulators belong to one tile, so the
// epilogue does not overlap the next tile's main loop.  At the board's power
// cap what counts is energy per operation, not idle cycles.
constexpr int WIDE_TILE_M = 256;
constexpr int kWideStages = 3;
constexpr int kWideEpilogueWarps = 8;                     // two per TMEM lane quarter, each takes every other 32-column chunk
constexpr int WIDE_THREADS = (2 + kWideEpilogueWarps) * 32;
constexpr uint32_t WIDE_EPI_BYTES = kWideEpilogueWarps * EPI_TILE_BYTES;   // a 4 KiB staging tile per epilogue warp
constexpr uint32_t kWideEpilogueBarrier = 1;              // named barrier of the eight epilogue warps (0 is __syncthreads')
constexpr uint32_t WIDE_A_BYTES = WIDE_TILE_M * TILE_K;   // 32 KiB
constexpr uint32_t WIDE_B_BYTES = TILE_N * TILE_K;        // 32 KiB
constexpr uint32_t WIDE_STAGE_BYTES = WIDE_A_BYTES + WIDE_B_BYTES;
constexpr int WIDE_GROUP_M = 16;     // 256-row m-tiles per rasterisation group; measured on the large GEMM (sustained):
                                     // 8 / 12 / 16 -> 27.6-27.7 ms, 6 -> 28.3 ms, 24 -> 28.6 ms, 32 -> 29.4 ms

struct __align__(16) WideShared {
    uint64_t full[kWideStages];
    uint64_t empty[kWideStages];
    uint64_t acc_full;               // MMA -> epilogue: both accumulators complete
    uint64_t acc_empty[2];           // epilogue -> MMA: the upper / the lower accumulator drained
    uint32_t tmem_base;
    volatile int abort_flag;
    alignas(16) float w_scales[TILE_N];   // one copy for all epilogue warps (the eight staging tiles leave no room for more)
    alignas(16) float bias[TILE_N];
};
// The stage ring needs a 1024-byte aligned base.  Dynamic shared memory starts at a 128-byte boundary at least on
// this architecture (in practice at a 1024-byte one), so 896 bytes of slack are asked for instead of 1024: with the
// eight staging tiles every byte counts (232,400 of the 232,448 a CTA may have).  The kernel checks the assumption
// and gives up with a status code, touching nothing, if it ever fails.
constexpr size_t WIDE_ALIGN_SLACK = 896;
constexpr size_t WIDE_SMEM_BYTES = WIDE_ALIGN_SLACK + (size_t)kWideStages * WIDE_STAGE_BYTES + WIDE_EPI_BYTES + sizeof(WideShared);
static_assert(WIDE_SMEM_BYTES <= 232448, "the 256 x 256 kernel's shared memory exceeds what a CTA may have");

template <int MODE>
__global__ void __launch_bounds__(WIDE_THREADS, 1)
gemm_i8_tc_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_out, const GemmProblem p, uint32_t tiles_m, uint32_t tiles_n,
                       uint32_t num_kb, int tma_out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_tiles = smem + (size_t)kWideStages * WIDE_STAGE_BYTES;
    WideShared* sh = reinterpret_cast<WideShared*>(epi_tiles + WIDE_EPI_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t total_tiles = tiles_m * tiles_n;      // tiles of 256 x 256
    if ((size_t)(smem - smem_raw) > WIDE_ALIGN_SLACK) {   // never seen; see WIDE_ALIGN_SLACK
        if (threadIdx.x == 0) atomicCAS(status, 0, (int)TC_SMEM_BASE);
        return;
    }
    // Walk the m-tiles starting at the tile that holds the first block of A in place at launch.
    const uint32_t rotate = p.a_ready ? p.a_local_first / 2 : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWideStages; s++) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        mbar_init(&sh->acc_full, 1);
        mbar_init(&sh->acc_empty[0], kWideEpilogueWarps);
        mbar_init(&sh->acc_empty[1], kWideEpilogueWarps);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                uint32_t tm, tn;
                tile_coords(tile, tiles_m, tiles_n, tm, tn, WIDE_GROUP_M, rotate);
                if (p.a_ready) {
                    // A 256-row tile spans two arrival words; rows that come from another GPU must have landed.
                    const uint32_t blocks = (uint32_t)((p.M + 127) / 128);
                    for (uint32_t b = 2 * tm; ok && b < 2 * tm + 2 && b < blocks; b++)
                        if (!(b - p.a_local_first < p.a_local_count))
                            ok = wait_rows_ready(p.a_ready + b, p.a_epoch, &sh->abort_flag, status);
                    if (!ok) break;
                }
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->empty[stage], phase ^ 1, &sh->abort_flag, status, TC_WAIT_EMPTY)) { ok = false; break; }
                    uint8_t* a_dst = smem + (size_t)stage * WIDE_STAGE_BYTES;
                    uint8_t* b_dst = a_dst + WIDE_A_BYTES;
                    mbar_expect_tx(&sh->full[stage], WIDE_STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, &sh->full[stage], (int32_t)(kb * TILE_K), (int32_t)(tm * WIDE_TILE_M));
                    tma_load_2d(b_dst, &map_w, &sh->full[stage], (int32_t)(kb * TILE_K), (int32_t)(tn * TILE_N));
                    if (++stage == kWideStages) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                // The epilogue drains the upper accumulator first.  As soon as that one is free the next tile's
                // main loop starts on it; the MMAs of the lower half of up to kWideStages K blocks are held back
                // (their stages stay occupied) until the lower accumulator is free too, so about half of the
                // epilogue runs under tensor work although both accumulators belong to one tile.
                if (!mbar_wait_bounded(&sh->acc_empty[0], acc_phase ^ 1, &sh->abort_flag, status, TC_WAIT_ACC_EMPTY)) break;
                tc_fence_after();
                bool lower_free = false;
                uint32_t held = 0, held_stage[kWideStages], held_kb[kWideStages];
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_bounded(&sh->full[stage], phase, &sh->abort_flag, status, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    {
                        const uint32_t a_addr = smem_u32(smem + (size_t)stage * WIDE_STAGE_BYTES);
                        const uint64_t a_lo = make_kmajor_sw128_desc(a_addr);
                        const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + WIDE_A_BYTES);
                        #pragma unroll
                        for (int k = 0; k < TILE_K / MMA_K; k++) {
                            const uint64_t adv = (uint64_t)(k * (MMA_K >> 4));
                            tc_mma_i8(tmem_base, a_lo + adv, b_desc + adv, kIdescI8, (kb | (uint32_t)k) != 0 ? 1u : 0u);   // columns 0..255
                        }
                    }
                    held_stage[held] = stage;
                    held_kb[held] = kb;
                    held++;
                    if (!lower_free) {
                        if (held == (uint32_t)kWideStages || kb + 1 == num_kb) {
                            // Every stage is held (or the tile ends): nothing more can be done without the lower accumulator.
                            if (!mbar_wait_bounded(&sh->acc_empty[1], acc_phase ^ 1, &sh->abort_flag, status, TC_WAIT_ACC_EMPTY)) { ok = false; break; }
                            lower_free = true;
                        } else {
                            lower_free = mbar_try_wait(&sh->acc_empty[1], acc_phase ^ 1);
                        }
                        if (lower_free) tc_fence_after();
                    }
                    if (lower_free) {
                        for (uint32_t h = 0; h < held; h++) {
                            const uint32_t a_addr = smem_u32(smem + (size_t)held_stage[h] * WIDE_STAGE_BYTES);
                            const uint64_t a_hi = make_kmajor_sw128_desc(a_addr + 128 * TILE_K);     // rows 128..255 of the A stage
                            const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + WIDE_A_BYTES);
                            #pragma unroll
                            for (int k = 0; k < TILE_K / MMA_K; k++) {
                                const uint64_t adv = (uint64_t)(k * (MMA_K >> 4));
                                tc_mma_i8(tmem_base + TILE_N, a_hi + adv, b_desc + adv, kIdescI8, (held_kb[h] | (uint32_t)k) != 0 ? 1u : 0u);   // columns 256..511
                            }
                            tc_commit(&sh->empty[held_stage[h]]);
                        }
                        held = 0;
                    }
                    if (++stage == kWideStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(&sh->acc_full);
                acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------- epilogue
        // Eight warps.  The epilogue of this kernel is not hidden under a main loop (both accumulators belong to one
        // tile), and measured with timestamps it is a chain of latencies per 32-column chunk (TMEM load, conversion,
        // staging, proxy fence, store issue: about 800 cycles) that a warp walks once per chunk it owns.  The two
        // warps that may read a TMEM lane quarter therefore take every other chunk each, with a staging tile of
        // their own: eight steps per tile and warp instead of sixteen.
        const uint32_t quarter = (uint32_t)warp & 3u;
        const int ew = warp - kEpilogueWarp0;
        const int first_chunk = ew >> 2;                     // warps 2-5: chunks 0, 2, 4, 6; warps 6-9: chunks 1, 3, 5, 7
        float* s_scales = sh->w_scales;
        float* s_bias = sh->bias;
        uint8_t* my_tile = epi_tiles + ew * EPI_TILE_BYTES;
        const bool tma = tma_out != 0;
        const float a_scale = (MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) ? __ldg(p.a_scale) : 0.0f;
        const QuantConsts oq = make_quant_consts(MODE == EPI_DEQUANT_I8 ? __ldg(p.out_scale) : 1.0f, p.out_zp);
        float absmax = 0.0f;
        uint64_t staged_n0 = ~0ull;
        uint32_t acc_phase = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            uint32_t tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn, WIDE_GROUP_M, rotate);
            const uint64_t n0 = (uint64_t)tn * TILE_N;
            bool ok = mbar_wait_bounded(&sh->acc_full, acc_phase, &sh->abort_flag, status, TC_WAIT_ACC_FULL);
            // All eight warps go on, or none: they are about to meet at a barrier.  Everyone who arrives here has
            // also finished the previous tile, so the shared per-column values may be replaced.
            ok = named_barrier_all(kWideEpilogueBarrier, kWideEpilogueWarps * 32, ok);
            if (!ok) break;
            if (n0 != staged_n0) {                           // the same test in every warp
                if (ew == 0) stage_columns<MODE>(p, n0, lane, s_scales, s_bias);
                named_barrier(kWideEpilogueBarrier, kWideEpilogueWarps * 32);
                staged_n0 = n0;
            }
            tc_fence_after();
            #pragma unroll 1
            for (int half = 0; half < 2; half++) {
                const uint64_t m_base = (uint64_t)tm * WIDE_TILE_M + half * 128 + quarter * 32;
                const uint64_t m = m_base + lane;
                const int32_t row_sum = (MODE == EPI_REQUANT_I32 && p.a_row_sums && m < p.M) ? __ldg(p.a_row_sums + m) : 0;
                #pragma unroll 1
                for (int chunk = first_chunk; chunk < TILE_N / 32; chunk += 2) {
                    const uint64_t n_first = n0 + (uint64_t)chunk * 32;
                    if (n_first >= p.N) break;
                    uint32_t r[32];
                    tc_ld_32x32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)half * TILE_N + (uint32_t)chunk * 32u, r);
                    tc_wait_ld();
                    epilogue_chunk<MODE, false>(p, &map_out, tma, my_tile, r, m_base, lane, n_first, a_scale,
                                                s_scales + chunk * 32, s_bias + chunk * 32, oq, row_sum, absmax);
                }
                // This half's accumulator has been read: the next tile's MMAs may overwrite it.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->acc_empty[half]);
            }
            acc_phase ^= 1;
        }
        if (tma && lane == 0) bulk_wait_all();
        if ((MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) && p.absmax_out) absmax_publish(p.absmax_out, absmax);
    }

    // ----------------------------------------------------------------- teardown
    if (sh->abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// --------------------------------------------------------------------------- self-test of the bounded wait
// One warp waits, with a limit of about a millisecond, on an mbarrier that
// nothing ever arrives on.  The wait must give up, record its code in the
// status word and let the kernel return normally; result[0] = 1 when
// mbar_wait_bounded returned false, result[1] = the abort flag it raised.
__global__ void bounded_wait_selftest_kernel(int* status, int* result, long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait_bounded(&bar, 0, &abort_flag, status, TC_WAIT_SELFTEST, limit_cycles);
        result[0] = ok ? 0 : 1;
        result[1] = abort_flag;
    }
}

// --------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the
// library does not link against libcuda directly.
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        else
            cudaGetLastError();
    });
    return fn;
}

// Tensor maps depend only on the address, the shape and the box, not on the
// contents, so a layer that is called again with the same buffers gets its maps
// from a small per-thread cache instead of from the driver.
struct MapKey {
    const void* base;
    uint64_t dim0, dim1, stride;
    uint32_t box0, box1;
    int elem;                        // 1 = int8 operand, 4 = four-byte output
    bool operator==(const MapKey& o) const {
        return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && stride == o.stride && box0 == o.box0 &&
               box1 == o.box1 && elem == o.elem;
    }
};
constexpr int kMapCacheEntries = 16;
struct MapCache {
    MapKey key[kMapCacheEntries];
    CUtensorMap map[kMapCacheEntries];
    int used = 0, next = 0;
};
static thread_local MapCache t_maps;

// 2-D map of a row-major matrix: dim0 contiguous elements per row, dim1 rows, row
// stride in bytes; box0 x box1 elements per copy, 128-byte swizzle.
int make_map_2d(CUtensorMap* map, const void* base, int elem, uint64_t dim0, uint64_t dim1, uint64_t stride_bytes,
                       uint32_t box0, uint32_t box1, const char* what) {
    const MapKey key = {base, dim0, dim1, stride_bytes, box0, box1, elem};
    for (int i = 0; i < t_maps.used; i++)
        if (t_maps.key[i] == key) { *map = t_maps.map[i]; return 0; }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(RPLB_E_NO_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)dim0, (cuuint64_t)dim1};
    cuuint64_t strides[1] = {(cuuint64_t)stride_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    // elem: 1 = bytes, 4 = four-byte values, both with the 128-byte swizzle; 5 = four-byte values laid out plainly
    CUresult r = enc(map, elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base),
                     dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, elem == 5 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RPLB_E_BAD_ARG, "cuTensorMapEncodeTiled (%s) failed with CUresult %d", what, (int)r);
    const int slot = t_maps.next;
    t_maps.key[slot] = key;
    t_maps.map[slot] = *map;
    t_maps.next = (slot + 1) % kMapCacheEntries;
    if (t_maps.used < kMapCacheEntries) t_maps.used++;
    return 0;
}

// Map of a row-major [rows, K] int8 matrix, box = box_rows x 128 bytes.
static int make_map(CUtensorMap* map, const int8_t* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    return make_map_2d(map, base, 1, K, rows, K, (uint32_t)TILE_K, box_rows, "operand [rows,K]");
}

// Map of gemm_int8's row-major B [K, N]: inner dimension N, box = 128 N-bytes x 128 K-rows.
static int make_map_kn(CUtensorMap* map, const int8_t* base, uint64_t K, uint64_t N) {
    return make_map_2d(map, base, 1, N, K, N, 128, (uint32_t)TILE_K, "B [K,N]");
}

// Which store path this host thread's GEMMs use: 0 = through the tensor map when
// the output allows it, 1 = always from registers.
static thread_local int t_epilogue = 0;
int thread_gemm_epilogue(int which) {
    const int prev = t_epilogue;
    if (which == 0 || which == 1) t_epilogue = which;
    return prev;
}

// Map of the four-byte output [M, ldo] (N valid columns), box = 32 x 32 values, for
// the epilogue's stores.  *usable = 0 when the output cannot be described (base or
// row stride not a multiple of 16 bytes, int8 output) or the caller asked for
// register stores; the kernel then stores from registers.
static int make_map_out(CUtensorMap* map, const GemmProblem& p, int* usable) {
    *usable = 0;
    memset(map, 0, sizeof(*map));
    if (t_epilogue == 1 || p.mode == EPI_DEQUANT_I8) return 0;
    if (((uintptr_t)p.out & 15) || (p.ldo % 4) != 0 || p.ldo * 4 >= (1ull << 40)) return 0;
    if (int rc = make_map_2d(map, p.out, 4, p.N, p.M, p.ldo * 4, 32, 32, "output")) return rc;
    *usable = 1;
    return 0;
}

bool gemm_tcgen05_supports(const GemmProblem& p) {
    // B as [K,N] is read in place by the 128 x 256 kernel (MN-major operand) when its rows are 16-byte multiples.
    if (p.b_is_kn && p.N % 16 != 0) return false;
    if (p.M == 0 || p.N == 0 || p.K == 0) return false;
    if (p.K % 16 != 0) return false;                              // TMA: row stride in multiples of 16 bytes
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.B & 15)) return false;
    // zero points need the row sums of A and the column sums of B for the epilogue correction
    if (p.mode == EPI_REQUANT_I32 && (p.za != 0 || p.zb != 0) && !(p.a_row_sums && p.b_col_sums)) return false;
    if (p.M > 0x7fffffffull || p.N > 0x7fffffffull || p.K > 0x7fffffffull) return false;
    const uint64_t tiles = ((p.M + TILE_M - 1) / TILE_M) * ((p.N + TILE_N - 1) / TILE_N);
    return tiles < 0x7fffffffull;
}

// Status words the kernels write when a bounded wait expires: page-locked host
// memory mapped into the device, so the host can read them without touching a
// stream.  Every host thread launches with a word of its own (threads beyond
// kStatusSlots share), so a give-up is reported to the thread whose kernel it was.
constexpr int kStatusSlots = 1024;
static int* kernel_status_words() {
    static int* words = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        if (cudaHostAlloc(&p, kStatusSlots * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
            words = static_cast<int*>(p);
            memset(words, 0, kStatusSlots * sizeof(int));
        } else {
            cudaGetLastError();
        }
    });
    return words;
}
static int* kernel_status_word() {
    static std::atomic<unsigned int> next_slot{0};
    static thread_local int slot = -1;
    int* words = kernel_status_words();
    if (!words) return nullptr;
    if (slot < 0) slot = (int)(next_slot.fetch_add(1) % kStatusSlots);
    return words + slot;
}

// Runs the kernel above and checks that the give-up path works end to end:
// the kernel returns, the status word carries the code, and clearing it leaves
// the library usable.  Returns 0 when everything behaved as designed.
int bounded_wait_selftest(cudaStream_t st) {
    int* status_host = kernel_status_word();
    if (!status_host) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
    if (*reinterpret_cast<volatile int*>(status_host) != 0)
        return fail(RPLB_E_KERNEL, "status word not clear before the self-test (%d)", *status_host);
    int* status_dev = nullptr;
    if (int rc = cuda_ok(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0), "cudaHostGetDevicePointer")) return rc;
    int* result = nullptr;
    if (int rc = cuda_ok(cudaMalloc((void**)&result, 2 * sizeof(int)), "cudaMalloc(selftest)")) return rc;
    cudaMemsetAsync(result, 0xff, 2 * sizeof(int), st);
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(status_dev, result, 2000000LL);
    int rc = launched("bounded_wait_selftest_kernel");
    int host_result[2] = {-1, -1};
    if (!rc) rc = cuda_ok(cudaMemcpyAsync(host_result, result, sizeof(host_result), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(selftest)");
    if (!rc) rc = cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize(selftest)");
    cudaFree(result);
    if (rc) return rc;
    const int code = *reinterpret_cast<volatile int*>(status_host);
    *reinterpret_cast<volatile int*>(status_host) = 0;
    if (host_result[0] != 1 || host_result[1] != 1 || code != TC_WAIT_SELFTEST)
        return fail(RPLB_E_KERNEL, "bounded wait self-test: gave_up=%d abort=%d status=%d (expected 1, 1, %d)",
                    host_result[0], host_result[1], code, (int)TC_WAIT_SELFTEST);
    return 0;
}

// The same give-up, left in the calling thread's status word for the caller to find.
int bounded_wait_leave_status(cudaStream_t st) {
    int* status_host = kernel_status_word();
    if (!status_host) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
    int* status_dev = nullptr;
    if (int rc = cuda_ok(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0), "cudaHostGetDevicePointer")) return rc;
    int* result = nullptr;
    if (int rc = cuda_ok(cudaMalloc((void**)&result, 2 * sizeof(int)), "cudaMalloc(selftest)")) return rc;
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(status_dev, result, 2000000LL);
    int rc = launched("bounded_wait_selftest_kernel");
    if (!rc) rc = cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize(selftest)");
    cudaFree(result);
    return rc;
}

int* kernel_status_word_device() {
    int* host = kernel_status_word();
    if (!host) return nullptr;
    int* dev = nullptr;
    if (cudaHostGetDevicePointer((void**)&dev, host, 0) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return dev;
}

int gemm_tcgen05_status(bool clear) {
    int* w = kernel_status_word();
    if (!w) return 0;
    int v = *reinterpret_cast<volatile int*>(w);
    if (clear) *reinterpret_cast<volatile int*>(w) = 0;
    return v;
}

// Opting in to more than 48 KiB of dynamic shared memory is a per-device
// attribute of each kernel: set once per (kernel, device), remembered here.
constexpr int kMaxDevices = 64;
enum KernelFamily : int { FAM_TC = 0, FAM_TC_PEERS = 1, FAM_PAIR = 2, FAM_WIDE = 3, FAM_COUNT = 4 };
static std::atomic<uint64_t> g_attr_done[FAM_COUNT][4];      // one bit per device ordinal
static std::atomic<int> g_resident_pairs[kMaxDevices][4];    // 0 = not asked yet

template <typename Kernel>
static int ensure_smem_attr(Kernel kernel, int family, int mode, size_t bytes, const char* what) {
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    if (tracked && ((g_attr_done[family][mode].load(std::memory_order_acquire) >> dev) & 1ull)) return 0;
    if (int rc = cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what)) return rc;
    if (tracked) g_attr_done[family][mode].fetch_or(1ull << dev, std::memory_order_release);
    return 0;
}

template <int MODE, bool PEERS = false>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmProblem& p, uint32_t tiles_m,
                     uint32_t tiles_n, uint32_t num_kb, int tma_out, int* status_dev, unsigned int grid, cudaStream_t st) {
    if (int rc = ensure_smem_attr(gemm_i8_tc_kernel<MODE, PEERS>, PEERS ? FAM_TC_PEERS : FAM_TC, MODE, TC_SMEM_BYTES,
                                  "cudaFuncSetAttribute(gemm_i8_tc_kernel)")) return rc;
    gemm_i8_tc_kernel<MODE, PEERS><<<grid, TC_THREADS, TC_SMEM_BYTES, st>>>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev);
    return launched("gemm_i8_tc_kernel");
}

// How many CTA pairs can be resident at once (SMs pair up inside a TPC; a GPC
// with an odd number of usable SMs leaves one without a partner).  Asked once
// per device and epilogue mode.
template <int MODE>
static int max_resident_pairs(int* pairs) {
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    if (tracked) {
        const int known = g_resident_pairs[dev][MODE].load(std::memory_order_acquire);
        if (known > 0) { *pairs = known; return 0; }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (int rc = cuda_ok(cudaOccupancyMaxActiveClusters(&n, gemm_i8_tc_pair_kernel<MODE>, &cfg), "cudaOccupancyMaxActiveClusters")) return rc;
    if (tracked && n > 0) g_resident_pairs[dev][MODE].store(n, std::memory_order_release);
    *pairs = n;
    return 0;
}

template <int MODE>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmProblem& p, uint32_t num_kb,
                          int tma_out, int* status_dev, cudaStream_t st) {
    if (int rc = ensure_smem_attr(gemm_i8_tc_pair_kernel<MODE>, FAM_PAIR, MODE, PAIR_SMEM_BYTES,
                                  "cudaFuncSetAttribute(gemm_i8_tc_pair_kernel)")) return rc;
    int pairs = 0;
    if (int rc = max_resident_pairs<MODE>(&pairs)) return rc;
    if (pairs <= 0) return fail(RPLB_E_UNSUPPORTED, "no CTA pair fits on this device");
    const uint32_t tiles_m = (uint32_t)((p.M + PAIR_TILE_M - 1) / PAIR_TILE_M);
    const uint32_t tiles_n = (uint32_t)((p.N + TILE_N - 1) / TILE_N);
    const uint64_t tiles = (uint64_t)tiles_m * tiles_n;
    if (tiles < (uint64_t)pairs) pairs = (int)tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned int)pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_i8_tc_pair_kernel<MODE>, ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev);
    if (e != cudaSuccess) return cuda_ok(e, "cudaLaunchKernelEx(gemm_i8_tc_pair_kernel)");
    return launched("gemm_i8_tc_pair_kernel");
}

template <int MODE>
static int launch_tc_wide(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmProblem& p, uint32_t num_kb,
                          int tma_out, int* status_dev, unsigned int sms, cudaStream_t st) {
    if (int rc = ensure_smem_attr(gemm_i8_tc_wide_kernel<MODE>, FAM_WIDE, MODE, WIDE_SMEM_BYTES,
                                  "cudaFuncSetAttribute(gemm_i8_tc_wide_kernel)")) return rc;
    const uint32_t tiles_m = (uint32_t)((p.M + WIDE_TILE_M - 1) / WIDE_TILE_M);
    const uint32_t tiles_n = (uint32_t)((p.N + TILE_N - 1) / TILE_N);
    const uint64_t tiles = (uint64_t)tiles_m * tiles_n;
    const unsigned int grid = (unsigned int)(tiles < sms ? tiles : sms);
    gemm_i8_tc_wide_kernel<MODE><<<grid, WIDE_THREADS, WIDE_SMEM_BYTES, st>>>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev);
    return launched("gemm_i8_tc_wide_kernel");
}

// variant: 0 = choose, 1 = one CTA per 128 x 256 tile, 2 = CTA pair per 256 x 256 tile,
// 3 = one CTA per 256 x 256 tile (two accumulators sharing each W stage), 4 = the kernel for few output
// features (N <= 128, K <= 896, fp32 epilogue; gemm_i8_fused_quant.cu).
int gemm_tcgen05(const GemmProblem& p, cudaStream_t st, int variant) {
    if (!gemm_tcgen05_supports(p))
        return fail(RPLB_E_UNSUPPORTED, "tcgen05 GEMM needs W as [N,K], K %% 16 == 0, 16-byte aligned A and W");
    if (int prev = gemm_tcgen05_status(true))
        return fail(RPLB_E_KERNEL, "an earlier tcgen05 GEMM of this thread gave up waiting (code %d)", prev);
    int* status_host = kernel_status_word();
    if (!status_host) return fail(RPLB_E_NO_DEVICE, "could not allocate the kernel status word");
    int* status_dev = nullptr;
    if (int rc = cuda_ok(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0), "cudaHostGetDevicePointer")) return rc;

    const uint32_t num_kb = (uint32_t)((p.K + TILE_K - 1) / TILE_K);
    unsigned int sms = (unsigned int)sm_count();
    if (sms == 0) sms = 148;
    if (p.b_is_kn) variant = 1;          // only the 128 x 256 kernel reads B[K,N] in place
    if (p.n_peers > 0) {
        // Only the 128 x 256 kernel with the fp32 epilogue stores to further destinations.
        if (p.mode != EPI_DEQUANT_F32 || p.b_is_kn || p.n_peers > kMaxPeers)
            return fail(RPLB_E_UNSUPPORTED, "peer destinations need the fp32 epilogue, W as [N,K] and at most %d peers", kMaxPeers);
        variant = 1;
    }
    // A GEMM long enough for the board to settle on its power cap: what counts then is work per joule.
    const bool sustained = (double)p.M * (double)p.N * (double)p.K >= 1.1e12;
    // The 256 x 256 kernel does not overlap a tile's epilogue with the next tile's main loop, so it needs a long
    // reduction to come out ahead: +4 % at K = 8192, -1 % at K = 4096 (the fused Q/K/V projection) against
    // the 128 x 256 kernel.
    const bool wide_pays = sustained && p.K >= 6144;
    if (p.a_ready) {
        // The 128 x 256 kernel and the 256 x 256 kernel wait for rows that are still arriving.
        const uint64_t tiles_m = (p.M + TILE_M - 1) / TILE_M;
        if (p.b_is_kn || (uint64_t)p.a_local_first + p.a_local_count > tiles_m || (p.a_local_first >= tiles_m && tiles_m))
            return fail(RPLB_E_BAD_ARG, "arriving rows: local blocks [%u, +%u) outside the %llu row blocks of A",
                        p.a_local_first, p.a_local_count, (unsigned long long)tiles_m);
        variant = (variant == 3 || (variant == 0 && wide_pays)) ? 3 : 1;
    }
    if (variant == 4) return gemm_narrow(p, st);         // asked for by name: refused if the shape does not fit
    if (variant == 0 && gemm_narrow_supports(p) && p.M >= (uint64_t)TILE_M * sms) {
        // Few output features over many rows: an HBM-bound layer.  The kernel that keeps the whole weight matrix
        // in shared memory and cuts the accumulator into four 128-column buffers hands tiles over faster than
        // the 256-column kernels, which compute (and wait for) columns that do not exist.
        return gemm_narrow(p, st);
    }
    if (variant == 0) {
        // Measured on B200 (1000 W cap): un-throttled, the pair kernel keeps the
        // tensor pipe busier (86 % against 71 % of cycles) and is ~10 % faster than
        // the 128 x 256 kernel; in a long run every kernel sits at the power cap and
        // the order is work per joule: the 256 x 256 single-CTA kernel (a third less
        // operand traffic into the SM) runs at ~1.42 GHz against ~1.38 GHz and is
        // ~4 % faster than the 128 x 256 kernel, which in turn beats the pair kernel
        // by ~6 %.  So: the 256 x 256 kernel for GEMMs long enough for the governor
        // to settle whose reduction is long enough to hide its exposed epilogue; the
        // 128 x 256 kernel for the other long ones; the pair kernel for shorter ones,
        // provided every pair of SMs gets a 256 x 256 tile of its own; the 128 x 256
        // kernel otherwise.
        const uint64_t pair_tiles = ((p.M + PAIR_TILE_M - 1) / PAIR_TILE_M) * ((p.N + TILE_N - 1) / TILE_N);
        variant = wide_pays ? 3 : (sustained ? 1 : (pair_tiles >= sms / 2 ? 2 : 1));
    }
    CUtensorMap ma, mw, mo;
    int tma_out = 0;
    if (int rc = make_map_out(&mo, p, &tma_out)) return rc;
    if (variant == 3) {
        if (int rc = make_map(&ma, p.A, p.M, p.K, WIDE_TILE_M)) return rc;
        if (int rc = make_map(&mw, p.B, p.N, p.K, TILE_N)) return rc;
        switch (p.mode) {
            case EPI_RAW_I32:     return launch_tc_wide<EPI_RAW_I32>(ma, mw, mo, p, num_kb, tma_out, status_dev, sms, st);
            case EPI_REQUANT_I32: return launch_tc_wide<EPI_REQUANT_I32>(ma, mw, mo, p, num_kb, tma_out, status_dev, sms, st);
            case EPI_DEQUANT_F32: return launch_tc_wide<EPI_DEQUANT_F32>(ma, mw, mo, p, num_kb, tma_out, status_dev, sms, st);
            case EPI_DEQUANT_I8:  return launch_tc_wide<EPI_DEQUANT_I8>(ma, mw, mo, p, num_kb, tma_out, status_dev, sms, st);
        }
        return fail(RPLB_E_BAD_ARG, "unknown epilogue mode %d", p.mode);
    }
    if (variant == 2) {
        if (int rc = make_map(&ma, p.A, p.M, p.K, 128)) return rc;
        if (int rc = make_map(&mw, p.B, p.N, p.K, 128)) return rc;
        switch (p.mode) {
            case EPI_RAW_I32:     return launch_tc_pair<EPI_RAW_I32>(ma, mw, mo, p, num_kb, tma_out, status_dev, st);
            case EPI_REQUANT_I32: return launch_tc_pair<EPI_REQUANT_I32>(ma, mw, mo, p, num_kb, tma_out, status_dev, st);
            case EPI_DEQUANT_F32: return launch_tc_pair<EPI_DEQUANT_F32>(ma, mw, mo, p, num_kb, tma_out, status_dev, st);
            case EPI_DEQUANT_I8:  return launch_tc_pair<EPI_DEQUANT_I8>(ma, mw, mo, p, num_kb, tma_out, status_dev, st);
        }
        return fail(RPLB_E_BAD_ARG, "unknown epilogue mode %d", p.mode);
    }
    if (int rc = make_map(&ma, p.A, p.M, p.K, TILE_M)) return rc;
    if (int rc = p.b_is_kn ? make_map_kn(&mw, p.B, p.K, p.N) : make_map(&mw, p.B, p.N, p.K, TILE_N)) return rc;
    const uint32_t tiles_m = (uint32_t)((p.M + TILE_M - 1) / TILE_M);
    const uint32_t tiles_n = (uint32_t)((p.N + TILE_N - 1) / TILE_N);
    const uint64_t tiles = (uint64_t)tiles_m * tiles_n;
    const unsigned int grid = (unsigned int)(tiles < sms ? tiles : sms);
    switch (p.mode) {
        case EPI_RAW_I32:     return launch_tc<EPI_RAW_I32>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev, grid, st);
        case EPI_REQUANT_I32: return launch_tc<EPI_REQUANT_I32>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev, grid, st);
        case EPI_DEQUANT_F32:
            if (p.n_peers > 0) return launch_tc<EPI_DEQUANT_F32, true>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev, grid, st);
            return launch_tc<EPI_DEQUANT_F32>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev, grid, st);
        case EPI_DEQUANT_I8:  return launch_tc<EPI_DEQUANT_I8>(ma, mw, mo, p, tiles_m, tiles_n, num_kb, tma_out, status_dev, grid, st);
    }
    return fail(RPLB_E_BAD_ARG, "unknown epilogue mode %d", p.mode);
}

}  // namespace rplb
