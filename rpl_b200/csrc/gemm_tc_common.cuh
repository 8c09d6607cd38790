// What the tensor-core kernels share: tile constants, the PTX wrappers (mbarrier,
// TMA, tcgen05), shared-memory and instruction descriptors, the bounded waits and
// the epilogue of one 32-column chunk.
#pragma once
#include "gemm_common.cuh"
#include <cuda.h>

namespace rplb {

constexpr int TILE_M = 128;          // rows of A per tile = TMEM lanes
constexpr int TILE_N = 256;          // rows of W per tile = accumulator columns
constexpr int TILE_K = 128;          // bytes of K per stage = one 128-byte swizzle row
constexpr int MMA_K = 32;            // K per tcgen05.mma.kind::i8
constexpr int GROUP_M = 32;          // 128-row m-tiles per rasterisation group (single-CTA kernel); measured:
                                     // 16 -> 29.5 ms, 24/32 -> 29.0 ms, 48 -> 31.8 ms, 64+ -> 33.7 ms on the large GEMM
constexpr uint32_t EPI_TILE_BYTES = 32 * 128;            // one epilogue warp's staging tile: 32 rows x 32 four-byte results
constexpr uint32_t EPI_STAGE_BYTES = 4 * EPI_TILE_BYTES;  // four epilogue warps; follows the stage ring, so it is 1024-byte aligned

// Status codes written to the status word when a wait gives up.
enum : int { TC_WAIT_EMPTY = 1, TC_WAIT_FULL = 2, TC_WAIT_ACC_EMPTY = 3, TC_WAIT_ACC_FULL = 4, TC_WAIT_ROWS = 5, TC_SMEM_BASE = 8, TC_WAIT_SELFTEST = 99 };

// --------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity.  Gives up after about a second
// (or as soon as another role has given up) and returns false.
constexpr long long kWaitLimitCycles = 2000000000LL;
// Rows from another GPU: half of that, so that this wait is the one that runs out
// (and names the cause) before the roles waiting further down the pipeline do.
constexpr long long kRowWaitLimitCycles = kWaitLimitCycles / 2;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                                  long long limit = kWaitLimitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until a 128-row block of A sent by another GPU is in place: its arrival
// word must have reached the call's epoch (compared modulo 2^32).  Bounded like
// the mbarrier waits; on success the TMA unit is fenced so that its loads see
// what the acquire saw.
__device__ __forceinline__ bool wait_rows_ready(const uint32_t* word, uint32_t epoch, volatile int* abort_flag, int* status) {
    if ((int32_t)(ld_acquire_sys(word) - epoch) < 0) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(word) - epoch) < 0) {
            __nanosleep(100);
            if ((++spins & 63u) == 0) {
                if (*abort_flag) return false;
                if (clock64() - t0 > kRowWaitLimitCycles) {
                    *abort_flag = 1;
                    atomicCAS(status, 0, (int)TC_WAIT_ROWS);
                    return false;
                }
            }
        }
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Store of a shared-memory tile through a tensor map (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Every bulk store of this thread has finished reading its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Every bulk store of this thread is complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Makes this thread's shared-memory writes visible to the TMA unit.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (base lane + i), registers 0..31 = columns.
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// stored with the 128-byte swizzle in 1024-byte atoms of 8 rows:
//   bits  0-13  start address >> 4
//   bits 16-29  leading byte offset >> 4 (not used by swizzled K-major layouts; 1)
//   bits 32-45  stride byte offset >> 4  = 1024 >> 4 (distance between 8-row groups)
//   bits 46-47  descriptor version = 1
//   bits 61-63  layout = 2 (128-byte swizzle)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Descriptor of an MN-major operand tile (rows of the stage are K, the 128 bytes of
// a row are 128 consecutive N) with the 128-byte swizzle: atoms of 8 K-rows x 128
// bytes; leading byte offset = distance between 128-wide N blocks, stride byte
// offset = distance between groups of 8 K-rows (1024 bytes).
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t n_block_stride_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((n_block_stride_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: dense, no saturation, int32 accumulator (2 << 4),
// A and B signed int8 (1 << 7, 1 << 10), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24.
constexpr uint32_t kIdescI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
constexpr uint32_t kIdescI8BMn = kIdescI8 | (1u << 16);      // B operand MN-major: gemm_int8's B[K,N] as it lies in memory

// A named barrier over `threads` threads with a vote: true only if every participant passed true.  Used after a
// bounded wait by warps that go on to meet at barriers, so that they all take the same decision (one that gave up
// while another just got through would otherwise leave its partners waiting for ever).
__device__ __forceinline__ bool named_barrier_all(uint32_t barrier_id, uint32_t threads, bool mine) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.and.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out) : "r"(barrier_id), "r"(threads), "r"(mine ? 1u : 0u) : "memory");
    return out != 0;
}
__device__ __forceinline__ void named_barrier(uint32_t barrier_id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(threads) : "memory");
}

// Tile index -> (m-tile, n-tile): tiles are numbered so that CTAs running at the
// same time cover GROUP_M consecutive m-tiles of a few n-tiles, which keeps the
// set of A and W rows being streamed small enough to be served from L2.
// `rotate` shifts the m-tile numbering (modulo tiles_m) so that the walk starts at
// that m-tile: used when the first rows of A in place are not rows 0...
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t& tm, uint32_t& tn,
                                            uint32_t group_m = GROUP_M, uint32_t rotate = 0) {
    const uint32_t per_group = group_m * tiles_n;
    const uint32_t group = tile / per_group;
    const uint32_t first_m = group * group_m;
    const uint32_t rows = min(group_m, tiles_m - first_m);
    const uint32_t in_group = tile - group * per_group;
    tm = first_m + in_group % rows + rotate;
    if (tm >= tiles_m) tm -= tiles_m;
    tn = in_group / rows;
}

// --------------------------------------------------------------------------- epilogue of one 32-column chunk
// A warp's staging tile holds 32 rows of 128 bytes with the 128-byte swizzle the
// tensor map of the output expects: the 16-byte piece j of row r lies at piece
// j ^ (r & 7).  Lane = row, so the eight lanes of a quarter warp write eight
// different pieces: no bank conflicts.
__device__ __forceinline__ void stage_row_swizzled(uint8_t* tile, int row, const uint32_t (&w)[32]) {
    #pragma unroll
    for (int j = 0; j < 8; j++)
        *reinterpret_cast<uint4*>(tile + row * 128 + ((j ^ (row & 7)) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// The staged fp32 chunk once more, for the other ranks' buffers.  Read back with
// lanes along the columns, so that each instruction writes four rows of 128
// contiguous bytes: over NVLink a 16-byte piece per row would travel as a packet
// of its own.  All 32 lanes take part (rows beyond M are read but not stored).
__device__ __forceinline__ void store_tile_to_peers(const GemmProblem& p, const uint8_t* tile, uint64_t m_base,
                                                    uint64_t n_first, int lane) {
    const uint64_t n_left = p.N - n_first;
    const int sub = lane >> 3, j = lane & 7, c4 = j * 4;         // four rows per instruction, eight lanes per row
    for (int d = 0; d < p.n_peers; d++) {
        float* base = p.peer_out[d] + n_first + c4;
        #pragma unroll
        for (int it = 0; it < 8; it++) {
            const int row = it * 4 + sub;
            const uint64_t mm = m_base + (uint64_t)row;
            if (mm >= p.M) continue;
            const float4 q = *reinterpret_cast<const float4*>(tile + row * 128 + ((j ^ (row & 7)) << 4));
            float* dst = base + mm * p.ldo;
            if ((uint64_t)(c4 + 3) < n_left && (((uintptr_t)dst & 15) == 0)) {
                *reinterpret_cast<float4*>(dst) = q;
            } else {
                if ((uint64_t)c4 < n_left) dst[0] = q.x;
                if ((uint64_t)(c4 + 1) < n_left) dst[1] = q.y;
                if ((uint64_t)(c4 + 2) < n_left) dst[2] = q.z;
                if ((uint64_t)(c4 + 3) < n_left) dst[3] = q.w;
            }
        }
    }
}

// Lane = one output row (m_base + lane); r[0..31] = accumulators of columns
// n_first..n_first+31.  s_scales / s_aux: this warp's shared-memory copies of the
// per-column values of the chunk (weight scales and bias for the fp32 modes;
// s_aux holds the column sums, as int32 bit patterns, when gemm_int8 runs with
// zero points).  tile: this warp's staging tile; tma_out: the four-byte results
// leave through map_out (whole warp takes part), otherwise each lane stores its row.
template <int MODE, bool PEERS>
__device__ __forceinline__ void epilogue_chunk(const GemmProblem& p, const CUtensorMap* map_out, bool tma_out, uint8_t* tile,
                                               const uint32_t (&r)[32], uint64_t m_base, int lane, uint64_t n_first,
                                               float a_scale, const float* s_scales, const float* s_aux,
                                               const QuantConsts& oq, int32_t row_sum, float& absmax) {
    const uint64_t m = m_base + (uint64_t)lane;
    const bool row_ok = m < p.M;
    const uint64_t n_left = p.N - n_first;          // caller guarantees n_first < N
    const bool full = n_left >= 32;
    uint32_t w[32];                                  // the row's 32 results as bit patterns
    if (MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) {
        const bool has_bias = p.bias_f32 != nullptr;
        const bool relu = p.relu != 0;
        float v[32];
        #pragma unroll
        for (int c = 0; c < 32; c++) v[c] = dequant_f32((int32_t)r[c], a_scale, s_scales[c], has_bias, s_aux[c], relu);
        if (p.absmax_out && row_ok) {
            #pragma unroll
            for (int c = 0; c < 32; c++)
                if (full || (uint64_t)c < n_left) absmax_fold(absmax, v[c]);
        }
        if (MODE == EPI_DEQUANT_I8) {
            if (!row_ok) return;
            int8_t* row = static_cast<int8_t*>(p.out) + m * p.ldo + n_first;
            uint32_t q[8];
            #pragma unroll
            for (int c = 0; c < 8; c++) q[c] = quantize_quad_packed(make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]), oq);
            if (full && (((uintptr_t)row & 15) == 0)) {
                __stcs(reinterpret_cast<uint4*>(row), make_uint4(q[0], q[1], q[2], q[3]));
                __stcs(reinterpret_cast<uint4*>(row + 16), make_uint4(q[4], q[5], q[6], q[7]));
            } else {
                #pragma unroll
                for (int c = 0; c < 32; c++)
                    if ((uint64_t)c < n_left) row[c] = (int8_t)((q[c >> 2] >> (8 * (c & 3))) & 0xff);
            }
            return;
        }
        #pragma unroll
        for (int c = 0; c < 32; c++) w[c] = __float_as_uint(v[c]);
    } else {
        #pragma unroll
        for (int c = 0; c < 32; c++) {
            int32_t s = (int32_t)r[c];
            if (MODE == EPI_RAW_I32) {
                if (p.bias_i8 && (uint64_t)c < n_left) s = (int32_t)((uint32_t)s + (uint32_t)(int32_t)__ldg(p.bias_i8 + n_first + c));
            } else {
                if (p.a_row_sums) s = apply_zero_points(s, row_sum, __float_as_int(s_aux[c]), p.za, p.zb, (uint32_t)p.K);
                s = requant_i32(s, p.sa, p.sb, p.sc);
            }
            w[c] = (uint32_t)s;
        }
    }
    // A tensor store clips at the map's edge in whole 16-byte pieces, not in elements (measured: with N % 4 != 0 the
    // piece that straddles the edge was written in full, up to three columns beyond the block), so the chunk that
    // holds a ragged edge leaves from registers, element by element.
    const bool by_tma = tma_out && (full || (n_left & 3) == 0);
    if (by_tma) {
        if (lane == 0) bulk_wait_read_all();         // the previous chunk has left the tile
        __syncwarp();
        stage_row_swizzled(tile, lane, w);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_out, tile, (int32_t)n_first, (int32_t)m_base);
            bulk_commit();
        }
    } else {
        if (row_ok) {
            uint32_t* row = static_cast<uint32_t*>(p.out) + m * p.ldo + n_first;
            if (full && (((uintptr_t)row & 15) == 0)) {
                #pragma unroll
                for (int c = 0; c < 32; c += 4) __stcs(reinterpret_cast<uint4*>(row + c), make_uint4(w[c], w[c + 1], w[c + 2], w[c + 3]));
            } else {
                #pragma unroll
                for (int c = 0; c < 32; c++)
                    if ((uint64_t)c < n_left) row[c] = w[c];
            }
        }
        if (PEERS) {
            if (tma_out && lane == 0) bulk_wait_read_all();      // a tensor store of an earlier chunk may still read the tile
            __syncwarp();                            // the previous chunk has been read out of the tile
            stage_row_swizzled(tile, lane, w);
            __syncwarp();
        }
    }
    if (PEERS) store_tile_to_peers(p, tile, m_base, n_first, lane);
}

// Per-tile staging of the per-column epilogue inputs into this warp's shared-memory slots.
template <int MODE>
__device__ __forceinline__ void stage_columns(const GemmProblem& p, uint64_t n0, int lane, float* s_scales, float* s_aux) {
    // All loads are issued before the first store, so the warp (alone on its
    // scheduler) waits for global memory once, not once per 32 columns.
    if (MODE == EPI_DEQUANT_F32 || MODE == EPI_DEQUANT_I8) {
        float sc[TILE_N / 32], bi[TILE_N / 32];
        #pragma unroll
        for (int j = 0; j < TILE_N / 32; j++) {
            const uint64_t n = n0 + (uint64_t)(lane + 32 * j);
            sc[j] = n < p.N ? __ldg(p.w_scales + n) : 0.0f;
            bi[j] = (p.bias_f32 && n < p.N) ? __ldg(p.bias_f32 + n) : 0.0f;
        }
        __syncwarp();
        #pragma unroll
        for (int j = 0; j < TILE_N / 32; j++) {
            s_scales[lane + 32 * j] = sc[j];
            s_aux[lane + 32 * j] = bi[j];
        }
        __syncwarp();
    } else if (MODE == EPI_REQUANT_I32) {
        if (p.b_col_sums) {
            int32_t cs[TILE_N / 32];
            #pragma unroll
            for (int j = 0; j < TILE_N / 32; j++) {
                const uint64_t n = n0 + (uint64_t)(lane + 32 * j);
                cs[j] = n < p.N ? __ldg(p.b_col_sums + n) : 0;
            }
            __syncwarp();
            #pragma unroll
            for (int j = 0; j < TILE_N / 32; j++) s_aux[lane + 32 * j] = __int_as_float(cs[j]);
            __syncwarp();
        }
    }
}

// Host side, implemented in gemm_i8_tcgen05.cu: a (cached) 2-D tensor map of a row-major matrix with the
// 128-byte swizzle (elem = 1: int8 operand, 4: four-byte values; 5: four-byte values without swizzle), and the calling thread's status word
// as the device sees it (nullptr when it cannot be allocated).
int make_map_2d(CUtensorMap* map, const void* base, int elem, uint64_t dim0, uint64_t dim1, uint64_t stride_bytes,
                uint32_t box0, uint32_t box1, const char* what);
int* kernel_status_word_device();
int gemm_tcgen05_status(bool clear);

}  // namespace rplb
