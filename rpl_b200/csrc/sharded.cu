// A quantized Linear layer spread over the GPUs of one node, one process per
// GPU, driven from C: the multi-GPU form of linear_int8 (src/rpl_quantization.c:
// 314-353) behind tensor_quantize_int8_symmetric (src/rpl_quantization.c:77-91).
//
// The output columns (rows of the [N,K] weight) are split over the ranks, and so
// are the rows of the fp32 activation: rank r holds rows [r0, r0 + rc) of x.
// One forward pass on every rank:
//
//   1. min/max of the local rows (minmax_kernel), one max-all-reduce of the pair
//      (-min, max) over NCCL, and the scale from the combined pair by the same
//      statements as on one GPU: every rank ends up with the scale a single GPU
//      would compute for the whole tensor.
//   2. quantize the local rows into this rank's copy of the int8 activation.
//   3. send those int8 rows to every other rank: one peer copy per destination
//      over NVLink on a side stream (the copy engines, so no SM is taken from
//      the GEMM), nearest consumer first, each followed by a small copy that
//      sets the arrival words of the 128-row blocks just delivered.
//   4. the tensor-core GEMM over ALL rows against this rank's weight rows,
//      started at once: it begins with the local rows and, before loading any
//      other 128-row block, its TMA producer waits (bounded) for that block's
//      arrival word.  The transfer of step 3 runs underneath the GEMM.
//
// The max-all-reduce of step 1 doubles as the fence between passes: a rank can
// pass it only after every rank has entered it, i.e. after every rank's previous
// GEMM has finished reading its copy of the activation, so the copies of step 3
// never overwrite rows that are still being read.
//
// NCCL is loaded at run time (dlopen): a program that only ever runs on one GPU
// needs no NCCL library.
#include "gemm_common.cuh"
#include <dlfcn.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

extern "C" {
int rplb_minmax_f32(const float* x, uint64_t n, rplb_qparams* params, void* stream);
int rplb_quantize_f32_i8_dev(const float* x, int8_t* q, uint64_t n, const float* scale_dev, const int32_t* zp_dev, void* stream);
int rplb_qparams_to_pair(const rplb_qparams* params, float* pair, void* stream);
int rplb_qparams_from_pair(const float* pair, rplb_qparams* params, void* stream);
int rplb_shard_range(uint64_t n, int world, int rank, uint64_t align, uint64_t* begin, uint64_t* count);
int rplb_kernel_status(int clear);
}

namespace rplb {

// --------------------------------------------------------------------------- NCCL, loaded at run time
// The few declarations needed; the ABI of these has been stable across NCCL 2.x.
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[RPLB_NCCL_ID_BYTES]; } ncclUniqueId;
enum { kNcclInt8 = 0, kNcclFloat32 = 7 };
enum { kNcclSum = 0, kNcclMax = 2 };

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    char error[256] = "";
};

static NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // RPLB_NCCL_LIBRARY names a specific file; otherwise the usual sonames.
        const char* names[3] = {getenv("RPLB_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
        for (int i = names[0] ? 0 : 1; i < (names[0] ? 1 : 3) && !api.lib; i++) {
            api.lib = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
            if (!api.lib) snprintf(api.error, sizeof(api.error), "cannot load %s: %s", names[i], dlerror());
        }
        if (!api.lib) return;
        bool ok = true;
        auto sym = [&](const char* n) { void* s = dlsym(api.lib, n); if (!s) { ok = false; snprintf(api.error, sizeof(api.error), "%s missing from the NCCL library", n); } return s; };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        if (!ok) { dlclose(api.lib); api.lib = nullptr; }
    });
    return &api;
}

static int nccl_ok(int r, const char* what) {
    if (r == 0) return 0;
    NcclApi* n = nccl_api();
    return fail(RPLB_E_COMM, "%s: %s", what, (n->lib && n->GetErrorString) ? n->GetErrorString(r) : "NCCL error");
}

// --------------------------------------------------------------------------- small kernels
__global__ void fill_u32_kernel(uint32_t* dst, uint32_t value, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value;
}

// The other way to send the rows: quantize this rank's fp32 rows once more and store the packed int8 straight into
// the other ranks' activation buffers (plain 16-byte stores over NVLink, 512 contiguous bytes per warp), then set the
// arrival word of each 128-row block in every destination.  One CTA per 128-row block; the block's word is written
// after a CTA-wide barrier and a system-scope fence, so it cannot overtake the rows.  Kept beside the copy-engine
// route for comparison (rplb_sharded_linear_transfer): it costs SM time and a second read of the rows, the copy
// engines cost neither.
struct PeerRows {
    int8_t* xq[7];
    uint32_t* words[7];
    int n;
};

__global__ void __launch_bounds__(512)
quantize_rows_to_peers_kernel(const float* __restrict__ x, uint64_t rows, uint64_t K, uint64_t row0, const float* __restrict__ scale,
                              PeerRows peers, uint32_t epoch) {
    const QuantConsts qc = make_quant_consts(__ldg(scale), 0);
    const uint64_t first = (uint64_t)blockIdx.x * 128, last = first + 128 < rows ? first + 128 : rows;
    const uint64_t pieces = (last - first) * K / 16;                          // 16 int8 = four quads per piece (K % 16 == 0)
    const float4* src = reinterpret_cast<const float4*>(x + first * K);
    for (uint64_t i = threadIdx.x; i < pieces; i += blockDim.x) {
        const float4 a = __ldcs(src + 4 * i), b = __ldcs(src + 4 * i + 1), c = __ldcs(src + 4 * i + 2), d = __ldcs(src + 4 * i + 3);
        const uint4 w = make_uint4(quantize_quad_packed(a, qc), quantize_quad_packed(b, qc), quantize_quad_packed(c, qc), quantize_quad_packed(d, qc));
        const uint64_t at = (row0 + first) * K + 16 * i;
        for (int p = 0; p < peers.n; p++) *reinterpret_cast<uint4*>(peers.xq[p] + at) = w;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint64_t block = (row0 + first) / 128;
        for (int p = 0; p < peers.n; p++) *reinterpret_cast<volatile uint32_t*>(peers.words[p] + block) = epoch;
    }
}

// Where each rank's column block begins (entry `world` = the total): passed to kernels by value.
struct ColumnSplit {
    uint64_t begin[9];
};

// landing[r][m][0..cmax) -> full[m][begin_r .. begin_r + count_r).  VEC = 4: four columns (16 bytes) per thread
// and step, for splits and widths that are multiples of four columns and 16-byte aligned buffers; VEC = 1 otherwise.
template <int VEC>
__global__ void unpack_columns_kernel(const float* __restrict__ landing, float* __restrict__ full, uint64_t M, uint64_t n_total,
                                      uint64_t cmax, int world, ColumnSplit split) {
    const uint64_t per_row = n_total / VEC;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * per_row; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t m = i / per_row, n = (i % per_row) * VEC;
        int r = 0;
        while (r + 1 < world && n >= split.begin[r + 1]) r++;           // owner of column n
        const float* src = landing + ((uint64_t)r * M + m) * cmax + (n - split.begin[r]);
        float* dst = full + m * n_total + n;
        if (VEC == 4) *reinterpret_cast<float4*>(dst) = __ldcs(reinterpret_cast<const float4*>(src));
        else *dst = *src;
    }
}

__global__ void pack_columns_kernel(const float* __restrict__ block, uint64_t ld, float* __restrict__ packed, uint64_t M,
                                    uint64_t count, uint64_t cmax) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * cmax; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t m = i / cmax, c = i % cmax;
        packed[i] = c < count ? block[m * ld + c] : 0.0f;
    }
}

// --------------------------------------------------------------------------- the layer
constexpr int kMaxWorld = 8;
constexpr int kDepth = 2;            // calls in flight in the host-buffer pipeline
constexpr int kMaxBlocks = 16;       // row blocks of one host-buffer call

struct ShardedLinear {
    int rank = 0, world = 1;
    uint64_t max_rows = 0, K = 0, n_total = 0, col_begin = 0, col_count = 0;
    ColumnSplit split = {};              // every rank's first column; split.begin[world] = n_total
    const int8_t* w = nullptr;
    const float* w_scales = nullptr;
    const float* bias = nullptr;
    ncclComm_t comm = nullptr;
    bool owns_comm = false;
    // One device block per rank, shared with the other ranks: [arrival words | int8 activation].
    uint8_t* block = nullptr;
    size_t words_bytes = 0;
    uint8_t* peer_block[kMaxWorld] = {};     // the same block of every other rank, mapped into this process
    uint32_t* epoch_words = nullptr;         // source of the copies that set a peer's arrival words
    rplb_qparams* params = nullptr;
    float* pair = nullptr;
    uint32_t epoch = 0;
    cudaStream_t s_push = nullptr;
    cudaEvent_t ev_quantized = nullptr, ev_pushed = nullptr;
    bool pushed = false;
    int transfer = 0;                        // 0 = peer copies by the copy engines, 1 = stores from a quantize kernel
    // gather
    float* landing = nullptr;
    size_t landing_bytes = 0;
    // host-buffer pipeline
    cudaStream_t s_main = nullptr, s_in = nullptr, s_out = nullptr;
    bool owns_main = false;
    float* din[kDepth] = {};
    float* dout[kDepth] = {};
    size_t din_bytes[kDepth] = {}, dout_bytes[kDepth] = {};
    cudaEvent_t ev_uploaded[kDepth] = {}, ev_computed[kDepth] = {}, ev_downloaded[kDepth] = {};
    cudaEvent_t ev_block[kDepth][kMaxBlocks] = {};
    bool slot_used[kDepth] = {};
    uint64_t calls = 0;
    bool complete = false;           // set-up finished on every rank: tearing down is then a collective step

    uint32_t* words() const { return reinterpret_cast<uint32_t*>(block); }
    int8_t* xq() const { return reinterpret_cast<int8_t*>(block + words_bytes); }
    uint32_t* peer_words(int r) const { return reinterpret_cast<uint32_t*>(peer_block[r]); }
    int8_t* peer_xq(int r) const { return reinterpret_cast<int8_t*>(peer_block[r] + words_bytes); }
};

static int stream_fence(ShardedLinear* h, cudaStream_t st);

static void destroy(ShardedLinear* h) {
    if (!h) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < kMaxWorld; r++)
        if (h->peer_block[r] && r != h->rank) cudaIpcCloseMemHandle(h->peer_block[r]);
    // A block may be freed only after every other rank has unmapped it.
    if (h->complete && h->world > 1 && stream_fence(h, nullptr) == 0) cudaStreamSynchronize(nullptr);
    if (h->comm && h->owns_comm && nccl_api()->lib) nccl_api()->CommDestroy(h->comm);
    device_free(h->block);
    device_free(h->epoch_words);
    device_free(h->params);
    device_free(h->landing);
    for (int i = 0; i < kDepth; i++) {
        device_free(h->din[i]);
        device_free(h->dout[i]);
        if (h->ev_uploaded[i]) cudaEventDestroy(h->ev_uploaded[i]);
        if (h->ev_computed[i]) cudaEventDestroy(h->ev_computed[i]);
        if (h->ev_downloaded[i]) cudaEventDestroy(h->ev_downloaded[i]);
        for (int b = 0; b < kMaxBlocks; b++)
            if (h->ev_block[i][b]) cudaEventDestroy(h->ev_block[i][b]);
    }
    if (h->ev_quantized) cudaEventDestroy(h->ev_quantized);
    if (h->ev_pushed) cudaEventDestroy(h->ev_pushed);
    if (h->s_push) cudaStreamDestroy(h->s_push);
    if (h->s_in) cudaStreamDestroy(h->s_in);
    if (h->s_out) cudaStreamDestroy(h->s_out);
    if (h->s_main && h->owns_main) cudaStreamDestroy(h->s_main);
    cudaGetLastError();
    delete h;
}

// One max-all-reduce of a word: every rank has reached this point of its stream.
static int stream_fence(ShardedLinear* h, cudaStream_t st) {
    if (h->world == 1) return 0;
    return nccl_ok(nccl_api()->AllReduce(h->pair + 2, h->pair + 2, 1, kNcclFloat32, kNcclMax, h->comm, st), "ncclAllReduce(fence)");
}

static int create(ShardedLinear** out, int rank, int world, const void* nccl_id, void* nccl_comm, uint64_t max_rows,
                  uint64_t K, uint64_t n_total, const uint64_t* column_counts, const int8_t* w, const float* w_scales,
                  const float* bias) {
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
        return fail(RPLB_E_BAD_ARG, "sharded linear: rank %d of %d (at most %d ranks)", rank, world, kMaxWorld);
    if (max_rows == 0 || K == 0 || n_total == 0) return fail(RPLB_E_BAD_ARG, "sharded linear: empty shape");
    if (world > 1 && K % 16 != 0)
        return fail(RPLB_E_UNSUPPORTED, "sharded linear over several GPUs needs in_features %% 16 == 0 (tensor-core kernel)");
    if (world > 1 && !nccl_id && !nccl_comm) return fail(RPLB_E_BAD_ARG, "sharded linear: neither an NCCL id nor a communicator given");
    if (world > 1) {
        NcclApi* n = nccl_api();
        if (!n->lib) return fail(RPLB_E_COMM, "sharded linear: %s", n->error);
    }
    ShardedLinear* h = new ShardedLinear();
    h->rank = rank; h->world = world; h->max_rows = max_rows; h->K = K; h->n_total = n_total;
    h->w = w; h->w_scales = w_scales; h->bias = bias;
    // The column blocks: dealt evenly, or as the caller says (e.g. in proportion to each GPU's measured speed).
    uint64_t at = 0;
    for (int r = 0; r < world; r++) {
        uint64_t b = 0, c = 0;
        if (column_counts) { b = at; c = column_counts[r]; }
        else rplb_shard_range(n_total, world, r, 256, &b, &c);
        if (b != at || (c % 256 != 0 && at + c != n_total) || at + c > n_total) {
            delete h;
            return fail(RPLB_E_BAD_ARG, "sharded linear: column blocks must be contiguous multiples of 256 (the last may be ragged) that add up to %llu",
                        (unsigned long long)n_total);
        }
        h->split.begin[r] = b;
        at += c;
    }
    if (at != n_total) { delete h; return fail(RPLB_E_BAD_ARG, "sharded linear: the column blocks cover %llu of %llu columns",
                                               (unsigned long long)at, (unsigned long long)n_total); }
    h->split.begin[world] = n_total;
    h->col_begin = h->split.begin[rank];
    h->col_count = h->split.begin[rank + 1] - h->split.begin[rank];
    if (h->col_count && (!w || !w_scales)) { delete h; return fail(RPLB_E_BAD_ARG, "sharded linear: null weight or scale pointer"); }
    const uint64_t max_tiles = (max_rows + 127) / 128;
    h->words_bytes = (size_t)((max_tiles * 4 + 4095) & ~(uint64_t)4095);
    int rc = 0;
    void* p = nullptr;
    if (!rc) { rc = device_alloc(&p, h->words_bytes + (size_t)max_rows * K, "sharded linear: activation block"); h->block = (uint8_t*)p; }
    if (!rc) rc = cuda_ok(cudaMemset(h->block, 0, h->words_bytes), "cudaMemset(arrival words)");
    if (!rc) { rc = device_alloc(&p, (size_t)max_tiles * 4, "sharded linear: epoch words"); h->epoch_words = (uint32_t*)p; }
    if (!rc) { rc = device_alloc(&p, 256, "sharded linear: parameters"); h->params = (rplb_qparams*)p; }
    if (!rc) rc = cuda_ok(cudaMemset(h->params, 0, 256), "cudaMemset(parameters)");
    if (!rc) h->pair = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(h->params) + 64);
    if (!rc) rc = cuda_ok(cudaStreamCreateWithFlags(&h->s_push, cudaStreamNonBlocking), "cudaStreamCreate");
    if (!rc) rc = cuda_ok(cudaEventCreateWithFlags(&h->ev_quantized, cudaEventDisableTiming), "cudaEventCreate");
    if (!rc) rc = cuda_ok(cudaEventCreateWithFlags(&h->ev_pushed, cudaEventDisableTiming), "cudaEventCreate");
    h->peer_block[rank] = h->block;
    if (!rc && world > 1) {
        NcclApi* n = nccl_api();
        if (nccl_comm) {
            h->comm = static_cast<ncclComm_t>(nccl_comm);
        } else {
            ncclUniqueId id;
            memcpy(&id, nccl_id, sizeof(id));
            rc = nccl_ok(n->CommInitRank(&h->comm, world, id, rank), "ncclCommInitRank");
            h->owns_comm = rc == 0;
        }
        // Every rank's block, mapped into this process: the handles travel through the communicator itself.
        uint8_t* handles = nullptr;
        std::vector<uint8_t> host((size_t)world * RPLB_IPC_HANDLE_BYTES);
        if (!rc) { rc = device_alloc(&p, host.size(), "sharded linear: handle exchange"); handles = (uint8_t*)p; }
        cudaIpcMemHandle_t mine;
        if (!rc) rc = cuda_ok(cudaIpcGetMemHandle(&mine, h->block), "cudaIpcGetMemHandle");
        if (!rc) rc = cuda_ok(cudaMemcpy(handles + (size_t)rank * RPLB_IPC_HANDLE_BYTES, &mine, sizeof(mine), cudaMemcpyHostToDevice), "cudaMemcpy(handle)");
        if (!rc) rc = nccl_ok(n->AllGather(handles + (size_t)rank * RPLB_IPC_HANDLE_BYTES, handles, RPLB_IPC_HANDLE_BYTES, kNcclInt8, h->comm, nullptr),
                              "ncclAllGather(handles)");
        if (!rc) rc = cuda_ok(cudaMemcpy(host.data(), handles, host.size(), cudaMemcpyDeviceToHost), "cudaMemcpy(handles)");
        for (int r = 0; !rc && r < world; r++) {
            if (r == rank) continue;
            cudaIpcMemHandle_t theirs;
            memcpy(&theirs, host.data() + (size_t)r * RPLB_IPC_HANDLE_BYTES, sizeof(theirs));
            void* mapped = nullptr;
            rc = cuda_ok(cudaIpcOpenMemHandle(&mapped, theirs, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
            h->peer_block[r] = static_cast<uint8_t*>(mapped);
        }
        device_free(handles);
        if (!rc) rc = stream_fence(h, nullptr);            // nobody starts sending before everybody has mapped
        if (!rc) rc = cuda_ok(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
    }
    if (rc) { destroy(h); return rc; }
    h->complete = true;
    *out = h;
    return 0;
}

// Row block of this rank for an activation of M rows, in multiples of 128 rows (one arrival word each).
static void row_range(const ShardedLinear* h, uint64_t M, uint64_t* r0, uint64_t* rc) {
    rplb_shard_range(M, h->world, h->rank, 128, r0, rc);
}

// Steps 1-3 of a pass on stream st: the scale, the local int8 rows, and the copies to the other ranks.
static int quantize_and_send(ShardedLinear* h, const float* x_local, uint64_t M, cudaStream_t st) {
    uint64_t r0, rc;
    row_range(h, M, &r0, &rc);
    if (rc && !x_local) return fail(RPLB_E_BAD_ARG, "sharded linear: null activation");
    h->epoch++;
    // The copies of the previous pass read the local rows of the int8 activation.
    if (h->pushed) if (int e = cuda_ok(cudaStreamWaitEvent(st, h->ev_pushed, 0), "cudaStreamWaitEvent")) return e;
    if (int e = rplb_minmax_f32(x_local, rc * h->K, h->params, st)) return e;
    if (h->world > 1) {
        if (int e = rplb_qparams_to_pair(h->params, h->pair, st)) return e;
        if (int e = nccl_ok(nccl_api()->AllReduce(h->pair, h->pair, 2, kNcclFloat32, kNcclMax, h->comm, st), "ncclAllReduce(min/max)")) return e;
        if (int e = rplb_qparams_from_pair(h->pair, h->params, st)) return e;
    }
    if (rc)
        if (int e = rplb_quantize_f32_i8_dev(x_local, h->xq() + r0 * h->K, rc * h->K, &h->params->scale_sym, nullptr, st)) return e;
    if (h->world == 1) return 0;
    const uint32_t t0 = (uint32_t)(r0 / 128), nt = (uint32_t)((rc + 127) / 128);
    if (nt) {
        fill_u32_kernel<<<(nt + 255) / 256, 256, 0, st>>>(h->epoch_words + t0, h->epoch, nt);
        if (int e = launched("fill_u32_kernel")) return e;
    }
    if (int e = cuda_ok(cudaEventRecord(h->ev_quantized, st), "cudaEventRecord")) return e;
    if (int e = cuda_ok(cudaStreamWaitEvent(h->s_push, h->ev_quantized, 0), "cudaStreamWaitEvent")) return e;
    if (nt && h->transfer == 1) {
        PeerRows peers = {};
        for (int d = 1; d < h->world; d++) {
            const int peer = (h->rank - d + h->world) % h->world;
            peers.xq[peers.n] = h->peer_xq(peer);
            peers.words[peers.n] = h->peer_words(peer);
            peers.n++;
        }
        quantize_rows_to_peers_kernel<<<nt, 512, 0, h->s_push>>>(x_local, rc, h->K, r0, &h->params->scale_sym, peers, h->epoch);
        if (int e = launched("quantize_rows_to_peers_kernel")) return e;
    } else if (nt) {
        // Rank r - 1 reaches these rows first (every rank walks the blocks upwards from its own), then r - 2, ...
        for (int d = 1; d < h->world; d++) {
            const int peer = (h->rank - d + h->world) % h->world;
            if (int e = cuda_ok(cudaMemcpyAsync(h->peer_xq(peer) + r0 * h->K, h->xq() + r0 * h->K, rc * h->K, cudaMemcpyDeviceToDevice, h->s_push),
                                "cudaMemcpyAsync(rows to peer)")) return e;
            if (int e = cuda_ok(cudaMemcpyAsync(h->peer_words(peer) + t0, h->epoch_words + t0, (size_t)nt * 4, cudaMemcpyDeviceToDevice, h->s_push),
                                "cudaMemcpyAsync(arrival words)")) return e;
        }
    }
    if (int e = cuda_ok(cudaEventRecord(h->ev_pushed, h->s_push), "cudaEventRecord")) return e;
    h->pushed = true;
    return 0;
}

// Step 4 for rows [b0, b1) of the activation (b0 a multiple of 128): GEMM against this rank's weight rows.
static int gemm_rows(ShardedLinear* h, uint64_t M, uint64_t b0, uint64_t b1, float* out, uint64_t ldo, int relu, cudaStream_t st) {
    if (h->col_count == 0 || b1 <= b0) return 0;
    GemmProblem p = {};
    p.A = h->xq() + b0 * h->K; p.B = h->w; p.out = out + b0 * ldo;
    p.M = b1 - b0; p.N = h->col_count; p.K = h->K; p.ldo = ldo;
    p.b_is_kn = 0; p.mode = EPI_DEQUANT_F32;
    p.a_scale = &h->params->scale_sym; p.w_scales = h->w_scales; p.bias_f32 = h->bias; p.relu = relu;
    if (h->world == 1) return run_gemm(p, st);
    uint64_t r0, rc;
    row_range(h, M, &r0, &rc);
    const uint64_t lo = r0 > b0 ? r0 : b0, hi = (r0 + rc) < b1 ? (r0 + rc) : b1;      // local rows inside [b0, b1)
    p.a_ready = h->words() + b0 / 128;
    p.a_epoch = h->epoch;
    if (hi > lo) { p.a_local_first = (uint32_t)((lo - b0) / 128); p.a_local_count = (uint32_t)((hi - lo + 127) / 128); }
    if (!gemm_tcgen05_supports(p))
        return fail(RPLB_E_UNSUPPORTED, "sharded linear over several GPUs: the tensor-core kernel cannot take this shape or alignment");
    // The library's own choice between the two kernels that can wait for rows (256 x 256 tiles for long GEMMs,
    // 128 x 256 otherwise), unless the thread asked for one of them by name.
    const int asked = thread_gemm_backend(-1);
    return gemm_tcgen05(p, st, asked == 3 ? 1 : asked == 5 ? 3 : 0);
}

// With the kernel-store route the caller's fp32 rows are read on the side stream: the caller's stream must not run
// ahead of that read (its next work may overwrite the rows).
static int after_gemm(ShardedLinear* h, cudaStream_t st) {
    if (h->world > 1 && h->transfer == 1 && h->pushed) return cuda_ok(cudaStreamWaitEvent(st, h->ev_pushed, 0), "cudaStreamWaitEvent");
    return 0;
}

static int check_call(const ShardedLinear* h, uint64_t M, const void* out, uint64_t ldo) {
    if (!h) return fail(RPLB_E_BAD_ARG, "sharded linear: null handle");
    if (M == 0 || M > h->max_rows) return fail(RPLB_E_TOO_LARGE, "sharded linear: %llu rows (the layer was created for at most %llu)",
                                               (unsigned long long)M, (unsigned long long)h->max_rows);
    if (h->col_count && !out) return fail(RPLB_E_BAD_ARG, "sharded linear: null output");
    if (ldo < h->col_count) return fail(RPLB_E_BAD_ARG, "sharded linear: output row stride %llu < %llu columns",
                                        (unsigned long long)ldo, (unsigned long long)h->col_count);
    return 0;
}

// --------------------------------------------------------------------------- host-buffer pipeline
static int pipeline_ready(ShardedLinear* h, cudaStream_t compute) {
    if (h->s_in) {
        if (compute && compute != h->s_main) {
            if (int e = cuda_ok(cudaStreamSynchronize(h->s_main), "cudaStreamSynchronize")) return e;
            if (h->owns_main) cudaStreamDestroy(h->s_main);
            h->s_main = compute;
            h->owns_main = false;
        }
        return 0;
    }
    if (compute) { h->s_main = compute; h->owns_main = false; }
    else { if (int e = cuda_ok(cudaStreamCreateWithFlags(&h->s_main, cudaStreamNonBlocking), "cudaStreamCreate")) return e; h->owns_main = true; }
    if (int e = cuda_ok(cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking), "cudaStreamCreate")) return e;
    if (int e = cuda_ok(cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking), "cudaStreamCreate")) return e;
    for (int i = 0; i < kDepth; i++) {
        if (int e = cuda_ok(cudaEventCreateWithFlags(&h->ev_uploaded[i], cudaEventDisableTiming), "cudaEventCreate")) return e;
        if (int e = cuda_ok(cudaEventCreateWithFlags(&h->ev_computed[i], cudaEventDisableTiming), "cudaEventCreate")) return e;
        if (int e = cuda_ok(cudaEventCreateWithFlags(&h->ev_downloaded[i], cudaEventDisableTiming), "cudaEventCreate")) return e;
        for (int b = 0; b < kMaxBlocks; b++)
            if (int e = cuda_ok(cudaEventCreateWithFlags(&h->ev_block[i][b], cudaEventDisableTiming), "cudaEventCreate")) return e;
    }
    return 0;
}

static int grow(float** p, size_t* have, size_t want, const char* what) {
    if (*have >= want) return 0;
    device_free(*p);
    *p = nullptr;
    *have = 0;
    void* q = nullptr;
    if (int e = device_alloc(&q, want, what)) return e;
    *p = static_cast<float*>(q);
    *have = want;
    return 0;
}

}  // namespace rplb

using namespace rplb;

extern "C" {

int rplb_nccl_unique_id(void* id) {
    if (!id) return fail(RPLB_E_BAD_ARG, "rplb_nccl_unique_id: null pointer");
    NcclApi* n = nccl_api();
    if (!n->lib) return fail(RPLB_E_COMM, "rplb_nccl_unique_id: %s", n->error);
    ncclUniqueId u;
    if (int e = nccl_ok(n->GetUniqueId(&u), "ncclGetUniqueId")) return e;
    memcpy(id, &u, sizeof(u));
    return 0;
}

int rplb_sharded_linear_create_split(rplb_sharded_linear** layer, int rank, int world, const void* nccl_id, void* nccl_comm,
                                     uint64_t max_rows, uint64_t in_features, uint64_t out_features_total,
                                     const uint64_t* column_counts, const int8_t* weight_rows, const float* scales,
                                     const float* bias) {
    if (!layer) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_create: null result pointer");
    ShardedLinear* h = nullptr;
    const int rc = create(&h, rank, world, nccl_id, nccl_comm, max_rows, in_features, out_features_total, column_counts,
                          weight_rows, scales, bias);
    *layer = reinterpret_cast<rplb_sharded_linear*>(h);
    return rc;
}

int rplb_sharded_linear_create(rplb_sharded_linear** layer, int rank, int world, const void* nccl_id, void* nccl_comm,
                               uint64_t max_rows, uint64_t in_features, uint64_t out_features_total,
                               const int8_t* weight_rows, const float* scales, const float* bias) {
    return rplb_sharded_linear_create_split(layer, rank, world, nccl_id, nccl_comm, max_rows, in_features, out_features_total,
                                            nullptr, weight_rows, scales, bias);
}

int rplb_shard_weighted(uint64_t n, int world, uint64_t align, const double* weights, uint64_t* counts) {
    if (world <= 0 || world > kMaxWorld || !weights || !counts) return fail(RPLB_E_BAD_ARG, "rplb_shard_weighted: bad arguments");
    if (align == 0) align = 1;
    double total = 0.0;
    for (int r = 0; r < world; r++) {
        if (!(weights[r] > 0.0) || weights[r] > 1e300) return fail(RPLB_E_BAD_ARG, "rplb_shard_weighted: weight %d is not a positive number", r);
        total += weights[r];
    }
    // Whole units of `align` columns by largest remainder; ties go to the lower rank.  The last unit may be ragged.
    const uint64_t units = (n + align - 1) / align;
    uint64_t given = 0, share[kMaxWorld];
    double rest[kMaxWorld];
    for (int r = 0; r < world; r++) {
        const double exact = (double)units * (weights[r] / total);
        share[r] = (uint64_t)exact;
        rest[r] = exact - (double)share[r];
        given += share[r];
    }
    while (given < units) {
        int best = 0;
        for (int r = 1; r < world; r++) if (rest[r] > rest[best]) best = r;
        share[best]++;
        rest[best] = -1.0;
        given++;
    }
    uint64_t at = 0;
    for (int r = 0; r < world; r++) {
        uint64_t e = at + share[r] * align;
        if (e > n) e = n;
        counts[r] = e - at;
        at = e;
    }
    return 0;
}

void rplb_sharded_linear_free(rplb_sharded_linear* layer) { destroy(reinterpret_cast<ShardedLinear*>(layer)); }

int rplb_sharded_linear_columns(const rplb_sharded_linear* layer, uint64_t* begin, uint64_t* count) {
    const ShardedLinear* h = reinterpret_cast<const ShardedLinear*>(layer);
    if (!h || !begin || !count) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_columns: null pointer");
    *begin = h->col_begin;
    *count = h->col_count;
    return 0;
}

int rplb_sharded_linear_rows(const rplb_sharded_linear* layer, uint64_t rows, uint64_t* begin, uint64_t* count) {
    const ShardedLinear* h = reinterpret_cast<const ShardedLinear*>(layer);
    if (!h || !begin || !count) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_rows: null pointer");
    row_range(h, rows, begin, count);
    return 0;
}

int rplb_sharded_linear_forward(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, float* out, uint64_t ldo,
                                int relu, void* stream) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (int e = check_call(h, rows, out, ldo)) return e;
    cudaStream_t st = as_stream(stream);
    if (int e = quantize_and_send(h, x_local, rows, st)) return e;
    if (int e = gemm_rows(h, rows, 0, rows, out, ldo, relu, st)) return e;
    return after_gemm(h, st);
}

int rplb_sharded_linear_quantize(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, void* stream) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (!h) return fail(RPLB_E_BAD_ARG, "sharded linear: null handle");
    if (rows == 0 || rows > h->max_rows) return fail(RPLB_E_TOO_LARGE, "sharded linear: %llu rows (the layer was created for at most %llu)",
                                                     (unsigned long long)rows, (unsigned long long)h->max_rows);
    return quantize_and_send(h, x_local, rows, as_stream(stream));
}

int rplb_sharded_linear_gemm(rplb_sharded_linear* layer, uint64_t rows, float* out, uint64_t ldo, int relu, void* stream) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (int e = check_call(h, rows, out, ldo)) return e;
    if (int e = gemm_rows(h, rows, 0, rows, out, ldo, relu, as_stream(stream))) return e;
    return after_gemm(h, as_stream(stream));
}

int rplb_sharded_linear_transfer(rplb_sharded_linear* layer, int which) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (!h) return fail(RPLB_E_BAD_ARG, "sharded linear: null handle");
    if (which != 0 && which != 1) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_transfer: 0 (copy engines) or 1 (stores from a kernel)");
    if (which == 1 && h->K % 16 != 0) return fail(RPLB_E_UNSUPPORTED, "stores from a kernel need in_features %% 16 == 0");
    h->transfer = which;
    return 0;
}

int rplb_sharded_linear_activation(const rplb_sharded_linear* layer, const int8_t** xq, const float** scale) {
    const ShardedLinear* h = reinterpret_cast<const ShardedLinear*>(layer);
    if (!h) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_activation: null handle");
    if (xq) *xq = h->xq();
    if (scale) *scale = &h->params->scale_sym;
    return 0;
}

int rplb_sharded_linear_gather(rplb_sharded_linear* layer, const float* block, uint64_t ld, uint64_t rows, float* full, void* stream) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (!h || !full || (h->col_count && !block)) return fail(RPLB_E_BAD_ARG, "rplb_sharded_linear_gather: null pointer");
    cudaStream_t st = as_stream(stream);
    if (h->world == 1) {
        return cuda_ok(cudaMemcpy2DAsync(full, h->n_total * 4, block, ld * 4, h->col_count * 4, rows, cudaMemcpyDeviceToDevice, st),
                       "cudaMemcpy2DAsync(gather)");
    }
    uint64_t cmax = 0;                                                   // the widest block
    for (int r = 0; r < h->world; r++) cmax = cmax > h->split.begin[r + 1] - h->split.begin[r] ? cmax : h->split.begin[r + 1] - h->split.begin[r];
    const size_t per_rank = (size_t)rows * cmax * 4;
    const size_t want = per_rank * (size_t)h->world;
    if (h->landing_bytes < want) {
        if (int e = cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return e;
        device_free(h->landing);
        h->landing = nullptr;
        h->landing_bytes = 0;
        void* p = nullptr;
        if (int e = device_alloc(&p, want, "sharded linear: gather landing buffer")) return e;
        h->landing = static_cast<float*>(p);
        h->landing_bytes = want;
    }
    // A block that is as wide as the widest and dense is sent as it lies; others are padded into the landing buffer first.
    const float* send = block;
    if (h->col_count != cmax || ld != cmax) {
        float* mine = h->landing + (size_t)h->rank * rows * cmax;
        pack_columns_kernel<<<(unsigned int)sm_count() * 8, 256, 0, st>>>(block, ld, mine, rows, h->col_count, cmax);
        if (int e = launched("pack_columns_kernel")) return e;
        send = mine;
    }
    if (int e = nccl_ok(nccl_api()->AllGather(send, h->landing, per_rank, kNcclInt8, h->comm, st), "ncclAllGather(columns)")) return e;
    bool vec = h->n_total % 4 == 0 && cmax % 4 == 0 && (((uintptr_t)full | (uintptr_t)h->landing) & 15) == 0;
    for (int r = 0; r < h->world; r++) vec = vec && h->split.begin[r] % 4 == 0;
    if (vec) unpack_columns_kernel<4><<<(unsigned int)sm_count() * 8, 256, 0, st>>>(h->landing, full, rows, h->n_total, cmax, h->world, h->split);
    else unpack_columns_kernel<1><<<(unsigned int)sm_count() * 8, 256, 0, st>>>(h->landing, full, rows, h->n_total, cmax, h->world, h->split);
    return launched("unpack_columns_kernel");
}

int rplb_sharded_linear_submit_host(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, float* out, int relu,
                                    int row_blocks, void* compute_stream) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (int e = check_call(h, rows, out, h ? h->col_count : 0)) return e;
    if (int e = pipeline_ready(h, as_stream(compute_stream))) return e;
    uint64_t r0, rc;
    row_range(h, rows, &r0, &rc);
    if (rc && !x_local) return fail(RPLB_E_BAD_ARG, "sharded linear: null activation");
    const uint64_t K = h->K, N = h->col_count;
    const int i = (int)(h->calls % kDepth);
    const size_t in_bytes = (size_t)(rc ? rc : 1) * K * 4, out_bytes = (size_t)rows * (N ? N : 1) * 4;
    if (h->din_bytes[i] < in_bytes || h->dout_bytes[i] < out_bytes) {
        // Buffers change size only with everything idle.
        if (int e = cuda_ok(cudaStreamSynchronize(h->s_in), "cudaStreamSynchronize")) return e;
        if (int e = cuda_ok(cudaStreamSynchronize(h->s_main), "cudaStreamSynchronize")) return e;
        if (int e = cuda_ok(cudaStreamSynchronize(h->s_out), "cudaStreamSynchronize")) return e;
        if (int e = grow(&h->din[i], &h->din_bytes[i], in_bytes, "sharded linear: activation slot")) return e;
        if (int e = grow(&h->dout[i], &h->dout_bytes[i], out_bytes, "sharded linear: output slot")) return e;
    }
    float* din = h->din[i];
    float* dout = h->dout[i];
    cudaStream_t st = h->s_main;
    if (h->slot_used[i]) if (int e = cuda_ok(cudaStreamWaitEvent(h->s_in, h->ev_computed[i], 0), "cudaStreamWaitEvent")) return e;
    if (rc) if (int e = cuda_ok(cudaMemcpyAsync(din, x_local, (size_t)rc * K * 4, cudaMemcpyHostToDevice, h->s_in), "cudaMemcpyAsync(upload)")) return e;
    if (int e = cuda_ok(cudaEventRecord(h->ev_uploaded[i], h->s_in), "cudaEventRecord")) return e;
    if (int e = cuda_ok(cudaStreamWaitEvent(st, h->ev_uploaded[i], 0), "cudaStreamWaitEvent")) return e;
    if (h->slot_used[i]) if (int e = cuda_ok(cudaStreamWaitEvent(st, h->ev_downloaded[i], 0), "cudaStreamWaitEvent")) return e;
    if (int e = quantize_and_send(h, din, rows, st)) return e;
    // Row blocks, beginning with the one that holds this rank's own rows; each is downloaded while the next computes.
    if (row_blocks < 1) row_blocks = 8;
    if (row_blocks > kMaxBlocks) row_blocks = kMaxBlocks;
    uint64_t step = (rows + (uint64_t)row_blocks - 1) / (uint64_t)row_blocks;
    step = (step + 127) / 128 * 128;
    const uint64_t nblocks = (rows + step - 1) / step;
    const uint64_t first = r0 / step < nblocks ? r0 / step : 0;
    for (uint64_t j = 0; j < nblocks; j++) {
        const uint64_t b = (first + j) % nblocks;
        const uint64_t b0 = b * step, b1 = b0 + step < rows ? b0 + step : rows;
        if (int e = gemm_rows(h, rows, b0, b1, dout, N, relu, st)) return e;
        if (int e = cuda_ok(cudaEventRecord(h->ev_block[i][j], st), "cudaEventRecord")) return e;
        if (int e = cuda_ok(cudaStreamWaitEvent(h->s_out, h->ev_block[i][j], 0), "cudaStreamWaitEvent")) return e;
        if (N) if (int e = cuda_ok(cudaMemcpyAsync(out + b0 * N, dout + b0 * N, (size_t)(b1 - b0) * N * 4, cudaMemcpyDeviceToHost, h->s_out),
                                   "cudaMemcpyAsync(download)")) return e;
    }
    if (int e = after_gemm(h, st)) return e;
    if (int e = cuda_ok(cudaEventRecord(h->ev_computed[i], st), "cudaEventRecord")) return e;
    if (int e = cuda_ok(cudaEventRecord(h->ev_downloaded[i], h->s_out), "cudaEventRecord")) return e;
    h->slot_used[i] = true;
    h->calls++;
    return 0;
}

int rplb_sharded_linear_drain(rplb_sharded_linear* layer) {
    ShardedLinear* h = reinterpret_cast<ShardedLinear*>(layer);
    if (!h || !h->s_in) return 0;
    for (int i = 0; i < kDepth; i++)
        if (h->slot_used[i]) if (int e = cuda_ok(cudaStreamWaitEvent(h->s_main, h->ev_downloaded[i], 0), "cudaStreamWaitEvent")) return e;
    if (int e = cuda_ok(cudaStreamSynchronize(h->s_out), "cudaStreamSynchronize")) return e;
    if (int e = cuda_ok(cudaStreamSynchronize(h->s_main), "cudaStreamSynchronize")) return e;
    if (int st = rplb_kernel_status(1)) return fail(RPLB_E_KERNEL, "sharded linear: a kernel gave up waiting (code %d)", st);
    return 0;
}

}  // extern "C"
