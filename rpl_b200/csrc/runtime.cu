// Host-side plumbing behind the rplb_* layer: error text, launch counter,
// per-stream scratch blocks, memory and stream helpers.
#include "common.cuh"
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <tuple>
#include <utility>

namespace rplb {

static thread_local char g_err_text[512] = "";
static std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err_text, sizeof(g_err_text), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    snprintf(g_err_text, sizeof(g_err_text), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) return RPLB_E_NO_DEVICE;
    return (int)e;
}

int launched(const char* kernel) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_ok(cudaGetLastError(), kernel);
}

// ---------------------------------------------------------------------------
struct ScratchBlock {
    void* base = nullptr;
    size_t bytes = 0;
};
// One block per (device, stream, host thread): two host threads that use the same stream (the reference-named API
// runs every thread on the default stream) must not share a block, because a call keeps data in it between two of
// its own kernels (a transposed B, row and column sums, min/max partials) and the other thread's kernels can be
// queued in between.
typedef std::tuple<int, cudaStream_t, std::thread::id> ScratchKey;
static std::mutex g_scratch_mu;
static std::map<ScratchKey, ScratchBlock> g_scratch;
static constexpr size_t kControlBytes = 256;

// Device allocator behind rplb_malloc / rplb_free and the scratch blocks:
// cudaMalloc / cudaFree unless the application installed its own pair.
static rplb_alloc_fn g_alloc_fn = nullptr;
static rplb_free_fn g_free_fn = nullptr;

int device_alloc(void** p, size_t bytes, const char* what) {
    *p = nullptr;
    if (g_alloc_fn) {
        const int rc = g_alloc_fn(p, bytes);
        if (rc != 0 || !*p) {
            *p = nullptr;
            return fail(rc != 0 ? rc : (int)cudaErrorMemoryAllocation, "%s: the installed allocator could not provide %zu bytes", what, bytes);
        }
        return 0;
    }
    return cuda_ok(cudaMalloc(p, bytes), what);
}

int device_free(void* p) {
    if (!p) return 0;
    if (g_free_fn) return g_free_fn(p);
    return cuda_ok(cudaFree(p), "cudaFree");
}

int scratch_for(cudaStream_t stream, size_t bytes, Scratch* out) {
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    ScratchBlock& b = g_scratch[ScratchKey(dev, stream, std::this_thread::get_id())];
    size_t want = kControlBytes + ((bytes + 255) & ~size_t(255));
    if (b.bytes < want) {
        // A block cannot be allocated, grown or cleared while the stream records a
        // graph: the graph would keep the address of a block that a later call
        // frees.  Reserve the largest size first (rplb_scratch_reserve), then capture.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
        if (cap != cudaStreamCaptureStatusNone)
            return fail(RPLB_E_UNSUPPORTED, "the stream is being captured and its scratch block (%zu bytes) is too small for %zu: "
                        "call rplb_scratch_reserve before the capture", b.bytes, want);
        if (b.base) {
            // Work queued on the stream may still use the old block.
            if (int rc = cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
            device_free(b.base);
            b.base = nullptr;
            b.bytes = 0;
        }
        size_t grow = want < (size_t(1) << 20) ? (size_t(1) << 20) : want;
        if (int rc = device_alloc(&b.base, grow, "scratch allocation")) return rc;
        if (int rc = cuda_ok(cudaMemsetAsync(b.base, 0, kControlBytes, stream), "cudaMemsetAsync(scratch)")) return rc;
        b.bytes = grow;
    }
    out->control = static_cast<unsigned int*>(b.base);
    out->data = static_cast<char*>(b.base) + kControlBytes;
    return 0;
}

int sm_count() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 0;
    cache[dev] = n;
    return n;
}

}  // namespace rplb

using namespace rplb;

extern "C" {

const char* rplb_last_error(void) { return g_err_text; }

int rplb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int rplb_device_sm_count(void) { return sm_count(); }

int rplb_set_device(int ordinal) { return cuda_ok(cudaSetDevice(ordinal), "cudaSetDevice"); }

uint64_t rplb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int rplb_malloc(void** dptr, size_t bytes) {
    if (!dptr) return fail(RPLB_E_BAD_ARG, "rplb_malloc: null result pointer");
    *dptr = nullptr;
    if (bytes == 0) bytes = 1;
    return device_alloc(dptr, bytes, "cudaMalloc");
}

int rplb_free(void* dptr) { return device_free(dptr); }

int rplb_set_allocator(rplb_alloc_fn alloc_fn, rplb_free_fn free_fn) {
    if ((alloc_fn == nullptr) != (free_fn == nullptr))
        return fail(RPLB_E_BAD_ARG, "rplb_set_allocator: give both functions or neither");
    g_alloc_fn = alloc_fn;
    g_free_fn = free_fn;
    return 0;
}

int rplb_scratch_reserve(void* stream, size_t bytes) {
    Scratch sc;
    return scratch_for(as_stream(stream), bytes, &sc);
}

int rplb_scratch_release(void* stream) {
    int dev = 0;
    if (int rc = cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    cudaStream_t st = as_stream(stream);
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    auto it = g_scratch.find(ScratchKey(dev, st, std::this_thread::get_id()));
    if (it == g_scratch.end()) return 0;
    if (it->second.base) {
        if (int rc = cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return rc;
        device_free(it->second.base);
    }
    g_scratch.erase(it);
    return 0;
}

int rplb_host_alloc(void** hptr, size_t bytes) {
    if (!hptr) return fail(RPLB_E_BAD_ARG, "rplb_host_alloc: null result pointer");
    *hptr = nullptr;
    if (bytes == 0) bytes = 1;
    return cuda_ok(cudaHostAlloc(hptr, bytes, cudaHostAllocDefault), "cudaHostAlloc");
}

int rplb_host_free(void* hptr) { return hptr ? cuda_ok(cudaFreeHost(hptr), "cudaFreeHost") : 0; }

int rplb_copy(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(RPLB_E_BAD_ARG, "rplb_copy: null pointer");
    return cuda_ok(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, as_stream(stream)), "cudaMemcpyAsync");
}

int rplb_stream_sync(void* stream) { return cuda_ok(cudaStreamSynchronize(as_stream(stream)), "cudaStreamSynchronize"); }

int rplb_stream_create(void** stream) {
    if (!stream) return fail(RPLB_E_BAD_ARG, "rplb_stream_create: null result pointer");
    cudaStream_t s = nullptr;
    if (int rc = cuda_ok(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags")) return rc;
    *stream = s;
    return 0;
}

int rplb_stream_destroy(void* stream) { return stream ? cuda_ok(cudaStreamDestroy(as_stream(stream)), "cudaStreamDestroy") : 0; }

int rplb_event_create(void** event) {
    if (!event) return fail(RPLB_E_BAD_ARG, "rplb_event_create: null result pointer");
    cudaEvent_t e = nullptr;
    if (int rc = cuda_ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreateWithFlags")) return rc;
    *event = e;
    return 0;
}

int rplb_event_destroy(void* event) { return event ? cuda_ok(cudaEventDestroy(static_cast<cudaEvent_t>(event)), "cudaEventDestroy") : 0; }

int rplb_event_record(void* event, void* stream) {
    return cuda_ok(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)), "cudaEventRecord");
}

int rplb_stream_wait_event(void* stream, void* event) {
    return cuda_ok(cudaStreamWaitEvent(as_stream(stream), static_cast<cudaEvent_t>(event), 0), "cudaStreamWaitEvent");
}

// Sharing a device block between the processes of one node (one process per
// GPU): the owner exports a 64-byte handle, the others open it and get an
// address of the same memory in their own address space, with peer access
// between the two GPUs switched on as needed.
static_assert(sizeof(cudaIpcMemHandle_t) == RPLB_IPC_HANDLE_BYTES, "handle size");

int rplb_ipc_export(const void* dptr, void* handle) {
    if (!dptr || !handle) return fail(RPLB_E_BAD_ARG, "rplb_ipc_export: null pointer");
    cudaIpcMemHandle_t h;
    if (int rc = cuda_ok(cudaIpcGetMemHandle(&h, const_cast<void*>(dptr)), "cudaIpcGetMemHandle")) return rc;
    memcpy(handle, &h, sizeof(h));
    return 0;
}

int rplb_ipc_open(const void* handle, void** dptr) {
    if (!handle || !dptr) return fail(RPLB_E_BAD_ARG, "rplb_ipc_open: null pointer");
    *dptr = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    return cuda_ok(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int rplb_ipc_close(void* dptr) { return dptr ? cuda_ok(cudaIpcCloseMemHandle(dptr), "cudaIpcCloseMemHandle") : 0; }

int rplb_pointer_kind(const void* p) {
    if (!p) return 0;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    switch (a.type) {
        case cudaMemoryTypeHost: return 1;
        case cudaMemoryTypeDevice: return 2;
        case cudaMemoryTypeManaged: return 3;
        default: return 0;
    }
}

int rplb_shard_range(uint64_t n, int world, int rank, uint64_t align, uint64_t* begin, uint64_t* count) {
    if (world <= 0 || rank < 0 || rank >= world || !begin || !count)
        return fail(RPLB_E_BAD_ARG, "rplb_shard_range: bad world/rank");
    if (align == 0) align = 1;
    // Units of `align` columns are dealt out as evenly as possible, the first
    // (units % world) ranks taking one more; the last unit may be ragged.
    uint64_t units = (n + align - 1) / align;
    uint64_t base = units / (uint64_t)world, extra = units % (uint64_t)world;
    uint64_t r = (uint64_t)rank;
    uint64_t u0 = r * base + (r < extra ? r : extra);
    uint64_t u1 = u0 + base + (r < extra ? 1 : 0);
    uint64_t b = u0 * align, e = u1 * align;
    if (b > n) b = n;
    if (e > n) e = n;
    *begin = b;
    *count = e - b;
    return 0;
}

}  // extern "C"
