/*
 * rpl_b200.h -- C ABI of librpl.so, the sm_100a (B200) implementation of the
 * INT8 quantized-inference path of RPL.
 *
 * Two layers, both plain C linkage, plain pointers and sizes:
 *
 *  1. "rplb_*"  device-level entry points.  Every data pointer is a CUDA device
 *     pointer on the current device; `stream` is a cudaStream_t passed as
 *     void* (NULL = the legacy default stream).  Calls are asynchronous on
 *     that stream unless stated.  Return value: 0 on success, otherwise a
 *     negative RPLB_E_* code or a positive cudaError_t; rplb_last_error()
 *     gives the text.
 *
 *  2. The reference's own exported names (tensor_quantize_int8, gemm_int8,
 *     linear_int8 ...), same signatures, struct layouts and ownership rules as
 *     the reference library, so a program built against the reference's
 *     include/rpl.h links against this library unchanged.  Each data pointer
 *     may be a host pointer (staged over PCIe) or a device pointer (used in
 *     place); results live where the inputs live.  These calls return after
 *     the result is complete.
 *
 * There is no CPU implementation behind any of these: without a CUDA device
 * every compute entry point fails (rplb_* return an error; the reference-named
 * producers return NULL and report on stderr, the reference's own convention
 * for a failed tensor_create, src/rpl_core.c:45).
 *
 * If the reference's rpl.h is included first its type definitions are used;
 * otherwise layout-identical ones are defined here.
 */
#ifndef RPL_B200_H
#define RPL_B200_H

#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------
 * Types shared with the reference (layouts frozen; x86-64 offsets in
 * brackets are checked by static assertions in the library).
 * ---------------------------------------------------------------------- */
#ifndef RPL_H
#define RPL_B200_OWN_TYPES 1
#define MAX_DIMS 8                      /* include/rpl.h:32 */

typedef enum { DEVICE_CPU, DEVICE_GPU } DeviceType;   /* include/rpl.h:23-26 */

/* include/rpl.h:57-78, sizeof 152 */
typedef struct Tensor {
    float*    data;                     /* [0]   host or device pointer        */
    float*    grad;                     /* [8]                                 */
    uint32_t  dims;                     /* [16]                                */
    uint32_t  shape[MAX_DIMS];          /* [20]                                */
    uint32_t  strides[MAX_DIMS];        /* [52]  row-major, in elements        */
    uint32_t  size;                     /* [84]  product of shape              */
    bool      requires_grad;            /* [88]                                */
    void*     _allocation;              /* [96]  what tensor_free releases     */
    size_t    _alloc_size;              /* [104]                               */
    DeviceType device;                  /* [112]                               */
    uint32_t  gpu_buffer;               /* [116]                               */
    bool      is_leaf;                  /* [120]                               */
    struct Tensor* parent1;             /* [128]                               */
    struct Tensor* parent2;             /* [136]                               */
    void (*backward_fn)(struct Tensor*);/* [144]                               */
} Tensor;

/* include/rpl.h:167-174, sizeof 56 */
typedef struct {
    int8_t*  data;                      /* [0]  separate 64-byte aligned block */
    float    scale;                     /* [8]                                 */
    int32_t  zero_point;                /* [12]                                */
    uint32_t size;                      /* [16]                                */
    uint32_t dims;                      /* [20]                                */
    uint32_t shape[MAX_DIMS];           /* [24]                                */
} QuantizedTensor;
#endif /* RPL_H */

/* src/rpl_quantization.c:110-118 (private to that file in the reference, but
 * returned by the exported tensor_quantize_per_channel). */
typedef struct {
    int8_t*  data;
    float*   scales;                    /* one per channel                     */
    int32_t* zero_points;               /* one per channel, always 0           */
    uint32_t num_channels;
    uint32_t channel_size;
    uint32_t dims;
    uint32_t shape[8];
} PerChannelQuantizedTensor;

/* src/rpl_quantization.c:18-24 */
typedef struct {
    float    min_val;
    float    max_val;
    float    scale;
    int32_t  zero_point;
    uint32_t num_samples;
} QuantizationCalibrator;

/* src/rpl_quantization.c:271-276 */
typedef struct {
    Tensor**          fp32_params;
    QuantizedTensor** int8_params;
    uint32_t          num_params;
    bool              is_quantized;
} QuantizedModel;

/* ------------------------------------------------------------------------
 * Error codes of the rplb_* layer (CUDA errors are returned as positive
 * cudaError_t values).
 * ---------------------------------------------------------------------- */
#define RPLB_OK              0
#define RPLB_E_NO_DEVICE    (-1)   /* no CUDA device / driver                  */
#define RPLB_E_BAD_ARG      (-2)   /* null pointer, misaligned or bad size     */
#define RPLB_E_TOO_LARGE    (-3)   /* size beyond what the entry point takes   */
#define RPLB_E_KERNEL       (-4)   /* a kernel reported a bounded wait expired */
#define RPLB_E_UNSUPPORTED  (-5)   /* shape the selected GEMM kernel can't run */
#define RPLB_E_COMM         (-6)   /* NCCL could not be loaded, or a communicator call failed */

const char* rplb_last_error(void);          /* text of this thread's last failure */
int  rplb_device_count(void);               /* 0 when there is no usable device   */
int  rplb_device_sm_count(void);            /* SMs of the current device           */
int  rplb_set_device(int ordinal);          /* device of the calling thread's later calls (one process per GPU: its rank) */

/* ------------------------------------------------------------------------
 * Memory and stream helpers, so that a C host needs no CUDA headers.
 * ---------------------------------------------------------------------- */
int  rplb_malloc(void** dptr, size_t bytes);
int  rplb_free(void* dptr);
/* An application that manages device memory itself installs its allocator here
 * (both functions, or NULL and NULL to go back to cudaMalloc / cudaFree);
 * rplb_malloc, rplb_free and the library's scratch blocks then use it.  The
 * functions return 0 on success; a non-zero code from alloc_fn is handed back
 * to the caller of the entry point that needed the memory.  Install before the
 * first allocation.  The reference allocates with posix_memalign and has no
 * hook (src/rpl_core.c:33-43). */
typedef int (*rplb_alloc_fn)(void** dptr, size_t bytes);
typedef int (*rplb_free_fn)(void* dptr);
int  rplb_set_allocator(rplb_alloc_fn alloc_fn, rplb_free_fn free_fn);
/* Scratch memory of the library: one block per (device, stream, calling host
 * thread), allocated on first use and grown (after a stream synchronize, by
 * free + allocate) when a call needs more: min/max partial results, a
 * transposed B, row and column sums.  Host threads never share a block, so
 * they may call into the library at the same time, on the same stream or on
 * different ones; reserve and release act on the calling thread's block.  A CUDA graph captured from rplb_* calls keeps the block's address, so
 * reserve the largest size the stream will ever need before capturing; a call
 * that would have to grow the block of a capturing stream fails with
 * RPLB_E_UNSUPPORTED instead.  release frees the block of a stream that is
 * about to be destroyed. */
int  rplb_scratch_reserve(void* stream, size_t bytes);
int  rplb_scratch_release(void* stream);
int  rplb_host_alloc(void** hptr, size_t bytes);     /* page-locked host memory */
int  rplb_host_free(void* hptr);
int  rplb_copy(void* dst, const void* src, size_t bytes, void* stream);   /* any direction, async */
int  rplb_stream_sync(void* stream);
int  rplb_stream_create(void** stream);              /* a non-blocking stream */
int  rplb_stream_destroy(void* stream);
int  rplb_event_create(void** event);                /* ordering only, no timing */
int  rplb_event_destroy(void* event);
int  rplb_event_record(void* event, void* stream);
int  rplb_stream_wait_event(void* stream, void* event);
/* 0 = ordinary host memory, 1 = page-locked host, 2 = device, 3 = managed */
int  rplb_pointer_kind(const void* p);

/* One process per GPU on one node: a block from rplb_malloc is shared by
 * exporting a handle of RPLB_IPC_HANDLE_BYTES bytes (sent to the other
 * processes by any means), which they open to get an address of the same
 * memory in their own address space; peer access between the two GPUs is
 * switched on as needed.  Close before the owner frees the block.  No
 * counterpart in the reference (single process, no accelerator memory). */
#define RPLB_IPC_HANDLE_BYTES 64
int  rplb_ipc_export(const void* dptr, void* handle);
int  rplb_ipc_open(const void* handle, void** dptr);
int  rplb_ipc_close(void* dptr);

/* ------------------------------------------------------------------------
 * Quantization parameters as the reduction kernel leaves them on the device.
 * ---------------------------------------------------------------------- */
typedef struct {
    float   min_val;      /* min over non-NaN elements, seeded +FLT_MAX (src/rpl_quantization.c:79-85) */
    float   max_val;      /* max over non-NaN elements, seeded -FLT_MAX                                */
    float   scale_sym;    /* fmaxf(|min|,|max|) / 127.0f            (src/rpl_quantization.c:87-88)    */
    float   scale_asym;   /* (max - min) / 255.0f                   (src/rpl_quantization.c:102-103)  */
    int32_t zp_asym;      /* (int32) roundf(-min / scale_asym)      (src/rpl_quantization.c:104)      */
    float   first;        /* x[0]; tensor_get_min_max seeds with it (src/ops_extended.c:54-55)        */
    float   true_min;     /* min over non-NaN elements, seeded +inf                                    */
    float   true_max;     /* max over non-NaN elements, seeded -inf                                    */
} rplb_qparams;           /* 32 bytes */

/* Replaces the min/max loops of tensor_get_min_max (src/ops_extended.c:52-61),
 * tensor_quantize_int8_symmetric/_asymmetric (src/rpl_quantization.c:79-85,
 * :96-100) and calibrator_update (src/rpl_quantization.c:33-49).
 * x: n floats on the device; params: one rplb_qparams on the device.
 * Uses the library's per-stream scratch buffer (allocated on first use). */
int  rplb_minmax_f32(const float* x, uint64_t n, rplb_qparams* params, void* stream);

/* No counterpart in the reference.  rplb_minmax_f32 for callers that must not
 * allocate device memory: plugins running inside a host application that owns
 * the whole GPU memory budget, real-time loops where cudaMalloc's implicit
 * synchronisation is unacceptable, code that runs after the application has
 * frozen its allocations.  The per-CTA partial results and the ticket counter
 * live in a fixed 8.25 KiB array that is part of the library image on every
 * device that loads it; the call itself performs no cudaMalloc/cudaFree.
 *   - n above RPLB_STATIC_MINMAX_MAX_ELEMENTS is rejected (RPLB_E_TOO_LARGE).
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that call before any stream capture.
 *   - All calls share the one array: calls that may overlap on the GPU
 *     (different streams, no ordering between them) race.  Calls ordered by a
 *     stream or an event are safe; the counter is cleared at every call.
 * Same inputs, outputs and results as rplb_minmax_f32. */
#define RPLB_STATIC_MINMAX_MAX_CTAS      1024u
#define RPLB_STATIC_MINMAX_MAX_ELEMENTS  (1ull << 30)
int  rplb_minmax_f32_static(const float* x, uint64_t n, rplb_qparams* params, void* stream);

/* A tensor whose rows live on several GPUs (src/rpl_quantization.c:79-88 over
 * a row-sharded activation): every GPU runs rplb_minmax_f32 on its rows,
 * to_pair leaves (-min, max) in two device floats, the caller combines the
 * pairs of all GPUs with a max-reduction (ncclAllReduce, op max), and from_pair
 * derives all parameters from the combined pair with the statements
 * rplb_minmax_f32 itself ends with, IEEE division included, so every GPU holds
 * the scale a single GPU would have computed. */
int  rplb_qparams_to_pair(const rplb_qparams* params, float* pair, void* stream);
int  rplb_qparams_from_pair(const float* pair, rplb_qparams* params, void* stream);

/* Replaces the loop of tensor_quantize_int8 (src/rpl_core.c:521-527):
 * q = clamp((int32)roundf(x/scale) + zp, -128, 127). */
int  rplb_quantize_f32_i8(const float* x, int8_t* q, uint64_t n, float scale, int32_t zero_point, void* stream);

/* Same statement with scale (and optionally the zero point) read from device
 * memory, so that no host round trip separates it from rplb_minmax_f32.
 * zp_dev may be NULL (zero point 0). */
int  rplb_quantize_f32_i8_dev(const float* x, int8_t* q, uint64_t n, const float* scale_dev,
                              const int32_t* zp_dev, void* stream);

/* tensor_quantize_int8_symmetric (src/rpl_quantization.c:77-91) on device
 * buffers: min/max pass, then quantize with params->scale_sym, zero point 0.
 * Tensors of up to a few million elements (what fits in the registers of one
 * resident grid; 16-byte aligned x, 4-byte aligned q) are done in one
 * cooperative launch that reads the tensor once; larger ones in two kernels. */
int  rplb_quantize_symmetric_f32_i8(const float* x, int8_t* q, uint64_t n, rplb_qparams* params, void* stream);

/* tensor_quantize_int8_asymmetric (src/rpl_quantization.c:93-107). */
int  rplb_quantize_asymmetric_f32_i8(const float* x, int8_t* q, uint64_t n, rplb_qparams* params, void* stream);

/* Whether the two calls above may take their one-launch path (per host thread;
 * 1 = yes, the default; 0 = always two kernels).  Same results; for
 * measurements.  Returns the previous setting. */
int  rplb_quantize_onepass(int which);

/* tensor_quantize_per_channel (src/rpl_quantization.c:134-157): channel c is
 * the contiguous block [c*channel_size, (c+1)*channel_size).  scales and
 * zero_points (may be NULL) have num_channels entries. */
int  rplb_quantize_per_channel_f32_i8(const float* x, int8_t* q, float* scales, int32_t* zero_points,
                                      uint64_t num_channels, uint64_t channel_size, void* stream);

/* How rplb_quantize_per_channel_f32_i8 treats channels of 32 to 232 KiB (8192
 * to 59392 floats) for the calling thread: 1 (default) = the channel is kept on
 * chip (part in registers, the rest staged in shared memory by bulk copies) and
 * read from HBM once, 0 = two passes over the channel (the second normally
 * served by L2).  Same results; for measurements.
 * Returns the previous setting. */
int  rplb_per_channel_staging(int which);

/* tensor_dequantize_int8 (src/ops_extended.c:67-70): out = (float)(q - zp) * scale. */
int  rplb_dequantize_i8_f32(const int8_t* q, float* out, uint64_t n, float scale, int32_t zero_point, void* stream);

/* Per-channel form of the same statement, out = (float)q * scales[c]; the
 * reference has no such function (its PerChannelQuantizedTensor has no
 * dequantizer), the arithmetic is src/ops_extended.c:69 with zp 0. */
int  rplb_dequantize_per_channel_i8_f32(const int8_t* q, const float* scales, float* out,
                                        uint64_t num_channels, uint64_t channel_size, void* stream);

/* ------------------------------------------------------------------------
 * INT8 x INT8 -> INT32 contraction.
 * ---------------------------------------------------------------------- */
/* linear_int8 (src/rpl_quantization.c:314-353): out[m,n] = sum_k x[m,k]*w[n,k]
 * (+ (int8) bias[n] when bias != NULL), raw int32.  x [M,K], w [N,K], out [M,N]. */
int  rplb_linear_i8_i32(const int8_t* x, const int8_t* w, const int8_t* bias, int32_t* out,
                        uint64_t M, uint64_t K, uint64_t N, void* stream);

/* gemm_int8 / gemm_int8_fallback, scalar branch (src/ops_extended.c:83-129):
 * C[i,j] = (int32) roundf( (((float) sum_k (A[i,k]-za)(B[k,j]-zb)) * sa * sb) / sc ),
 * A [M,K], B [K,N] (row-major), C [M,N]. */
int  rplb_gemm_i8_requant_i32(const int8_t* A, const int8_t* B, int32_t* C,
                              uint64_t M, uint64_t N, uint64_t K,
                              float sa, float sb, float sc, int32_t za, int32_t zb, void* stream);

/* Fused fp32 epilogue (no counterpart function in the reference; it composes
 * linear_int8 src/rpl_quantization.c:340-350, the dequantize statement
 * src/ops_extended.c:69, the bias broadcast src/rpl_nn.c:69-71 and ReLU
 * src/rpl_core.c:254-255):
 *   out[m,n] = relu?( (((float)acc[m,n] * *a_scale) * w_scales[n]) + bias[n] )
 * a_scale: one float on the device; w_scales: N floats; bias: N floats or NULL;
 * ldo: row stride of out in elements (>= N), so a column block of a wider
 * matrix can be written in place. */
int  rplb_linear_i8_dequant_f32(const int8_t* x, const int8_t* w, float* out,
                                uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                const float* a_scale, const float* w_scales, const float* bias,
                                int relu, void* stream);

/* The same call for an output whose column blocks are computed on different
 * GPUs and wanted whole on each of them: besides `out`, the values are stored
 * at the same [m, n] offsets (row stride ldo) in n_peers further buffers
 * (at most 7), normally the other ranks' [M, N_total] outputs opened with
 * rplb_ipc_open, every pointer already advanced to this rank's first column.
 * peer_out is a host array.  The exchange rides in the GEMM's epilogue as plain
 * stores over NVLink; no gather pass follows.  The caller orders the ranks:
 * nobody may still read a destination when the call starts, and a rank may
 * read its own buffer only after every rank's call has completed (a barrier
 * on the streams, e.g. an NCCL all-reduce of one word).  Needs K % 16 == 0
 * and 16-byte aligned x and w; other shapes are refused, not emulated.  No
 * counterpart in the reference (single device). */
int  rplb_linear_i8_dequant_f32_peers(const int8_t* x, const int8_t* w, float* out,
                                      uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                      const float* a_scale, const float* w_scales, const float* bias,
                                      int relu, float* const* peer_out, int n_peers, void* stream);

/* The same call for an activation whose rows are still arriving from other GPUs
 * when the kernel starts (the consumer half of an all-gather fused into the
 * GEMM).  row_block_ready: one 32-bit word in this GPU's memory per block of
 * 128 rows of x; a block is complete once its word has reached `epoch`
 * (compared modulo 2^32), which the sender writes after the rows (for example a
 * peer copy of the rows followed by a peer copy of the words on the same
 * stream).  Blocks [local_first_block, local_first_block + local_blocks) are
 * complete at launch: the kernel starts with them, takes the other blocks in
 * ascending order (wrapping round), and before the first load of each waits,
 * for about a second at most, for its word; if the wait runs out the kernel
 * returns and rplb_kernel_status reports 5.  Needs K % 16 == 0 and 16-byte
 * aligned x and w.  No counterpart in the reference (single device). */
int  rplb_linear_i8_dequant_f32_arriving(const int8_t* x, const int8_t* w, float* out,
                                         uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                         const float* a_scale, const float* w_scales, const float* bias,
                                         int relu, const uint32_t* row_block_ready, uint32_t epoch,
                                         uint32_t local_first_block, uint32_t local_blocks, void* stream);

/* The same call that also reports what the next layer's per-tensor quantizer
 * needs, so that layer can skip its min/max pass over the fp32 output (no
 * counterpart in the reference, which always re-scans: src/rpl_quantization.c:79-85).
 * absmax (device, one float) receives max |out| over non-NaN outputs; if
 * next_scale (device, one float) is not NULL it receives absmax / 127.0f, the
 * scale tensor_quantize_int8_symmetric would compute for `out`
 * (src/rpl_quantization.c:87-88).  Feed it to rplb_quantize_f32_i8_dev. */
int  rplb_linear_i8_dequant_f32_absmax(const int8_t* x, const int8_t* w, float* out,
                                       uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                       const float* a_scale, const float* w_scales, const float* bias,
                                       int relu, float* absmax, float* next_scale, void* stream);

/* tensor_quantize_int8 (src/rpl_core.c:521-527, zero point 0) fused into the
 * layer that consumes it, for layers with few output features: x is the fp32
 * activation [M,K]; it is quantized with *a_scale on its way into the
 * contraction (the int8 activation is never written to memory), and the result
 * is out[m,n] = relu?(((float)acc * *a_scale) * w_scales[n] + bias[n]) as
 * rplb_linear_i8_dequant_f32 computes it from a quantized copy: same bits.
 * Such layers are bound by HBM, and this removes a write and a read of the
 * int8 activation and the buffer that holds it.  absmax / next_scale (both may
 * be NULL) as in rplb_linear_i8_dequant_f32_absmax.  Shapes: N <= 16 with
 * K <= 512 and K % 4 == 0 run on dp4a (measured faster than quantize + GEMM:
 * 14.5 against 18.6 us for 65536 x 128 -> 10); N <= 128 with K <= 896 and
 * K % 16 == 0 run on the tensor cores with the whole weight matrix resident in
 * shared memory and converter warps between the TMA loads of fp32 rows and the
 * MMAs (the conversion is instruction-bound: about as fast as the two kernels
 * it replaces, 80 against 71 us for 65536 x 784 -> 128; use it to save the
 * buffer, not the time); anything else is refused with RPLB_E_UNSUPPORTED
 * (quantize into a buffer instead).
 * x and w 16-byte aligned.  No counterpart in the reference, which always
 * materialises the quantized tensor (src/rpl_quantization.c:77-91). */
int  rplb_quantize_linear_dequant_f32(const float* x, const int8_t* w, float* out,
                                      uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                                      const float* a_scale, const float* w_scales, const float* bias,
                                      int relu, float* absmax, float* next_scale, void* stream);

/* Chained quantized layers with a calibrated (static) output scale: the fp32
 * value of rplb_linear_i8_dequant_f32 is quantized in the epilogue exactly as
 * tensor_quantize_int8 would (src/rpl_core.c:523-526) and stored as int8, so
 * the fp32 activation never reaches memory.  out_scale: one float on the
 * device (e.g. from calibrator_compute_params, src/rpl_quantization.c:55-67). */
int  rplb_linear_i8_requant_i8(const int8_t* x, const int8_t* w, int8_t* out,
                               uint64_t M, uint64_t K, uint64_t N, uint64_t ldo,
                               const float* a_scale, const float* w_scales, const float* bias,
                               int relu, const float* out_scale, int32_t out_zero_point, void* stream);

/* tensor_relu_inplace, scalar branch (src/rpl_core.c:254-255): x < 0 -> 0 in
 * place.  (The fused entry point above applies it inside the GEMM epilogue.) */
int  rplb_relu_f32_inplace(float* x, uint64_t n, void* stream);

/* Status word of the tensor-core kernels launched by the calling host thread:
 * 0, or the code of the bounded wait that expired (1 stage-free, 2 stage-loaded,
 * 3 accumulator-free, 4 accumulator-ready, 5 rows from another GPU; 6 = a bulk
 * copy of the per-channel quantizer's staged rows did not complete, 7 = the
 * grid barrier of the one-launch per-tensor quantizer, 8 = the 256x256
 * kernel found its shared memory starting off a 128-byte boundary and did
 * nothing: never seen on sm_100a, checked because the kernel counts on it).  Every
 * host thread has a word of its own, so a give-up is seen by the thread that
 * launched the kernel (and refuses that thread's next GEMM until cleared).
 * Readable at any time; clear != 0 resets it.  A kernel that gave up leaves
 * its output incomplete: check after synchronising. */
int  rplb_kernel_status(int clear);

/* Exercises the give-up path of the tensor-core kernels without a GEMM: one
 * warp waits about a millisecond on a barrier that nothing signals, gives up,
 * records its code and returns.  0 = the kernel returned, the status word held
 * the expected code and has been cleared.  Never blocks longer than the limit. */
int  rplb_selftest_bounded_wait(void* stream);
/* The same give-up, but its code (99) is left in the calling thread's status
 * word for rplb_kernel_status to find; synchronises the stream. */
int  rplb_selftest_bounded_wait_keep(void* stream);

/* Which contraction kernel the calling host thread's calls use: 0 = automatic (tcgen05
 * tensor-core kernel when the shape allows it, else the dp4a kernel),
 * 1 = dp4a kernel, 2 = tcgen05 kernel (RPLB_E_UNSUPPORTED if the shape does
 * not fit it), 3 = tcgen05 with one CTA per 128x256 tile, 4 = tcgen05 with a
 * CTA pair (cta_group::2) per 256x256 tile, 5 = tcgen05 with one CTA per
 * 256x256 tile (two accumulators), 6 = the tcgen05 kernel for few output
 * features (N <= 128, K <= 896, fp32 epilogue only; the automatic choice for
 * such layers over many rows); 0 and 2 pick between 3, 4, 5 and 6 by shape:
 * 5 for GEMMs of 1.1e12 multiply-accumulates and more with K >= 6144 (measured:
 * the most work per joule, and a long GEMM runs at the board's power limit;
 * its epilogue is not overlapped, so a short reduction does not pay), 4 for
 * GEMMs under 1.1e12 that give every SM pair a tile, 3 otherwise.  The sharded layer with
 * several ranks honours 3 and 5 (the kernels that can wait for arriving rows)
 * and chooses between them itself for any other value.
 * Returns the previous setting.  All of them are CUDA kernels. */
int  rplb_gemm_backend(int which);
/* How the tensor-core kernels of the calling thread store four-byte outputs:
 * 0 = 32 x 32 chunks through shared memory and a TMA tensor store when the
 * output's base and row stride are multiples of 16 bytes (else from registers),
 * 1 = always from registers, one row per thread.  Same values either way.
 * Returns the previous setting. */
int  rplb_gemm_epilogue(int which);

/* Number of kernels this library has launched in this process (all threads). */
uint64_t rplb_launch_count(void);

/* Output-column block of rank `rank` out of `world` when N columns are split
 * in multiples of `align`: begin and count in columns.  Host arithmetic only. */
int  rplb_shard_range(uint64_t n, int world, int rank, uint64_t align, uint64_t* begin, uint64_t* count);

/* ------------------------------------------------------------------------
 * The quantized Linear layer over the GPUs of one node, one process per GPU:
 * the multi-GPU form of tensor_quantize_int8_symmetric + linear_int8
 * (src/rpl_quantization.c:77-91, :314-353; the reference is single-device).
 * Output columns (weight rows) and activation rows are both split over the
 * ranks: rplb_sharded_linear_columns / _rows give this rank's blocks (columns
 * in multiples of 256, rows in multiples of 128, as rplb_shard_range deals
 * them).  forward takes this rank's fp32 rows, agrees on the per-tensor scale
 * with one max-all-reduce, quantizes the rows, sends them to the other ranks
 * over NVLink while the GEMM already runs on the local rows, and writes this
 * rank's column block of the fp32 output [rows, ldo].  Results are the bits a
 * single GPU produces.  NCCL is loaded at run time (libnccl.so.2, or the file
 * named by RPLB_NCCL_LIBRARY) and only when world > 1.
 *
 * create is a collective call: rank 0 obtains an id with rplb_nccl_unique_id
 * and hands the 128 bytes to the other ranks by any means (or every rank passes
 * an ncclComm_t it already has as nccl_comm); all ranks then call create with
 * the same world, max_rows, in_features and out_features_total.  weight_rows
 * [count, in_features], scales [count] and bias [count] (may be NULL) are this
 * rank's rows, in device memory, and stay the caller's.  With world > 1
 * in_features must be a multiple of 16.  forward, gather and free are
 * collective too (every rank calls them in the same order).  All calls on one
 * layer must be issued on one stream, or be ordered by the caller: the layer
 * owns one activation buffer, which a pass overwrites.  A layer is not meant to
 * be shared between host threads.
 * ---------------------------------------------------------------------- */
#define RPLB_NCCL_ID_BYTES 128
typedef struct rplb_sharded_linear rplb_sharded_linear;
int  rplb_nccl_unique_id(void* id);
int  rplb_sharded_linear_create(rplb_sharded_linear** layer, int rank, int world, const void* nccl_id, void* nccl_comm,
                                uint64_t max_rows, uint64_t in_features, uint64_t out_features_total,
                                const int8_t* weight_rows, const float* scales, const float* bias);
/* The same with the column blocks chosen by the caller: column_counts[r] columns for rank r, contiguous in
 * rank order, each a multiple of 256 (the last non-empty one may be ragged), adding up to out_features_total;
 * NULL = the even split.  The GPUs of a node do not sustain the same clock under their power cap; a split in
 * proportion to each GPU's measured speed lets all ranks finish together (rplb_shard_weighted computes one:
 * weights[r] = relative speed of rank r, e.g. 1 / its measured GEMM time; every rank must pass the same
 * numbers).  weight_rows / scales / bias are the rows of this rank's block under that split. */
int  rplb_sharded_linear_create_split(rplb_sharded_linear** layer, int rank, int world, const void* nccl_id, void* nccl_comm,
                                      uint64_t max_rows, uint64_t in_features, uint64_t out_features_total,
                                      const uint64_t* column_counts, const int8_t* weight_rows, const float* scales,
                                      const float* bias);
int  rplb_shard_weighted(uint64_t n, int world, uint64_t align, const double* weights, uint64_t* counts);
void rplb_sharded_linear_free(rplb_sharded_linear* layer);
int  rplb_sharded_linear_columns(const rplb_sharded_linear* layer, uint64_t* begin, uint64_t* count);
int  rplb_sharded_linear_rows(const rplb_sharded_linear* layer, uint64_t rows, uint64_t* begin, uint64_t* count);
/* x_local: this rank's rows of the [rows, in_features] activation, fp32, device.
 * out: this rank's [rows, count] column block, row stride ldo >= count, device. */
int  rplb_sharded_linear_forward(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, float* out, uint64_t ldo,
                                 int relu, void* stream);
/* forward in its two halves, for callers that want to put something between
 * them (a timing event, other work on the stream): quantize = scale agreement,
 * quantization of the local rows and the start of their transfer; gemm = the
 * contraction over all `rows` rows of the activation quantized last. */
int  rplb_sharded_linear_quantize(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, void* stream);
int  rplb_sharded_linear_gemm(rplb_sharded_linear* layer, uint64_t rows, float* out, uint64_t ldo, int relu, void* stream);
/* How a rank's int8 rows reach the other ranks: 0 (default) = one peer copy per destination by the copy engines,
 * nearest consumer first, no SM involved; 1 = a second quantize kernel on a side stream stores the packed rows
 * straight into every destination (plain stores over NVLink).  Same results; every rank must choose the same.
 * Measured on 2 B200s the copy engines are the faster route (the kernel takes SM time from the GEMM and
 * reads the fp32 rows a second time), so they are the default. */
int  rplb_sharded_linear_transfer(rplb_sharded_linear* layer, int which);
/* After a forward: the whole int8 activation [rows, in_features] as this rank
 * holds it, and its scale (one device float).  Both stay the layer's. */
int  rplb_sharded_linear_activation(const rplb_sharded_linear* layer, const int8_t** xq, const float** scale);
/* The whole [rows, out_features_total] fp32 matrix on every rank from the
 * column blocks (row stride ld): ncclAllGather plus an unpack pass. */
int  rplb_sharded_linear_gather(rplb_sharded_linear* layer, const float* block, uint64_t ld, uint64_t rows, float* full,
                                void* stream);
/* forward on host buffers, enqueued and pipelined like
 * quantized_linear_submit_host: x_local (this rank's rows) and out (this rank's
 * [rows, count] block, row stride count) in host memory, page-locked for full
 * PCIe speed.  Every rank uploads only its own rows.  The GEMM runs in
 * row_blocks blocks (0 = 8), each downloaded while the next computes; the
 * upload of call n+1 overlaps the download of call n.  drain waits for all
 * queued calls of this rank. */
int  rplb_sharded_linear_submit_host(rplb_sharded_linear* layer, const float* x_local, uint64_t rows, float* out, int relu,
                                     int row_blocks, void* compute_stream);
int  rplb_sharded_linear_drain(rplb_sharded_linear* layer);

/* ------------------------------------------------------------------------
 * The reference's exported names for the path.  Same signatures, ownership
 * and struct layouts; data pointers may be host or device pointers.
 * ---------------------------------------------------------------------- */
/* include/rpl.h:99-102, src/rpl_core.c:33-77 */
Tensor* tensor_create(uint32_t dims, const uint32_t* shape, bool requires_grad);
void    tensor_free(Tensor* t);
void*   rpitorch_aligned_alloc(size_t alignment, size_t size);
void    rpitorch_aligned_free(void* ptr);

/* include/rpl.h:105-108, src/rpl_gpu.c:88-229 (the reference's accelerator
 * hooks).  rpl_gpu_init reports whether a CUDA device is present.
 * tensor_to_gpu gives the tensor a mirror in device memory, named by
 * Tensor.gpu_buffer, and sets Tensor.device = DEVICE_GPU; the host block
 * stays.  Every entry point below that takes a Tensor then works on the
 * mirror and returns device-resident results.  tensor_from_gpu copies the
 * mirror back into the host block (the tensor stays mirrored, as in the
 * reference); tensor_free releases the mirror.  rpl_gpu_shutdown frees the
 * calling thread's staging buffers. */
bool    rpl_gpu_init(void);
void    rpl_gpu_shutdown(void);
void    tensor_to_gpu(Tensor* t);
void    tensor_from_gpu(Tensor* t);

/* include/rpl.h:176, src/rpl_core.c:511-530 */
QuantizedTensor* tensor_quantize_int8(const Tensor* input, float scale, int32_t zero_point);
/* include/rpl.h:177, src/ops_extended.c:75-80 */
void    quantized_tensor_free(QuantizedTensor* qt);
/* include/rpl.h:178, src/ops_extended.c:52-61 */
void    tensor_get_min_max(const Tensor* t, float* min_val, float* max_val);
/* include/rpl.h:186, src/ops_extended.c:64-73 */
Tensor* tensor_dequantize_int8(QuantizedTensor* input);
/* include/rpl.h:187, src/ops_extended.c:124-129 and :83-123 */
void    gemm_int8(const int8_t* A, const int8_t* B, int32_t* C, uint32_t M, uint32_t N, uint32_t K,
                  float scale_a, float scale_b, float scale_c, int32_t zero_point_a, int32_t zero_point_b);
void    gemm_int8_fallback(const int8_t* A, const int8_t* B, int32_t* C, uint32_t M, uint32_t N, uint32_t K,
                           float scale_a, float scale_b, float scale_c, int32_t zero_point_a, int32_t zero_point_b);

/* Exported by the reference library but absent from its header. */
/* src/rpl_quantization.c:77-91 */
QuantizedTensor* tensor_quantize_int8_symmetric(const Tensor* input);
/* src/rpl_quantization.c:93-107 */
QuantizedTensor* tensor_quantize_int8_asymmetric(const Tensor* input);
/* src/rpl_quantization.c:120-160; channel_axis only selects num_channels = shape[axis] */
PerChannelQuantizedTensor* tensor_quantize_per_channel(const Tensor* input, uint32_t channel_axis);
/* src/rpl_quantization.c:162-168 */
void    per_channel_quantized_tensor_free(PerChannelQuantizedTensor* qt);
/* src/rpl_quantization.c:314-353; only ->data of the three tensors is read */
void    linear_int8(const QuantizedTensor* input, const QuantizedTensor* weight, const QuantizedTensor* bias,
                    int32_t* output, uint32_t batch_size, uint32_t in_features, uint32_t out_features);
/* src/rpl_quantization.c:26-71 */
QuantizationCalibrator* calibrator_create(void);
void    calibrator_update(QuantizationCalibrator* cal, const Tensor* t);
void    calibrator_compute_params(QuantizationCalibrator* cal, bool symmetric);
void    calibrator_free(QuantizationCalibrator* cal);
/* src/rpl_quantization.c:278-307 (per_channel is accepted and ignored, as there) */
QuantizedModel* model_quantize(Tensor** parameters, uint32_t num_params, bool per_channel);
void    quantized_model_free(QuantizedModel* qm);
/* What model_quantize's per_channel flag announces and the reference leaves as
 * a TODO (src/rpl_quantization.c:286-292); model_quantize itself keeps ignoring
 * the flag, as the reference does.  Parameters with dims >= 2 are quantized per
 * row of shape[0] (tensor_quantize_per_channel, axis 0), the others with one
 * scale for the whole tensor (a single channel). */
typedef struct {
    Tensor**                    fp32_params;
    PerChannelQuantizedTensor** int8_params;
    uint32_t                    num_params;
    bool                        is_quantized;
} PerChannelQuantizedModel;
PerChannelQuantizedModel* model_quantize_per_channel(Tensor** parameters, uint32_t num_params);
void    per_channel_quantized_model_free(PerChannelQuantizedModel* qm);
/* include/rpl.h:123, src/rpl_core.c:223-262 (ReLU between quantized layers) */
void    tensor_relu_inplace(Tensor* t);

/* ------------------------------------------------------------------------
 * Additions in the reference's style (no counterpart there).
 * ---------------------------------------------------------------------- */
/* Last failure of a reference-named call on this thread: 0 or an RPLB_E_* /
 * cudaError_t value.  Those calls cannot return errors through their
 * signatures; like the reference's accelerator file they print one line to
 * stderr and return (NULL for producers). */
int     rpl_cuda_last_error(void);

/* A Tensor whose data lives in device memory (device = DEVICE_GPU); release
 * with tensor_free.  tensor_upload copies a host tensor to a new device one,
 * tensor_download the other way. */
Tensor* tensor_create_device(uint32_t dims, const uint32_t* shape);
Tensor* tensor_upload(const Tensor* host);
Tensor* tensor_download(const Tensor* dev);

/* out[m,n] = relu?( ((float)acc * x->scale) * w->scales[n] + bias[n] ) with acc
 * as linear_int8 computes it: x [batch, in], w [out, in] quantized per output
 * row, bias fp32 [out] or NULL, out fp32 [batch, out].  Pointers host or
 * device, each on its own. */
void    linear_int8_dequant(const QuantizedTensor* x, const PerChannelQuantizedTensor* w, const float* bias,
                            float* out, uint32_t batch_size, uint32_t in_features, uint32_t out_features,
                            bool relu);

/* A quantized Linear layer, the INT8 counterpart of linear_create /
 * linear_forward / linear_free (include/rpl.h:230-232, src/rpl_nn.c:23-82):
 * y = x . W^T + b with W [out_features, in_features].  create quantizes the fp32
 * weight per output row (tensor_quantize_per_channel) and keeps it, its scales
 * and the fp32 bias (may be NULL) in device memory; forward quantizes the
 * activation per tensor (symmetric) and runs the INT8 GEMM with the fused
 * dequantize + bias (+ ReLU) epilogue.  The result is a new Tensor
 * [rows, out_features], in device memory if the input was, else in host memory. */
typedef struct QuantizedLinear QuantizedLinear;
QuantizedLinear* quantized_linear_create(const Tensor* weight, const Tensor* bias);
Tensor* quantized_linear_forward(QuantizedLinear* layer, const Tensor* input, bool relu);
/* Several layers over one input, as multi-head attention applies W_q, W_k, W_v
 * to the same activation (src/rpl_attention.c:175-177): the activation is
 * quantized once and every layer's GEMM reads that int8 copy.  All layers must
 * have the same in_features.  outputs[i] receives a new Tensor
 * [rows, out_features of layer i]; returns 0, or an error code with every
 * outputs[i] NULL. */
int     quantized_linear_forward_shared_input(QuantizedLinear* const* layers, uint32_t num_layers, const Tensor* input,
                                              Tensor** outputs, bool relu);
void    quantized_linear_free(QuantizedLinear* layer);
/* A layer over int8 weight rows [out,in], per-row scales and an optional fp32 bias
 * that already live in device memory and remain the caller's. */
QuantizedLinear* quantized_linear_wrap(const int8_t* weight_rows, const float* scales, const float* bias,
                                       uint32_t in_features, uint32_t out_features);
/* The same forward pass on host buffers, enqueued and pipelined: x [rows, in] and out
 * [rows, out] in host memory (page-locked for full PCIe speed).  submit returns once
 * the call is queued, drain waits for every queued call.  Inputs and outputs are
 * double-buffered on the device, so the upload of call n+1 overlaps the compute and
 * download of call n, and each row block of a call is downloaded while the next is in
 * the GEMM.  compute_stream (a cudaStream_t, may be NULL) is where quantize and GEMM
 * run; after drain it has also waited for the downloads.  Both return 0 or an error code. */
int     quantized_linear_submit_host(QuantizedLinear* layer, const float* x, uint32_t rows, float* out, bool relu,
                                     void* compute_stream);
int     quantized_linear_drain(QuantizedLinear* layer);

/* Quantized weights on disk, in the framing of the reference's fp32 checkpoint
 * writer (checkpoint_save_model, src/rpl_training.c:915-944; the reference has
 * no loader and no int8 format): header {count, tag "INT8", 0.0f}, then per
 * tensor dims, shape[dims], size, int8 data[size], num_channels, fp32
 * scales[num_channels].  save returns 0 on success; load returns a malloc'ed
 * array of *num_tensors tensors in host memory, or in device memory when
 * to_device is true (NULL on error). */
int     quantized_weights_save(const char* path, PerChannelQuantizedTensor* const* tensors, uint32_t num_tensors);
PerChannelQuantizedTensor** quantized_weights_load(const char* path, uint32_t* num_tensors, bool to_device);

/* out = (float)q * scales[channel], a new fp32 Tensor shaped like the input. */
Tensor* tensor_dequantize_per_channel(const PerChannelQuantizedTensor* input);

#ifdef __cplusplus
}
#endif
#endif /* RPL_B200_H */
