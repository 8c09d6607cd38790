/*
 * The reference's C API for the INT8 path, on top of the rplb_* device layer.
 *
 * Plain C, no CUDA headers: everything that touches the GPU goes through
 * rpl_b200.h.  Each entry point keeps the reference's signature, allocation
 * and ownership rules; the loops of the reference are replaced by kernel
 * launches.  A data pointer may be ordinary host memory (staged through device
 * buffers kept per thread), page-locked host memory (same, at full PCIe
 * speed), or device / managed memory (used in place; results are then left in
 * device memory too).
 *
 * Failures cannot be returned through these signatures.  Like the reference's
 * accelerator file (src/rpl_gpu.c:95-111) a failing call prints one line to
 * stderr; producers return NULL (the convention of tensor_create,
 * src/rpl_core.c:45), void functions leave their outputs untouched, and
 * rpl_cuda_last_error() holds the code.  There is no CPU fallback.
 */
#define _POSIX_C_SOURCE 200809L
#include "rpl_b200.h"
#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int rplb_kernel_status(int clear);
int rplb_relu_f32_inplace(float* x, uint64_t n, void* stream);

#if defined(RPL_B200_OWN_TYPES)
_Static_assert(sizeof(Tensor) == 152, "Tensor layout differs from the reference");
_Static_assert(offsetof(Tensor, size) == 84, "Tensor.size offset");
_Static_assert(offsetof(Tensor, _allocation) == 96, "Tensor._allocation offset");
_Static_assert(offsetof(Tensor, device) == 112, "Tensor.device offset");
_Static_assert(offsetof(Tensor, gpu_buffer) == 116, "Tensor.gpu_buffer offset");
_Static_assert(offsetof(Tensor, is_leaf) == 120, "Tensor.is_leaf offset");
_Static_assert(offsetof(Tensor, backward_fn) == 144, "Tensor.backward_fn offset");
_Static_assert(sizeof(QuantizedTensor) == 56, "QuantizedTensor layout differs from the reference");
_Static_assert(offsetof(QuantizedTensor, scale) == 8, "QuantizedTensor.scale offset");
_Static_assert(offsetof(QuantizedTensor, shape) == 24, "QuantizedTensor.shape offset");
#endif

static __thread int t_last_error = 0;

static int report(int rc, const char* where) {
    if (rc != 0) {
        t_last_error = rc;
        fprintf(stderr, "rpl (cuda): %s failed: %s [%d]\n", where, rplb_last_error(), rc);
    }
    return rc;
}

int rpl_cuda_last_error(void) { return t_last_error; }

/* Waits for the default stream and picks up a kernel-side give-up, if any. */
static int finish(const char* where) {
    int rc = rplb_stream_sync(NULL);
    if (rc == 0) {
        int st = rplb_kernel_status(1);
        if (st != 0) {
            t_last_error = RPLB_E_KERNEL;
            fprintf(stderr, "rpl (cuda): %s: a kernel gave up waiting (code %d)\n", where, st);
            return RPLB_E_KERNEL;
        }
        return 0;
    }
    return report(rc, where);
}

static int on_device(const void* p) { return rplb_pointer_kind(p) >= 2; }

/* ------------------------------------------------------------------------
 * Per-thread device staging buffers for host-resident arguments (grow-only).
 * ---------------------------------------------------------------------- */
#define STAGE_SLOTS 4
static __thread void*  t_stage[STAGE_SLOTS];
static __thread size_t t_stage_cap[STAGE_SLOTS];

static void* stage(int slot, size_t bytes) {
    if (bytes == 0) bytes = 16;
    if (t_stage_cap[slot] < bytes) {
        if (t_stage[slot]) { rplb_stream_sync(NULL); rplb_free(t_stage[slot]); }
        t_stage[slot] = NULL;
        t_stage_cap[slot] = 0;
        if (report(rplb_malloc(&t_stage[slot], bytes), "staging allocation") != 0) return NULL;
        t_stage_cap[slot] = bytes;
    }
    return t_stage[slot];
}

/* Device view of a read-only argument: the pointer itself when it is device
 * memory, else a staged copy. */
static const void* to_device(int slot, const void* p, size_t bytes) {
    if (p == NULL) return NULL;
    if (on_device(p)) return p;
    void* d = stage(slot, bytes);
    if (!d) return NULL;
    if (report(rplb_copy(d, p, bytes, NULL), "host to device copy") != 0) return NULL;
    return d;
}

/* ------------------------------------------------------------------------
 * Device mirrors: include/rpl.h:105-108, src/rpl_gpu.c:88-229.
 *
 * The reference's accelerator keeps a Tensor's host block and adds a buffer
 * object named by the 32-bit Tensor.gpu_buffer.  Here that field indexes a
 * table of device blocks; every entry point that takes a Tensor works on the
 * mirror when there is one, and then leaves its results in device memory.
 * ---------------------------------------------------------------------- */
#define MIRROR_MAX 65536u
static pthread_mutex_t g_mirror_mu = PTHREAD_MUTEX_INITIALIZER;
static void*    g_mirror[MIRROR_MAX];          /* handle h lives in g_mirror[h - 1] */
static uint32_t g_mirror_hint = 0;

static void* mirror_of(const Tensor* t) {
    if (t->device != DEVICE_GPU || t->gpu_buffer == 0 || t->gpu_buffer > MIRROR_MAX) return NULL;
    pthread_mutex_lock(&g_mirror_mu);
    void* d = g_mirror[t->gpu_buffer - 1];
    pthread_mutex_unlock(&g_mirror_mu);
    return d;
}

/* Where the tensor's elements are to be read or written by the device. */
static float* tensor_data(const Tensor* t) {
    void* d = mirror_of(t);
    return d ? (float*)d : t->data;
}

static void mirror_release(Tensor* t) {
    if (t->device != DEVICE_GPU || t->gpu_buffer == 0 || t->gpu_buffer > MIRROR_MAX) return;
    pthread_mutex_lock(&g_mirror_mu);
    void* d = g_mirror[t->gpu_buffer - 1];
    g_mirror[t->gpu_buffer - 1] = NULL;
    pthread_mutex_unlock(&g_mirror_mu);
    if (d) rplb_free(d);
    t->gpu_buffer = 0;
    t->device = DEVICE_CPU;
}

bool rpl_gpu_init(void) { return rplb_device_count() > 0; }

/* Releases the calling thread's staging buffers.  Mirrors belong to their
 * tensors and go with tensor_free. */
void rpl_gpu_shutdown(void) {
    rplb_stream_sync(NULL);
    for (int i = 0; i < STAGE_SLOTS; i++) {
        if (t_stage[i]) rplb_free(t_stage[i]);
        t_stage[i] = NULL;
        t_stage_cap[i] = 0;
    }
}

void tensor_to_gpu(Tensor* t) {
    if (!t) return;
    if (t->device == DEVICE_GPU) return;                 /* mirrored already, or born in device memory */
    t_last_error = 0;
    const size_t bytes = (size_t)t->size * sizeof(float);
    void* d = NULL;
    if (report(rplb_malloc(&d, bytes), "tensor_to_gpu") != 0) return;
    if (report(rplb_copy(d, t->data, bytes, NULL), "tensor_to_gpu") != 0 || finish("tensor_to_gpu") != 0) {
        rplb_free(d);
        return;
    }
    uint32_t h = 0;
    pthread_mutex_lock(&g_mirror_mu);
    for (uint32_t i = 0; i < MIRROR_MAX; i++) {
        uint32_t slot = (g_mirror_hint + i) % MIRROR_MAX;
        if (!g_mirror[slot]) { g_mirror[slot] = d; h = slot + 1; g_mirror_hint = slot + 1; break; }
    }
    pthread_mutex_unlock(&g_mirror_mu);
    if (h == 0) {
        rplb_free(d);
        t_last_error = RPLB_E_TOO_LARGE;
        fprintf(stderr, "rpl (cuda): tensor_to_gpu failed: %u tensors are mirrored already\n", MIRROR_MAX);
        return;
    }
    t->gpu_buffer = h;
    t->device = DEVICE_GPU;
}

/* Copies the mirror back into the host block; the tensor stays mirrored, as
 * in the reference (src/rpl_gpu.c:217-229). */
void tensor_from_gpu(Tensor* t) {
    if (!t || t->device == DEVICE_CPU) return;
    void* d = mirror_of(t);
    if (!d) return;                                      /* born in device memory: no host block to fill */
    t_last_error = 0;
    if (report(rplb_copy(t->data, d, (size_t)t->size * sizeof(float), NULL), "tensor_from_gpu") != 0) return;
    finish("tensor_from_gpu");
}

/* ------------------------------------------------------------------------
 * Allocation glue: src/rpl_core.c:33-77.
 * ---------------------------------------------------------------------- */
void* rpitorch_aligned_alloc(size_t alignment, size_t size) {
    void* p = NULL;
    if (posix_memalign(&p, alignment, size) != 0) return NULL;
    return p;
}

/* Releases host blocks with free() as the reference does, and blocks that
 * this library placed in device memory with the device allocator. */
void rpitorch_aligned_free(void* ptr) {
    if (!ptr) return;
    if (on_device(ptr)) rplb_free(ptr);
    else free(ptr);
}

static void fill_shape(Tensor* t, uint32_t dims, const uint32_t* shape) {
    t->dims = dims;
    t->size = 1;
    for (uint32_t i = 0; i < dims; i++) { t->shape[i] = shape[i]; t->size *= shape[i]; }
    if (dims) {
        t->strides[dims - 1] = 1;
        for (int i = (int)dims - 2; i >= 0; i--) t->strides[i] = t->strides[i + 1] * t->shape[i + 1];
    }
}

Tensor* tensor_create(uint32_t dims, const uint32_t* shape, bool requires_grad) {
    Tensor* t = (Tensor*)calloc(1, sizeof(Tensor));
    if (!t) return NULL;
    fill_shape(t, dims, shape);
    size_t bytes = (size_t)t->size * sizeof(float);
    t->_allocation = rpitorch_aligned_alloc(64, bytes);
    t->_alloc_size = bytes;
    t->data = (float*)t->_allocation;
    if (requires_grad) {
        t->grad = (float*)rpitorch_aligned_alloc(64, bytes);
        if (t->grad) memset(t->grad, 0, bytes);
    }
    t->requires_grad = requires_grad;
    t->is_leaf = true;
    return t;
}

Tensor* tensor_create_device(uint32_t dims, const uint32_t* shape) {
    Tensor* t = (Tensor*)calloc(1, sizeof(Tensor));
    if (!t) return NULL;
    fill_shape(t, dims, shape);
    size_t bytes = (size_t)t->size * sizeof(float);
    void* d = NULL;
    if (report(rplb_malloc(&d, bytes), "tensor_create_device") != 0) { free(t); return NULL; }
    t->_allocation = d;
    t->_alloc_size = bytes;
    t->data = (float*)d;
    t->device = DEVICE_GPU;
    t->is_leaf = true;
    return t;
}

void tensor_free(Tensor* t) {
    if (!t) return;
    mirror_release(t);
    if (t->_allocation) rpitorch_aligned_free(t->_allocation);
    if (t->grad) rpitorch_aligned_free(t->grad);
    free(t);
}

Tensor* tensor_upload(const Tensor* host) {
    if (!host) return NULL;
    Tensor* d = tensor_create_device(host->dims, host->shape);
    if (!d) return NULL;
    if (report(rplb_copy(d->data, host->data, (size_t)host->size * 4, NULL), "tensor_upload") != 0 ||
        finish("tensor_upload") != 0) { tensor_free(d); return NULL; }
    return d;
}

Tensor* tensor_download(const Tensor* dev) {
    if (!dev) return NULL;
    Tensor* h = tensor_create(dev->dims, dev->shape, false);
    if (!h) return NULL;
    if (report(rplb_copy(h->data, tensor_data(dev), (size_t)dev->size * 4, NULL), "tensor_download") != 0 ||
        finish("tensor_download") != 0) { tensor_free(h); return NULL; }
    return h;
}

/* ------------------------------------------------------------------------
 * Quantize / dequantize.
 * ---------------------------------------------------------------------- */
static QuantizedTensor* new_qt_like(const Tensor* input) {
    QuantizedTensor* qt = (QuantizedTensor*)malloc(sizeof(QuantizedTensor));
    if (!qt) return NULL;
    memset(qt, 0, sizeof(*qt));
    qt->size = input->size;
    qt->dims = input->dims;
    memcpy(qt->shape, input->shape, input->dims * sizeof(uint32_t));
    return qt;
}

/* Shared body of the three per-tensor quantizers.
 * how: 0 = caller's scale and zero point, 1 = symmetric, 2 = asymmetric. */
static QuantizedTensor* quantize_common(const Tensor* input, int how, float scale, int32_t zp, const char* who) {
    if (!input) return NULL;
    t_last_error = 0;
    const size_t n = input->size;
    const float* src = tensor_data(input);
    const int dev_in = on_device(src);
    QuantizedTensor* qt = new_qt_like(input);
    if (!qt) return NULL;

    const float* x = (const float*)to_device(0, src, n * 4);
    int8_t* q_dev = NULL;
    void* own_q = NULL;
    if (dev_in) {
        if (report(rplb_malloc(&own_q, n), who) != 0) { free(qt); return NULL; }
        q_dev = (int8_t*)own_q;
    } else {
        q_dev = (int8_t*)stage(1, n);
    }
    rplb_qparams* params = (rplb_qparams*)stage(2, sizeof(rplb_qparams));
    if ((n && !x) || !q_dev || !params) { rplb_free(own_q); free(qt); return NULL; }

    int rc;
    if (how == 1)      rc = rplb_quantize_symmetric_f32_i8(x, q_dev, n, params, NULL);
    else if (how == 2) rc = rplb_quantize_asymmetric_f32_i8(x, q_dev, n, params, NULL);
    else               rc = rplb_quantize_f32_i8(x, q_dev, n, scale, zp, NULL);
    if (report(rc, who) != 0) { rplb_free(own_q); free(qt); return NULL; }

    rplb_qparams hp;
    memset(&hp, 0, sizeof(hp));
    if (how != 0 && report(rplb_copy(&hp, params, sizeof(hp), NULL), who) != 0) { rplb_free(own_q); free(qt); return NULL; }
    if (dev_in) {
        qt->data = q_dev;
    } else {
        qt->data = (int8_t*)rpitorch_aligned_alloc(64, n ? n : 1);
        if (!qt->data || report(rplb_copy(qt->data, q_dev, n, NULL), who) != 0) { free(qt->data); free(qt); return NULL; }
    }
    if (finish(who) != 0) { rpitorch_aligned_free(qt->data); free(qt); return NULL; }
    if (how == 1)      { qt->scale = hp.scale_sym;  qt->zero_point = 0; }
    else if (how == 2) { qt->scale = hp.scale_asym; qt->zero_point = hp.zp_asym; }
    else               { qt->scale = scale;         qt->zero_point = zp; }
    return qt;
}

QuantizedTensor* tensor_quantize_int8(const Tensor* input, float scale, int32_t zero_point) {
    return quantize_common(input, 0, scale, zero_point, "tensor_quantize_int8");
}

QuantizedTensor* tensor_quantize_int8_symmetric(const Tensor* input) {
    return quantize_common(input, 1, 0.0f, 0, "tensor_quantize_int8_symmetric");
}

QuantizedTensor* tensor_quantize_int8_asymmetric(const Tensor* input) {
    return quantize_common(input, 2, 0.0f, 0, "tensor_quantize_int8_asymmetric");
}

void quantized_tensor_free(QuantizedTensor* qt) {
    if (!qt) return;
    if (qt->data) rpitorch_aligned_free(qt->data);
    free(qt);
}

/* min/max of the device reduction, fetched to the host. */
static int minmax_to_host(const Tensor* t, rplb_qparams* hp, const char* who) {
    const size_t n = t->size;
    const float* x = (const float*)to_device(0, tensor_data(t), n * 4);
    rplb_qparams* params = (rplb_qparams*)stage(2, sizeof(rplb_qparams));
    if ((n && !x) || !params) return -1;
    if (report(rplb_minmax_f32(x, n, params, NULL), who) != 0) return -1;
    if (report(rplb_copy(hp, params, sizeof(*hp), NULL), who) != 0) return -1;
    return finish(who);
}

void tensor_get_min_max(const Tensor* t, float* min_val, float* max_val) {
    if (!t || t->size == 0) return;                      /* src/ops_extended.c:53 */
    t_last_error = 0;
    rplb_qparams hp;
    if (minmax_to_host(t, &hp, "tensor_get_min_max") != 0) return;
    if (isnan(hp.first)) {
        /* The reference seeds both results with data[0]; no compare against a NaN succeeds. */
        *min_val = hp.first;
        *max_val = hp.first;
    } else {
        *min_val = hp.true_min;
        *max_val = hp.true_max;
    }
}

Tensor* tensor_dequantize_int8(QuantizedTensor* input) {
    if (!input) return NULL;
    t_last_error = 0;
    const size_t n = input->size;
    const int dev_in = on_device(input->data);
    Tensor* out = dev_in ? tensor_create_device(input->dims, input->shape)
                         : tensor_create(input->dims, input->shape, false);
    if (!out) return NULL;
    const int8_t* q = (const int8_t*)to_device(0, input->data, n);
    float* o_dev = dev_in ? out->data : (float*)stage(1, n * 4);
    if ((n && !q) || !o_dev) { tensor_free(out); return NULL; }
    if (report(rplb_dequantize_i8_f32(q, o_dev, n, input->scale, input->zero_point, NULL), "tensor_dequantize_int8") != 0) {
        tensor_free(out);
        return NULL;
    }
    if (!dev_in && report(rplb_copy(out->data, o_dev, n * 4, NULL), "tensor_dequantize_int8") != 0) { tensor_free(out); return NULL; }
    if (finish("tensor_dequantize_int8") != 0) { tensor_free(out); return NULL; }
    return out;
}

PerChannelQuantizedTensor* tensor_quantize_per_channel(const Tensor* input, uint32_t channel_axis) {
    if (!input || channel_axis >= MAX_DIMS) return NULL;
    t_last_error = 0;
    PerChannelQuantizedTensor* qt = (PerChannelQuantizedTensor*)calloc(1, sizeof(PerChannelQuantizedTensor));
    if (!qt) return NULL;
    /* src/rpl_quantization.c:124-127: the axis only supplies the channel count. */
    qt->num_channels = input->shape[channel_axis];
    qt->channel_size = qt->num_channels ? input->size / qt->num_channels : 0;
    qt->dims = input->dims;
    memcpy(qt->shape, input->shape, input->dims * sizeof(uint32_t));
    const size_t n = input->size, C = qt->num_channels;
    const float* src = tensor_data(input);
    const int dev_in = on_device(src);
    const char* who = "tensor_quantize_per_channel";

    const float* x = (const float*)to_device(0, src, n * 4);
    void *q_dev = NULL, *s_dev = NULL, *z_dev = NULL;
    if (dev_in) {
        if (report(rplb_malloc(&q_dev, n), who) || report(rplb_malloc(&s_dev, C * 4), who) || report(rplb_malloc(&z_dev, C * 4), who)) goto fail;
    } else {
        q_dev = stage(1, n);
        s_dev = stage(2, C * 4);
        z_dev = stage(3, C * 4);
    }
    if ((n && !x) || !q_dev || !s_dev || !z_dev) goto fail;
    if (report(rplb_quantize_per_channel_f32_i8(x, (int8_t*)q_dev, (float*)s_dev, (int32_t*)z_dev, C, qt->channel_size, NULL), who)) goto fail;
    if (dev_in) {
        qt->data = (int8_t*)q_dev; qt->scales = (float*)s_dev; qt->zero_points = (int32_t*)z_dev;
        q_dev = s_dev = z_dev = NULL;
    } else {
        qt->data = (int8_t*)rpitorch_aligned_alloc(64, n ? n : 1);
        qt->scales = (float*)malloc(C ? C * 4 : 4);
        qt->zero_points = (int32_t*)malloc(C ? C * 4 : 4);
        if (!qt->data || !qt->scales || !qt->zero_points) goto fail;
        if (report(rplb_copy(qt->data, q_dev, n, NULL), who) || report(rplb_copy(qt->scales, s_dev, C * 4, NULL), who) ||
            report(rplb_copy(qt->zero_points, z_dev, C * 4, NULL), who)) goto fail;
        q_dev = s_dev = z_dev = NULL;
    }
    if (finish(who) != 0) goto fail;
    return qt;
fail:
    if (dev_in) { rplb_free(q_dev); rplb_free(s_dev); rplb_free(z_dev); }
    per_channel_quantized_tensor_free(qt);
    return NULL;
}

void per_channel_quantized_tensor_free(PerChannelQuantizedTensor* qt) {
    if (!qt) return;
    rpitorch_aligned_free(qt->data);
    rpitorch_aligned_free(qt->scales);
    rpitorch_aligned_free(qt->zero_points);
    free(qt);
}

Tensor* tensor_dequantize_per_channel(const PerChannelQuantizedTensor* input) {
    if (!input) return NULL;
    t_last_error = 0;
    const size_t C = input->num_channels, L = input->channel_size, n = C * L;
    const int dev_in = on_device(input->data);
    const char* who = "tensor_dequantize_per_channel";
    Tensor* out = dev_in ? tensor_create_device(input->dims, input->shape)
                         : tensor_create(input->dims, input->shape, false);
    if (!out) return NULL;
    const int8_t* q = (const int8_t*)to_device(0, input->data, n);
    const float* s = (const float*)to_device(2, input->scales, C * 4);
    float* o_dev = dev_in ? out->data : (float*)stage(1, n * 4);
    if ((n && (!q || !s)) || !o_dev) { tensor_free(out); return NULL; }
    if (report(rplb_dequantize_per_channel_i8_f32(q, s, o_dev, C, L, NULL), who) != 0) { tensor_free(out); return NULL; }
    if (!dev_in && report(rplb_copy(out->data, o_dev, n * 4, NULL), who) != 0) { tensor_free(out); return NULL; }
    if (finish(who) != 0) { tensor_free(out); return NULL; }
    return out;
}

/* ------------------------------------------------------------------------
 * INT8 contraction.
 * ---------------------------------------------------------------------- */
/* src/rpl_quantization.c:314-353: reads only ->data of its three tensors and
 * writes raw int32 sums into the caller's buffer. */
void linear_int8(const QuantizedTensor* input, const QuantizedTensor* weight, const QuantizedTensor* bias,
                 int32_t* output, uint32_t batch_size, uint32_t in_features, uint32_t out_features) {
    if (!input || !weight || !output) return;
    t_last_error = 0;
    const char* who = "linear_int8";
    const size_t M = batch_size, K = in_features, N = out_features;
    if (M == 0 || N == 0) return;
    const int8_t* x = (const int8_t*)to_device(0, input->data, M * K);
    const int8_t* w = (const int8_t*)to_device(1, weight->data, N * K);
    const int8_t* b = bias ? (const int8_t*)to_device(2, bias->data, N) : NULL;
    const int out_dev = on_device(output);
    int32_t* o = out_dev ? output : (int32_t*)stage(3, M * N * 4);
    if ((K && (!x || !w)) || (bias && !b) || !o) return;
    if (report(rplb_linear_i8_i32(x, w, b, o, M, K, N, NULL), who) != 0) return;
    if (!out_dev && report(rplb_copy(output, o, M * N * 4, NULL), who) != 0) return;
    finish(who);
}

/* src/ops_extended.c:83-123, scalar branch. */
void gemm_int8_fallback(const int8_t* A, const int8_t* B, int32_t* C, uint32_t M, uint32_t N, uint32_t K,
                        float scale_a, float scale_b, float scale_c, int32_t zero_point_a, int32_t zero_point_b) {
    if (!A || !B || !C) return;
    t_last_error = 0;
    const char* who = "gemm_int8";
    const size_t m = M, n = N, k = K;
    if (m == 0 || n == 0) return;
    const int8_t* a = (const int8_t*)to_device(0, A, m * k);
    const int8_t* b = (const int8_t*)to_device(1, B, k * n);
    const int out_dev = on_device(C);
    int32_t* c = out_dev ? C : (int32_t*)stage(3, m * n * 4);
    if ((k && (!a || !b)) || !c) return;
    if (report(rplb_gemm_i8_requant_i32(a, b, c, m, n, k, scale_a, scale_b, scale_c, zero_point_a, zero_point_b, NULL), who) != 0) return;
    if (!out_dev && report(rplb_copy(C, c, m * n * 4, NULL), who) != 0) return;
    finish(who);
}

/* src/ops_extended.c:124-129 */
void gemm_int8(const int8_t* A, const int8_t* B, int32_t* C, uint32_t M, uint32_t N, uint32_t K,
               float scale_a, float scale_b, float scale_c, int32_t zero_point_a, int32_t zero_point_b) {
    gemm_int8_fallback(A, B, C, M, N, K, scale_a, scale_b, scale_c, zero_point_a, zero_point_b);
}

void linear_int8_dequant(const QuantizedTensor* x, const PerChannelQuantizedTensor* w, const float* bias,
                         float* out, uint32_t batch_size, uint32_t in_features, uint32_t out_features, bool relu) {
    if (!x || !w || !out) return;
    t_last_error = 0;
    const char* who = "linear_int8_dequant";
    const size_t M = batch_size, K = in_features, N = out_features;
    if (M == 0 || N == 0) return;
    /* Scales and bias travel in one small staged block: [a_scale | w_scales[N] | bias[N]]. */
    float* small = (float*)stage(2, (1 + 2 * N) * 4);
    if (!small) return;
    if (report(rplb_copy(small, &x->scale, 4, NULL), who) != 0) return;
    if (report(rplb_copy(small + 1, w->scales, N * 4, NULL), who) != 0) return;
    if (bias && report(rplb_copy(small + 1 + N, bias, N * 4, NULL), who) != 0) return;
    const int8_t* xd = (const int8_t*)to_device(0, x->data, M * K);
    const int8_t* wd = (const int8_t*)to_device(1, w->data, N * K);
    const int out_dev = on_device(out);
    float* o = out_dev ? out : (float*)stage(3, M * N * 4);
    if ((K && (!xd || !wd)) || !o) return;
    if (report(rplb_linear_i8_dequant_f32(xd, wd, o, M, K, N, N, small, small + 1, bias ? small + 1 + N : NULL,
                                          relu ? 1 : 0, NULL), who) != 0) return;
    if (!out_dev && report(rplb_copy(out, o, M * N * 4, NULL), who) != 0) return;
    finish(who);
}

/* src/rpl_core.c:223-262 */
void tensor_relu_inplace(Tensor* t) {
    if (!t || t->size == 0) return;
    t_last_error = 0;
    const char* who = "tensor_relu_inplace";
    const size_t n = t->size;
    float* resident = tensor_data(t);
    if (on_device(resident)) {
        if (report(rplb_relu_f32_inplace(resident, n, NULL), who) == 0) finish(who);
        return;
    }
    float* d = (float*)stage(0, n * 4);
    if (!d) return;
    if (report(rplb_copy(d, t->data, n * 4, NULL), who) != 0) return;
    if (report(rplb_relu_f32_inplace(d, n, NULL), who) != 0) return;
    if (report(rplb_copy(t->data, d, n * 4, NULL), who) != 0) return;
    finish(who);
}

/* ------------------------------------------------------------------------
 * Calibration and whole-model quantization: host bookkeeping over the device
 * min/max reduction.
 * ---------------------------------------------------------------------- */
/* src/rpl_quantization.c:26-31 */
QuantizationCalibrator* calibrator_create(void) {
    QuantizationCalibrator* cal = (QuantizationCalibrator*)calloc(1, sizeof(QuantizationCalibrator));
    if (!cal) return NULL;
    cal->min_val = FLT_MAX;
    cal->max_val = -FLT_MAX;
    return cal;
}

/* src/rpl_quantization.c:33-53: running min/max over the batches seen. */
void calibrator_update(QuantizationCalibrator* cal, const Tensor* t) {
    if (!cal || !t) return;
    t_last_error = 0;
    rplb_qparams hp;
    if (minmax_to_host(t, &hp, "calibrator_update") != 0) return;
    if (hp.min_val < cal->min_val) cal->min_val = hp.min_val;
    if (hp.max_val > cal->max_val) cal->max_val = hp.max_val;
    cal->num_samples++;
}

/* (int32_t)v as the reference's x86-64 build converts it. */
static int32_t f2i_x86(float v) {
    if (!(fabsf(v) < 2147483648.0f)) return INT32_MIN;
    return (int32_t)v;
}

/* src/rpl_quantization.c:55-67 */
void calibrator_compute_params(QuantizationCalibrator* cal, bool symmetric) {
    if (!cal) return;
    if (symmetric) {
        float abs_max = fmaxf(fabsf(cal->min_val), fabsf(cal->max_val));
        cal->scale = abs_max / 127.0f;
        cal->zero_point = 0;
    } else {
        float range = cal->max_val - cal->min_val;
        cal->scale = range / 255.0f;
        cal->zero_point = f2i_x86(roundf(-cal->min_val / cal->scale));
    }
}

void calibrator_free(QuantizationCalibrator* cal) { free(cal); }

/* src/rpl_quantization.c:278-298: every parameter is quantized per tensor,
 * symmetric; per_channel is accepted and, as in the reference, not acted on. */
QuantizedModel* model_quantize(Tensor** parameters, uint32_t num_params, bool per_channel) {
    (void)per_channel;
    QuantizedModel* qm = (QuantizedModel*)calloc(1, sizeof(QuantizedModel));
    if (!qm) return NULL;
    qm->num_params = num_params;
    qm->fp32_params = parameters;
    qm->int8_params = (QuantizedTensor**)calloc(num_params ? num_params : 1, sizeof(QuantizedTensor*));
    if (!qm->int8_params) { free(qm); return NULL; }
    for (uint32_t i = 0; i < num_params; i++)
        qm->int8_params[i] = tensor_quantize_int8_symmetric(parameters[i]);
    qm->is_quantized = true;
    return qm;
}

/* src/rpl_quantization.c:300-307 */
void quantized_model_free(QuantizedModel* qm) {
    if (!qm) return;
    for (uint32_t i = 0; i < qm->num_params; i++) quantized_tensor_free(qm->int8_params[i]);
    free(qm->int8_params);
    free(qm);
}

/* The per-channel counterpart of model_quantize: what the reference's flag
 * announces and leaves undone (src/rpl_quantization.c:286-292).  Parameters with
 * two or more dimensions (weights [out, ...]) are quantized per output channel,
 * i.e. per row of shape[0] (tensor_quantize_per_channel, axis 0); the others
 * (biases) get one scale for the whole tensor, stored as a single channel, which
 * is tensor_quantize_int8_symmetric's arithmetic (src/rpl_quantization.c:79-90
 * and :136-154 are the same statements over one block). */
PerChannelQuantizedModel* model_quantize_per_channel(Tensor** parameters, uint32_t num_params) {
    if (!parameters && num_params) return NULL;
    PerChannelQuantizedModel* qm = (PerChannelQuantizedModel*)calloc(1, sizeof(PerChannelQuantizedModel));
    if (!qm) return NULL;
    qm->num_params = num_params;
    qm->fp32_params = parameters;
    qm->int8_params = (PerChannelQuantizedTensor**)calloc(num_params ? num_params : 1, sizeof(PerChannelQuantizedTensor*));
    if (!qm->int8_params) { free(qm); return NULL; }
    for (uint32_t i = 0; i < num_params; i++) {
        const Tensor* t = parameters[i];
        if (!t) continue;
        if (t->dims >= 2) {
            qm->int8_params[i] = tensor_quantize_per_channel(t, 0);
        } else {
            Tensor view = *t;                      /* the same elements seen as one row */
            view.dims = 2;
            view.shape[0] = 1;
            view.shape[1] = t->size;
            PerChannelQuantizedTensor* q = tensor_quantize_per_channel(&view, 0);
            if (q) {
                q->dims = t->dims;
                memset(q->shape, 0, sizeof(q->shape));
                memcpy(q->shape, t->shape, t->dims * sizeof(uint32_t));
            }
            qm->int8_params[i] = q;
        }
        if (!qm->int8_params[i]) { per_channel_quantized_model_free(qm); return NULL; }
    }
    qm->is_quantized = true;
    return qm;
}

void per_channel_quantized_model_free(PerChannelQuantizedModel* qm) {
    if (!qm) return;
    for (uint32_t i = 0; i < qm->num_params; i++) per_channel_quantized_tensor_free(qm->int8_params[i]);
    free(qm->int8_params);
    free(qm);
}

/* ------------------------------------------------------------------------
 * Quantized weights on disk.
 *
 * The reference only writes fp32 checkpoints (checkpoint_save_model,
 * src/rpl_training.c:915-944) and has no loader.  The file written here keeps
 * that framing -- a three-word header, then per tensor `dims, shape[dims],
 * size, data[size]` -- with two changes that make it self-describing: the
 * header's second word (the reference's epoch) holds the tag 0x38544E49
 * ("INT8"), and each tensor's data is `size` int8 values followed by
 * `num_channels` and that many fp32 scales.  Zero points are not stored: the
 * per-channel quantizer only produces zero (src/rpl_quantization.c:148).
 * ---------------------------------------------------------------------- */
#define RPL_INT8_FILE_TAG 0x38544E49u

int quantized_weights_save(const char* path, PerChannelQuantizedTensor* const* tensors, uint32_t num_tensors) {
    if (!path || (!tensors && num_tensors)) return -1;
    FILE* f = fopen(path, "wb");
    if (!f) return -1;
    uint32_t tag = RPL_INT8_FILE_TAG;
    float zero = 0.0f;
    int ok = fwrite(&num_tensors, 4, 1, f) == 1 && fwrite(&tag, 4, 1, f) == 1 && fwrite(&zero, 4, 1, f) == 1;
    for (uint32_t i = 0; ok && i < num_tensors; i++) {
        const PerChannelQuantizedTensor* t = tensors[i];
        const size_t n = (size_t)t->num_channels * t->channel_size;
        uint32_t size = (uint32_t)n;
        int8_t* data = t->data;
        float* scales = t->scales;
        void *tmp_d = NULL, *tmp_s = NULL;
        if (on_device(t->data)) {           /* device-resident weights are fetched first */
            tmp_d = malloc(n ? n : 1);
            tmp_s = malloc(t->num_channels ? (size_t)t->num_channels * 4 : 4);
            ok = tmp_d && tmp_s && report(rplb_copy(tmp_d, t->data, n, NULL), "quantized_weights_save") == 0 &&
                 report(rplb_copy(tmp_s, t->scales, (size_t)t->num_channels * 4, NULL), "quantized_weights_save") == 0 &&
                 finish("quantized_weights_save") == 0;
            data = (int8_t*)tmp_d;
            scales = (float*)tmp_s;
        }
        ok = ok && fwrite(&t->dims, 4, 1, f) == 1 && fwrite(t->shape, 4, t->dims, f) == t->dims &&
             fwrite(&size, 4, 1, f) == 1 && fwrite(data, 1, n, f) == n &&
             fwrite(&t->num_channels, 4, 1, f) == 1 && fwrite(scales, 4, t->num_channels, f) == t->num_channels;
        free(tmp_d);
        free(tmp_s);
    }
    ok = (fclose(f) == 0) && ok;
    return ok ? 0 : -1;
}

/* Reads a file written by quantized_weights_save.  Returns a malloc'ed array of
 * *num_tensors tensors (each released with per_channel_quantized_tensor_free,
 * the array with free), in host memory, or in device memory when to_device is
 * true.  NULL on any error (bad tag, short file, allocation or copy failure). */
PerChannelQuantizedTensor** quantized_weights_load(const char* path, uint32_t* num_tensors, bool to_device) {
    if (!path || !num_tensors) return NULL;
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    uint32_t n_t = 0, tag = 0;
    float metric;
    if (fread(&n_t, 4, 1, f) != 1 || fread(&tag, 4, 1, f) != 1 || fread(&metric, 4, 1, f) != 1 ||
        tag != RPL_INT8_FILE_TAG || n_t > (1u << 20)) { fclose(f); return NULL; }
    PerChannelQuantizedTensor** out = (PerChannelQuantizedTensor**)calloc(n_t ? n_t : 1, sizeof(*out));
    int ok = out != NULL;
    for (uint32_t i = 0; ok && i < n_t; i++) {
        PerChannelQuantizedTensor* t = (PerChannelQuantizedTensor*)calloc(1, sizeof(*t));
        out[i] = t;
        uint32_t size = 0;
        ok = t && fread(&t->dims, 4, 1, f) == 1 && t->dims <= MAX_DIMS &&
             fread(t->shape, 4, t->dims, f) == t->dims && fread(&size, 4, 1, f) == 1;
        if (!ok) break;
        /* The element count must be the product of the shape (a file written by quantized_weights_save always is). */
        uint64_t prod = 1;
        for (uint32_t d = 0; d < t->dims; d++) prod *= t->shape[d];
        ok = prod == size;
        if (!ok) break;
        /* The tensor owns its blocks from the moment they exist, so the error path below frees them. */
        t->data = (int8_t*)rpitorch_aligned_alloc(64, size ? size : 1);
        ok = t->data && fread(t->data, 1, size, f) == size && fread(&t->num_channels, 4, 1, f) == 1 &&
             t->num_channels <= size + 1u;
        /* Channels are equal contiguous blocks: their count divides the size and is one of the
         * tensor's extents (tensor_quantize_per_channel takes it from shape[axis]), or 1. */
        int axis_ok = t->num_channels == 1 || (t->num_channels == 0 && size == 0);
        for (uint32_t d = 0; d < t->dims; d++) axis_ok = axis_ok || t->num_channels == t->shape[d];
        ok = ok && axis_ok && (t->num_channels ? size % t->num_channels == 0 : size == 0);
        if (!ok) break;
        const size_t cb = t->num_channels ? (size_t)t->num_channels * 4 : 4;
        t->scales = (float*)malloc(cb);
        t->zero_points = (int32_t*)calloc(1, cb);
        ok = t->scales && t->zero_points && fread(t->scales, 4, t->num_channels, f) == t->num_channels;
        if (!ok) break;
        t->channel_size = t->num_channels ? size / t->num_channels : 0;
        if (to_device) {
            void *dd = NULL, *ds = NULL, *dz = NULL;
            ok = report(rplb_malloc(&dd, size), "quantized_weights_load") == 0 &&
                 report(rplb_malloc(&ds, cb), "quantized_weights_load") == 0 &&
                 report(rplb_malloc(&dz, cb), "quantized_weights_load") == 0 &&
                 report(rplb_copy(dd, t->data, size, NULL), "quantized_weights_load") == 0 &&
                 report(rplb_copy(ds, t->scales, (size_t)t->num_channels * 4, NULL), "quantized_weights_load") == 0 &&
                 report(rplb_copy(dz, t->zero_points, (size_t)t->num_channels * 4, NULL), "quantized_weights_load") == 0 &&
                 finish("quantized_weights_load") == 0;
            if (!ok) { rplb_free(dd); rplb_free(ds); rplb_free(dz); break; }
            free(t->data); free(t->scales); free(t->zero_points);
            t->data = (int8_t*)dd; t->scales = (float*)ds; t->zero_points = (int32_t*)dz;
        }
    }
    fclose(f);
    if (!ok) {
        if (out) { for (uint32_t i = 0; i < n_t; i++) per_channel_quantized_tensor_free(out[i]); free(out); }
        return NULL;
    }
    *num_tensors = n_t;
    return out;
}

/* ------------------------------------------------------------------------
 * A quantized Linear layer: what linear_forward (src/rpl_nn.c:55-77) computes,
 * x . W^T + b with W [out_features, in_features], on the INT8 path.  The
 * weights are quantized per output row once, at creation, and stay in device
 * memory with their scales and the fp32 bias; forward quantizes the
 * activation per tensor (tensor_quantize_int8_symmetric's arithmetic) and runs
 * the INT8 GEMM with the fused dequantize + bias (+ ReLU) epilogue.
 * ---------------------------------------------------------------------- */
#define QL_DEPTH 2          /* calls in flight in the host-buffer pipeline */
#define QL_BLOCKS 8         /* row blocks per call: a block is downloaded while the next one computes */

struct QuantizedLinear {
    PerChannelQuantizedTensor* weight;   /* device-resident int8 rows, scales, zero points */
    float*   bias;                       /* device, out_features floats, or NULL */
    uint32_t in_features;
    uint32_t out_features;
    int      owns_weight;                /* 0 when the int8 rows / scales / bias belong to the caller */
    int8_t*  act;                        /* device buffer for the quantized activation */
    size_t   act_capacity;
    rplb_qparams* act_params;            /* device */
    /* host-buffer pipeline (quantized_linear_submit_host / _drain) */
    void*    s_main;                     /* compute stream: the caller's, or one owned by the layer */
    int      owns_main;
    void*    s_in;                       /* uploads */
    void*    s_out;                      /* downloads */
    float*   din[QL_DEPTH];              /* device copies of the activations in flight */
    float*   dout[QL_DEPTH];             /* device outputs in flight */
    size_t   din_capacity[QL_DEPTH], dout_capacity[QL_DEPTH];
    void*    ev_uploaded[QL_DEPTH];
    void*    ev_computed[QL_DEPTH];
    void*    ev_downloaded[QL_DEPTH];
    void*    ev_block[QL_DEPTH][QL_BLOCKS];
    int      slot_used[QL_DEPTH];
    uint64_t calls;
};

static void quantized_linear_release_pipeline(QuantizedLinear* layer) {
    if (layer->s_in) {                   /* nothing may be in flight when buffers and streams go */
        rplb_stream_sync(layer->s_in);
        rplb_stream_sync(layer->s_main);
        rplb_stream_sync(layer->s_out);
    }
    for (int i = 0; i < QL_DEPTH; i++) {
        rplb_free(layer->din[i]);
        rplb_free(layer->dout[i]);
        rplb_event_destroy(layer->ev_uploaded[i]);
        rplb_event_destroy(layer->ev_computed[i]);
        rplb_event_destroy(layer->ev_downloaded[i]);
        for (int b = 0; b < QL_BLOCKS; b++) rplb_event_destroy(layer->ev_block[i][b]);
    }
    rplb_stream_destroy(layer->s_in);
    rplb_stream_destroy(layer->s_out);
    if (layer->owns_main) rplb_stream_destroy(layer->s_main);
}

void quantized_linear_free(QuantizedLinear* layer) {
    if (!layer) return;
    quantized_linear_release_pipeline(layer);
    if (layer->owns_weight) {
        per_channel_quantized_tensor_free(layer->weight);
        rplb_free(layer->bias);
    } else {
        free(layer->weight);             /* the struct only; its blocks are the caller's */
    }
    rplb_free(layer->act);
    rplb_free(layer->act_params);
    free(layer);
}

QuantizedLinear* quantized_linear_create(const Tensor* weight, const Tensor* bias) {
    if (!weight || weight->dims != 2) return NULL;
    t_last_error = 0;
    const char* who = "quantized_linear_create";
    QuantizedLinear* layer = (QuantizedLinear*)calloc(1, sizeof(QuantizedLinear));
    if (!layer) return NULL;
    layer->out_features = weight->shape[0];
    layer->in_features = weight->shape[1];
    layer->owns_weight = 1;
    /* Quantize on the device and keep the result there: a device-resident input
     * makes tensor_quantize_per_channel return device-resident blocks. */
    Tensor* wdev = on_device(tensor_data(weight)) ? NULL : tensor_upload(weight);
    layer->weight = tensor_quantize_per_channel(wdev ? wdev : weight, 0);
    tensor_free(wdev);
    void* params = NULL;
    if (!layer->weight || report(rplb_malloc(&params, sizeof(rplb_qparams)), who) != 0) { quantized_linear_free(layer); return NULL; }
    layer->act_params = (rplb_qparams*)params;
    if (bias) {
        void* b = NULL;
        if (bias->size != layer->out_features || report(rplb_malloc(&b, (size_t)bias->size * 4), who) != 0 ||
            report(rplb_copy(b, tensor_data(bias), (size_t)bias->size * 4, NULL), who) != 0 || finish(who) != 0) {
            rplb_free(b);
            quantized_linear_free(layer);
            return NULL;
        }
        layer->bias = (float*)b;
    }
    return layer;
}

Tensor* quantized_linear_forward(QuantizedLinear* layer, const Tensor* input, bool relu) {
    if (!layer || !input || input->dims < 1 || input->size % layer->in_features != 0) return NULL;
    t_last_error = 0;
    const char* who = "quantized_linear_forward";
    if (quantized_linear_drain(layer) != 0) return NULL;      /* nothing of the host pipeline may be in flight */
    const size_t K = layer->in_features, N = layer->out_features, M = input->size / K;
    const float* src = tensor_data(input);
    const int dev_in = on_device(src);
    uint32_t out_shape[2] = {(uint32_t)M, (uint32_t)N};                      /* src/rpl_nn.c:57 */
    Tensor* out = dev_in ? tensor_create_device(2, out_shape) : tensor_create(2, out_shape, false);
    if (!out) return NULL;
    if (layer->act_capacity < M * K) {
        rplb_stream_sync(NULL);
        rplb_free(layer->act);
        layer->act = NULL;
        layer->act_capacity = 0;
        void* a = NULL;
        if (report(rplb_malloc(&a, M * K), who) != 0) { tensor_free(out); return NULL; }
        layer->act = (int8_t*)a;
        layer->act_capacity = M * K;
    }
    const float* x = (const float*)to_device(0, src, M * K * 4);
    float* o = dev_in ? out->data : (float*)stage(3, M * N * 4);
    if ((M * K && !x) || !o) { tensor_free(out); return NULL; }
    /* Layers with a handful of output features (N <= 16, K <= 512): the quantize step rides inside the dp4a
     * contraction and the int8 activation is never written, which is faster than two kernels there.  (For wider
     * layers the fused tensor-core kernel is no faster than quantize + GEMM, so those keep the two-step route.)
     * A refusal (alignment) falls back to the two-step route as well.  Same bits either way. */
    int rc = RPLB_E_UNSUPPORTED;
    if (N <= 16 && K <= 512 && K % 4 == 0) {
        rc = report(rplb_minmax_f32(x, M * K, layer->act_params, NULL), who);
        if (rc == 0)
            rc = rplb_quantize_linear_dequant_f32(x, layer->weight->data, o, M, K, N, N, &layer->act_params->scale_sym,
                                                  layer->weight->scales, layer->bias, relu ? 1 : 0, NULL, NULL, NULL);
        if (rc != 0 && rc != RPLB_E_UNSUPPORTED) report(rc, who);
    }
    if (rc == RPLB_E_UNSUPPORTED) {
        rc = report(rplb_quantize_symmetric_f32_i8(x, layer->act, M * K, layer->act_params, NULL), who);
        if (rc == 0)
            rc = report(rplb_linear_i8_dequant_f32(layer->act, layer->weight->data, o, M, K, N, N, &layer->act_params->scale_sym,
                                                   layer->weight->scales, layer->bias, relu ? 1 : 0, NULL), who);
    }
    if (rc != 0 || (!dev_in && report(rplb_copy(out->data, o, M * N * 4, NULL), who) != 0) || finish(who) != 0) {
        tensor_free(out);
        return NULL;
    }
    return out;
}

/* Several layers applied to the same input, the way multi-head attention
 * applies W_q, W_k and W_v to one activation (src/rpl_attention.c:175-177):
 * the activation is quantized once (into the first layer's buffer) and every
 * layer's GEMM reads that int8 copy.  outputs[i] receives a new Tensor
 * [rows, out_features of layer i]; 0 on success, else nothing is returned and
 * every outputs[i] is NULL. */
int quantized_linear_forward_shared_input(QuantizedLinear* const* layers, uint32_t num_layers, const Tensor* input,
                                          Tensor** outputs, bool relu) {
    const char* who = "quantized_linear_forward_shared_input";
    if (!layers || !outputs || num_layers == 0 || !input) return RPLB_E_BAD_ARG;
    for (uint32_t i = 0; i < num_layers; i++) outputs[i] = NULL;
    for (uint32_t i = 0; i < num_layers; i++)
        if (!layers[i] || layers[i]->in_features != layers[0]->in_features) return RPLB_E_BAD_ARG;
    QuantizedLinear* first = layers[0];
    if (input->dims < 1 || input->size % first->in_features != 0) return RPLB_E_BAD_ARG;
    t_last_error = 0;
    for (uint32_t i = 0; i < num_layers; i++)
        if (quantized_linear_drain(layers[i]) != 0) return t_last_error ? t_last_error : RPLB_E_KERNEL;
    const size_t K = first->in_features, M = input->size / K;
    const float* src = tensor_data(input);
    const int dev_in = on_device(src);
    if (first->act_capacity < M * K) {
        rplb_stream_sync(NULL);
        rplb_free(first->act);
        first->act = NULL;
        first->act_capacity = 0;
        void* a = NULL;
        if (report(rplb_malloc(&a, M * K), who) != 0) return t_last_error;
        first->act = (int8_t*)a;
        first->act_capacity = M * K;
    }
    const float* x = (const float*)to_device(0, src, M * K * 4);
    if (M * K && !x) return t_last_error ? t_last_error : RPLB_E_BAD_ARG;
    int rc = report(rplb_quantize_symmetric_f32_i8(x, first->act, M * K, first->act_params, NULL), who);
    for (uint32_t i = 0; rc == 0 && i < num_layers; i++) {
        const size_t N = layers[i]->out_features;
        uint32_t out_shape[2] = {(uint32_t)M, (uint32_t)N};
        outputs[i] = dev_in ? tensor_create_device(2, out_shape) : tensor_create(2, out_shape, false);
        if (!outputs[i]) { rc = RPLB_E_BAD_ARG; break; }
        /* Host results pass through one staging block: finish each layer's copy before the next GEMM reuses it. */
        float* o = dev_in ? outputs[i]->data : (float*)stage(3, M * N * 4);
        if (!o) { rc = t_last_error ? t_last_error : RPLB_E_BAD_ARG; break; }
        rc = report(rplb_linear_i8_dequant_f32(first->act, layers[i]->weight->data, o, M, K, N, N, &first->act_params->scale_sym,
                                               layers[i]->weight->scales, layers[i]->bias, relu ? 1 : 0, NULL), who);
        if (rc == 0 && !dev_in) rc = report(rplb_copy(outputs[i]->data, o, M * N * 4, NULL), who);
    }
    if (rc == 0) rc = finish(who);
    if (rc != 0) {
        for (uint32_t i = 0; i < num_layers; i++) { tensor_free(outputs[i]); outputs[i] = NULL; }
    }
    return rc;
}

/* A layer over int8 weight rows, scales and bias that already live in device
 * memory and stay the caller's (nothing is copied, nothing is freed by
 * quantized_linear_free). */
QuantizedLinear* quantized_linear_wrap(const int8_t* weight_rows, const float* scales, const float* bias,
                                       uint32_t in_features, uint32_t out_features) {
    if (!weight_rows || !scales || !on_device(weight_rows) || !on_device(scales) || (bias && !on_device(bias))) return NULL;
    t_last_error = 0;
    QuantizedLinear* layer = (QuantizedLinear*)calloc(1, sizeof(QuantizedLinear));
    PerChannelQuantizedTensor* w = (PerChannelQuantizedTensor*)calloc(1, sizeof(PerChannelQuantizedTensor));
    void* params = NULL;
    if (!layer || !w || report(rplb_malloc(&params, sizeof(rplb_qparams)), "quantized_linear_wrap") != 0) {
        free(layer);
        free(w);
        return NULL;
    }
    w->data = (int8_t*)weight_rows;
    w->scales = (float*)scales;
    w->num_channels = out_features;
    w->channel_size = in_features;
    w->dims = 2;
    w->shape[0] = out_features;
    w->shape[1] = in_features;
    layer->weight = w;
    layer->bias = (float*)bias;
    layer->in_features = in_features;
    layer->out_features = out_features;
    layer->act_params = (rplb_qparams*)params;
    return layer;
}

/* Streams and events of the host-buffer pipeline, created on first use.
 * compute_stream: the stream quantize and GEMM run on (a cudaStream_t); NULL lets the layer own one. */
static int quantized_linear_pipeline_ready(QuantizedLinear* layer, void* compute_stream, const char* who) {
    if (layer->s_in) {
        if (compute_stream && compute_stream != layer->s_main) {
            if (report(rplb_stream_sync(layer->s_main), who)) return -1;
            if (layer->owns_main) rplb_stream_destroy(layer->s_main);
            layer->s_main = compute_stream;
            layer->owns_main = 0;
        }
        return 0;
    }
    if (compute_stream) { layer->s_main = compute_stream; layer->owns_main = 0; }
    else { if (report(rplb_stream_create(&layer->s_main), who)) return -1; layer->owns_main = 1; }
    if (report(rplb_stream_create(&layer->s_out), who) || report(rplb_stream_create(&layer->s_in), who)) return -1;
    for (int i = 0; i < QL_DEPTH; i++) {
        if (report(rplb_event_create(&layer->ev_uploaded[i]), who) || report(rplb_event_create(&layer->ev_computed[i]), who) ||
            report(rplb_event_create(&layer->ev_downloaded[i]), who)) return -1;
        for (int b = 0; b < QL_BLOCKS; b++)
            if (report(rplb_event_create(&layer->ev_block[i][b]), who)) return -1;
    }
    return 0;
}

static int grow_device(void** p, size_t* cap, size_t bytes, const char* who) {
    if (*cap >= bytes) return 0;
    rplb_free(*p);
    *p = NULL;
    *cap = 0;
    if (report(rplb_malloc(p, bytes), who)) return -1;
    *cap = bytes;
    return 0;
}

/* y = x . W^T + b on host buffers, enqueued: x is [rows, in_features] fp32 and out
 * [rows, out_features] fp32, both in host memory (page-locked for full PCIe speed).
 * The call returns once everything is queued; quantized_linear_drain waits.  Inputs
 * and outputs are double-buffered on the device: the upload of call n+1 overlaps the
 * compute and download of call n, and within a call each row block is downloaded
 * while the next one is in the GEMM.  x must stay valid until its upload has run and
 * out must not be read before the drain.  Returns 0, or the error code also kept by
 * rpl_cuda_last_error(). */
int quantized_linear_submit_host(QuantizedLinear* layer, const float* x, uint32_t rows, float* out, bool relu,
                                 void* compute_stream) {
    if (!layer || !x || !out) return RPLB_E_BAD_ARG;
    if (rows == 0) return 0;
    t_last_error = 0;
    const char* who = "quantized_linear_submit_host";
    if (quantized_linear_pipeline_ready(layer, compute_stream, who)) return t_last_error;
    const size_t K = layer->in_features, N = layer->out_features, M = rows;
    const int i = (int)(layer->calls % QL_DEPTH);
    if (layer->din_capacity[i] < M * K * 4 || layer->dout_capacity[i] < M * N * 4 || layer->act_capacity < M * K) {
        /* Buffers change size only with everything idle. */
        if (report(rplb_stream_sync(layer->s_in), who) || report(rplb_stream_sync(layer->s_main), who) ||
            report(rplb_stream_sync(layer->s_out), who)) return t_last_error;
        if (grow_device((void**)&layer->din[i], &layer->din_capacity[i], M * K * 4, who) ||
            grow_device((void**)&layer->dout[i], &layer->dout_capacity[i], M * N * 4, who) ||
            grow_device((void**)&layer->act, &layer->act_capacity, M * K, who)) return t_last_error;
    }
    float* din = layer->din[i];
    float* dout = layer->dout[i];
    if (layer->slot_used[i] && report(rplb_stream_wait_event(layer->s_in, layer->ev_computed[i]), who)) return t_last_error;
    if (report(rplb_copy(din, x, M * K * 4, layer->s_in), who) || report(rplb_event_record(layer->ev_uploaded[i], layer->s_in), who) ||
        report(rplb_stream_wait_event(layer->s_main, layer->ev_uploaded[i]), who)) return t_last_error;
    if (layer->slot_used[i] && report(rplb_stream_wait_event(layer->s_main, layer->ev_downloaded[i]), who)) return t_last_error;
    if (report(rplb_quantize_symmetric_f32_i8(din, layer->act, M * K, layer->act_params, layer->s_main), who)) return t_last_error;
    size_t step = (M + QL_BLOCKS - 1) / QL_BLOCKS;
    step = (step + 127) / 128 * 128;
    int b = 0;
    for (size_t r0 = 0; r0 < M; r0 += step, b++) {
        const size_t r1 = r0 + step < M ? r0 + step : M;
        if (report(rplb_linear_i8_dequant_f32(layer->act + r0 * K, layer->weight->data, dout + r0 * N, r1 - r0, K, N, N,
                                              &layer->act_params->scale_sym, layer->weight->scales, layer->bias,
                                              relu ? 1 : 0, layer->s_main), who) ||
            report(rplb_event_record(layer->ev_block[i][b], layer->s_main), who) ||
            report(rplb_stream_wait_event(layer->s_out, layer->ev_block[i][b]), who) ||
            report(rplb_copy(out + r0 * N, dout + r0 * N, (r1 - r0) * N * 4, layer->s_out), who)) return t_last_error;
    }
    if (report(rplb_event_record(layer->ev_computed[i], layer->s_main), who) ||
        report(rplb_event_record(layer->ev_downloaded[i], layer->s_out), who)) return t_last_error;
    layer->slot_used[i] = 1;
    layer->calls++;
    return 0;
}

/* Waits until every submitted call has delivered its output.  The compute stream is
 * made to wait for the downloads first, so an event recorded on it after this call
 * also covers them. */
int quantized_linear_drain(QuantizedLinear* layer) {
    if (!layer || !layer->s_in) return 0;
    const char* who = "quantized_linear_drain";
    for (int i = 0; i < QL_DEPTH; i++)
        if (layer->slot_used[i] && report(rplb_stream_wait_event(layer->s_main, layer->ev_downloaded[i]), who)) return t_last_error;
    if (report(rplb_stream_sync(layer->s_out), who) || report(rplb_stream_sync(layer->s_main), who)) return t_last_error;
    int st = rplb_kernel_status(1);
    if (st != 0) {
        t_last_error = RPLB_E_KERNEL;
        fprintf(stderr, "rpl (cuda): %s: a kernel gave up waiting (code %d)\n", who, st);
        return RPLB_E_KERNEL;
    }
    return 0;
}
