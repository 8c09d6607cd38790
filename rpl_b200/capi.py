"""ctypes binding of ``librpl.so``: the structs of the reference ABI, the
``rplb_*`` device-level entry points and the reference-named C API.

This is a binding, not an implementation: every function here ends in a call
into the shared library, and loading fails loudly when the library has not
been built (``python -m rpl_b200.build``).
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "librpl.so")

MAX_DIMS = 8
f32p = C.POINTER(C.c_float)
i8p = C.POINTER(C.c_int8)
i32p = C.POINTER(C.c_int32)

RPLB_E_NO_DEVICE, RPLB_E_BAD_ARG, RPLB_E_TOO_LARGE, RPLB_E_KERNEL, RPLB_E_UNSUPPORTED, RPLB_E_COMM = -1, -2, -3, -4, -5, -6
RPLB_NCCL_ID_BYTES = 128
ALLOC_FN = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p), C.c_size_t)
FREE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)


class RplError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("librpl error %d: %s" % (code, text))
        self.code = code


class Tensor(C.Structure):
    """``Tensor`` (include/rpl.h:57-78 of the reference), sizeof 152."""


Tensor._fields_ = [
    ("data", C.c_void_p), ("grad", C.c_void_p), ("dims", C.c_uint32),
    ("shape", C.c_uint32 * MAX_DIMS), ("strides", C.c_uint32 * MAX_DIMS),
    ("size", C.c_uint32), ("requires_grad", C.c_bool),
    ("_allocation", C.c_void_p), ("_alloc_size", C.c_size_t),
    ("device", C.c_int), ("gpu_buffer", C.c_uint32),
    ("is_leaf", C.c_bool), ("parent1", C.c_void_p), ("parent2", C.c_void_p),
    ("backward_fn", C.c_void_p),
]


class QuantizedTensor(C.Structure):
    """``QuantizedTensor`` (include/rpl.h:167-174), sizeof 56."""
    _fields_ = [("data", C.c_void_p), ("scale", C.c_float), ("zero_point", C.c_int32),
                ("size", C.c_uint32), ("dims", C.c_uint32), ("shape", C.c_uint32 * MAX_DIMS)]


class PerChannelQuantizedTensor(C.Structure):
    """``PerChannelQuantizedTensor`` (src/rpl_quantization.c:110-118)."""
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("zero_points", C.c_void_p),
                ("num_channels", C.c_uint32), ("channel_size", C.c_uint32),
                ("dims", C.c_uint32), ("shape", C.c_uint32 * MAX_DIMS)]


class QuantizationCalibrator(C.Structure):
    """``QuantizationCalibrator`` (src/rpl_quantization.c:18-24)."""
    _fields_ = [("min_val", C.c_float), ("max_val", C.c_float), ("scale", C.c_float),
                ("zero_point", C.c_int32), ("num_samples", C.c_uint32)]


class QuantizedModel(C.Structure):
    """``QuantizedModel`` (src/rpl_quantization.c:271-276)."""
    _fields_ = [("fp32_params", C.POINTER(C.POINTER(Tensor))), ("int8_params", C.POINTER(C.POINTER(QuantizedTensor))),
                ("num_params", C.c_uint32), ("is_quantized", C.c_bool)]


class PerChannelQuantizedModel(C.Structure):
    """``PerChannelQuantizedModel``: what ``model_quantize_per_channel`` returns."""
    _fields_ = [("fp32_params", C.POINTER(C.POINTER(Tensor))), ("int8_params", C.POINTER(C.POINTER(PerChannelQuantizedTensor))),
                ("num_params", C.c_uint32), ("is_quantized", C.c_bool)]


class QParams(C.Structure):
    """``rplb_qparams``: what the min/max kernel leaves on the device (32 bytes)."""
    _fields_ = [("min_val", C.c_float), ("max_val", C.c_float), ("scale_sym", C.c_float),
                ("scale_asym", C.c_float), ("zp_asym", C.c_int32), ("first", C.c_float),
                ("true_min", C.c_float), ("true_max", C.c_float)]


# name -> (restype, argtypes); restype "rc" = int status checked by ``call``.
_vp, _u64, _f, _i, _sz = C.c_void_p, C.c_uint64, C.c_float, C.c_int32, C.c_size_t
_TP, _QP, _PP = C.POINTER(Tensor), C.POINTER(QuantizedTensor), C.POINTER(PerChannelQuantizedTensor)
_CP, _MP = C.POINTER(QuantizationCalibrator), C.POINTER(QuantizedModel)
SIGNATURES = {
    # device-level layer
    "rplb_last_error": (C.c_char_p, []),
    "rplb_device_count": (C.c_int, []),
    "rplb_device_sm_count": (C.c_int, []),
    "rplb_set_device": ("rc", [C.c_int]),
    "rplb_launch_count": (C.c_uint64, []),
    "rplb_malloc": ("rc", [C.POINTER(_vp), _sz]),
    "rplb_free": ("rc", [_vp]),
    "rplb_set_allocator": ("rc", [ALLOC_FN, FREE_FN]),
    "rplb_scratch_reserve": ("rc", [_vp, _sz]),
    "rplb_scratch_release": ("rc", [_vp]),
    "rplb_host_alloc": ("rc", [C.POINTER(_vp), _sz]),
    "rplb_host_free": ("rc", [_vp]),
    "rplb_copy": ("rc", [_vp, _vp, _sz, _vp]),
    "rplb_stream_sync": ("rc", [_vp]),
    "rplb_stream_create": ("rc", [C.POINTER(_vp)]),
    "rplb_stream_destroy": ("rc", [_vp]),
    "rplb_event_create": ("rc", [C.POINTER(_vp)]),
    "rplb_event_destroy": ("rc", [_vp]),
    "rplb_event_record": ("rc", [_vp, _vp]),
    "rplb_stream_wait_event": ("rc", [_vp, _vp]),
    "rplb_pointer_kind": (C.c_int, [_vp]),
    "rplb_ipc_export": ("rc", [_vp, _vp]),
    "rplb_ipc_open": ("rc", [_vp, C.POINTER(C.c_void_p)]),
    "rplb_ipc_close": ("rc", [_vp]),
    "rplb_minmax_f32": ("rc", [_vp, _u64, _vp, _vp]),
    "rplb_minmax_f32_static": ("rc", [_vp, _u64, _vp, _vp]),
    "rplb_qparams_to_pair": ("rc", [_vp, _vp, _vp]),
    "rplb_qparams_from_pair": ("rc", [_vp, _vp, _vp]),
    "rplb_quantize_f32_i8": ("rc", [_vp, _vp, _u64, _f, _i, _vp]),
    "rplb_quantize_f32_i8_dev": ("rc", [_vp, _vp, _u64, _vp, _vp, _vp]),
    "rplb_quantize_symmetric_f32_i8": ("rc", [_vp, _vp, _u64, _vp, _vp]),
    "rplb_quantize_asymmetric_f32_i8": ("rc", [_vp, _vp, _u64, _vp, _vp]),
    "rplb_quantize_onepass": (C.c_int, [C.c_int]),
    "rplb_quantize_per_channel_f32_i8": ("rc", [_vp, _vp, _vp, _vp, _u64, _u64, _vp]),
    "rplb_per_channel_staging": (C.c_int, [C.c_int]),
    "rplb_dequantize_i8_f32": ("rc", [_vp, _vp, _u64, _f, _i, _vp]),
    "rplb_dequantize_per_channel_i8_f32": ("rc", [_vp, _vp, _vp, _u64, _u64, _vp]),
    "rplb_relu_f32_inplace": ("rc", [_vp, _u64, _vp]),
    "rplb_linear_i8_i32": ("rc", [_vp, _vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "rplb_gemm_i8_requant_i32": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _f, _f, _f, _i, _i, _vp]),
    "rplb_linear_i8_dequant_f32": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int, _vp]),
    "rplb_linear_i8_dequant_f32_peers": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int,
                                                C.POINTER(C.c_void_p), C.c_int, _vp]),
    "rplb_linear_i8_dequant_f32_arriving": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int,
                                                   _vp, C.c_uint32, C.c_uint32, C.c_uint32, _vp]),
    "rplb_linear_i8_dequant_f32_absmax": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp]),
    "rplb_quantize_linear_dequant_f32": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp]),
    "rplb_linear_i8_requant_i8": ("rc", [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp, _vp, _vp, C.c_int, _vp, _i, _vp]),
    "rplb_gemm_backend": (C.c_int, [C.c_int]),
    "rplb_gemm_epilogue": (C.c_int, [C.c_int]),
    "rplb_selftest_bounded_wait_keep": ("rc", [_vp]),
    "rplb_nccl_unique_id": ("rc", [_vp]),
    "rplb_sharded_linear_create": ("rc", [C.POINTER(_vp), C.c_int, C.c_int, _vp, _vp, _u64, _u64, _u64, _vp, _vp, _vp]),
    "rplb_sharded_linear_create_split": ("rc", [C.POINTER(_vp), C.c_int, C.c_int, _vp, _vp, _u64, _u64, _u64, C.POINTER(_u64), _vp, _vp, _vp]),
    "rplb_shard_weighted": ("rc", [_u64, C.c_int, _u64, C.POINTER(C.c_double), C.POINTER(_u64)]),
    "rplb_sharded_linear_free": (None, [_vp]),
    "rplb_sharded_linear_columns": ("rc", [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "rplb_sharded_linear_rows": ("rc", [_vp, _u64, C.POINTER(_u64), C.POINTER(_u64)]),
    "rplb_sharded_linear_forward": ("rc", [_vp, _vp, _u64, _vp, _u64, C.c_int, _vp]),
    "rplb_sharded_linear_quantize": ("rc", [_vp, _vp, _u64, _vp]),
    "rplb_sharded_linear_gemm": ("rc", [_vp, _u64, _vp, _u64, C.c_int, _vp]),
    "rplb_sharded_linear_transfer": ("rc", [_vp, C.c_int]),
    "rplb_sharded_linear_activation": ("rc", [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "rplb_sharded_linear_gather": ("rc", [_vp, _vp, _u64, _u64, _vp, _vp]),
    "rplb_sharded_linear_submit_host": ("rc", [_vp, _vp, _u64, _vp, C.c_int, C.c_int, _vp]),
    "rplb_sharded_linear_drain": ("rc", [_vp]),
    "rplb_kernel_status": (C.c_int, [C.c_int]),
    "rplb_selftest_bounded_wait": ("rc", [_vp]),
    "rplb_shard_range": ("rc", [_u64, C.c_int, C.c_int, _u64, C.POINTER(_u64), C.POINTER(_u64)]),
    # reference-named layer
    "tensor_create": (_TP, [C.c_uint32, C.POINTER(C.c_uint32), C.c_bool]),
    "tensor_free": (None, [_TP]),
    "rpitorch_aligned_alloc": (_vp, [_sz, _sz]),
    "rpitorch_aligned_free": (None, [_vp]),
    "rpl_gpu_init": (C.c_bool, []),
    "rpl_gpu_shutdown": (None, []),
    "tensor_to_gpu": (None, [_TP]),
    "tensor_from_gpu": (None, [_TP]),
    "tensor_quantize_int8": (_QP, [_TP, _f, _i]),
    "quantized_tensor_free": (None, [_QP]),
    "tensor_get_min_max": (None, [_TP, f32p, f32p]),
    "tensor_dequantize_int8": (_TP, [_QP]),
    "gemm_int8": (None, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, C.c_uint32, _f, _f, _f, _i, _i]),
    "gemm_int8_fallback": (None, [_vp, _vp, _vp, C.c_uint32, C.c_uint32, C.c_uint32, _f, _f, _f, _i, _i]),
    "tensor_quantize_int8_symmetric": (_QP, [_TP]),
    "tensor_quantize_int8_asymmetric": (_QP, [_TP]),
    "tensor_quantize_per_channel": (_PP, [_TP, C.c_uint32]),
    "per_channel_quantized_tensor_free": (None, [_PP]),
    "linear_int8": (None, [_QP, _QP, _QP, _vp, C.c_uint32, C.c_uint32, C.c_uint32]),
    "calibrator_create": (_CP, []),
    "calibrator_update": (None, [_CP, _TP]),
    "calibrator_compute_params": (None, [_CP, C.c_bool]),
    "calibrator_free": (None, [_CP]),
    "model_quantize": (_MP, [C.POINTER(_TP), C.c_uint32, C.c_bool]),
    "quantized_model_free": (None, [_MP]),
    "model_quantize_per_channel": (_vp, [C.POINTER(_TP), C.c_uint32]),
    "per_channel_quantized_model_free": (None, [_vp]),
    "tensor_relu_inplace": (None, [_TP]),
    "rpl_cuda_last_error": (C.c_int, []),
    "tensor_create_device": (_TP, [C.c_uint32, C.POINTER(C.c_uint32)]),
    "tensor_upload": (_TP, [_TP]),
    "tensor_download": (_TP, [_TP]),
    "linear_int8_dequant": (None, [_QP, _PP, _vp, _vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_bool]),
    "tensor_dequantize_per_channel": (_TP, [_PP]),
    "quantized_linear_create": (_vp, [_TP, _TP]),
    "quantized_linear_forward": (_TP, [_vp, _TP, C.c_bool]),
    "quantized_linear_free": (None, [_vp]),
    "quantized_linear_wrap": (_vp, [_vp, _vp, _vp, C.c_uint32, C.c_uint32]),
    "quantized_linear_submit_host": (C.c_int, [_vp, _vp, C.c_uint32, _vp, C.c_bool, _vp]),
    "quantized_linear_forward_shared_input": (C.c_int, [C.POINTER(_vp), C.c_uint32, _TP, C.POINTER(_TP), C.c_bool]),
    "quantized_linear_drain": (C.c_int, [_vp]),
    "quantized_weights_save": (C.c_int, [C.c_char_p, C.POINTER(_PP), C.c_uint32]),
    "quantized_weights_load": (C.POINTER(_PP), [C.c_char_p, C.POINTER(C.c_uint32), C.c_bool]),
}

_lib = None


def load(path=None):
    """Load the shared library (once) and attach the signatures above."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise ImportError("%s is missing: build it with `python -m rpl_b200.build` (needs nvcc)" % p)
    L = C.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)          # AttributeError here = the library lacks a declared symbol
        fn.argtypes = args
        fn.restype = C.c_int if res == "rc" else res
    if path is None:
        _lib = L
    return L


def call(name, *args):
    """Call a status-returning ``rplb_*`` function; raise RplError on failure."""
    L = load()
    rc = getattr(L, name)(*args)
    if rc != 0:
        raise RplError(rc, (L.rplb_last_error() or b"").decode(errors="replace"))
    return 0
