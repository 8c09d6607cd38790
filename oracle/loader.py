"""numpy front-ends of the two CPU checkers (test infrastructure only).

``Port``  wraps ``librpl_oracle.so`` (the C restatement in ``rpl_oracle.c``).
``Ref``   wraps ``_ref/librpl_ref.so``: the reference's own functions, called
          through the reference's own structs (``Tensor`` include/rpl.h:57-78,
          ``QuantizedTensor`` include/rpl.h:167-174, ``PerChannelQuantizedTensor``
          src/rpl_quantization.c:110-118).

Only tests, the smoke check and the CPU legs of the benchmark may import this
module; the shipped library never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "librpl_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "librpl_ref.so")

MAX_DIMS = 8
_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)


def build(quiet=True):
    """Run the Makefile beside this file (port always; reference if its tree exists)."""
    out = subprocess.run(["make", "-C", HERE, "all"], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _ptr(a, typ):
    return a.ctypes.data_as(typ) if a is not None else typ()


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


class Port:
    """The C restatement."""

    def __init__(self):
        if not os.path.exists(PORT_SO):
            build()
        L = C.CDLL(PORT_SO)
        u64, f32, i32 = C.c_uint64, C.c_float, C.c_int32
        L.orc_num_threads.restype = C.c_int
        L.orc_minmax_serial.argtypes = [_f32p, u64, _f32p, _f32p]
        L.orc_minmax_seeded.argtypes = [_f32p, u64, _f32p, _f32p]
        L.orc_scale_symmetric.argtypes = [f32, f32]
        L.orc_scale_symmetric.restype = f32
        L.orc_params_asymmetric.argtypes = [f32, f32, _f32p, _i32p]
        L.orc_quantize_i8.argtypes = [_f32p, _i8p, u64, f32, i32]
        L.orc_quantize_symmetric.argtypes = [_f32p, _i8p, u64]
        L.orc_quantize_symmetric.restype = f32
        L.orc_quantize_asymmetric.argtypes = [_f32p, _i8p, u64, _f32p, _i32p]
        L.orc_quantize_per_channel.argtypes = [_f32p, _i8p, _f32p, _i32p, u64, u64]
        L.orc_dequantize_i8.argtypes = [_i8p, _f32p, u64, f32, i32]
        L.orc_dequantize_per_channel.argtypes = [_i8p, _f32p, _f32p, u64, u64]
        L.orc_gemm_i8_requant.argtypes = [_i8p, _i8p, _i32p, u64, u64, u64, f32, f32, f32, i32, i32]
        L.orc_linear_i8.argtypes = [_i8p, _i8p, _i8p, _i32p, u64, u64, u64]
        L.orc_linear_i8_dequant.argtypes = [_i8p, _i8p, _f32p, u64, u64, u64, u64, f32, _f32p, _f32p, C.c_int]
        L.orc_relu_inplace.argtypes = [_f32p, u64]
        self.L = L

    def num_threads(self):
        return int(self.L.orc_num_threads())

    def minmax_serial(self, x):
        x = _c(x, np.float32).ravel()
        mn, mx = C.c_float(np.nan), C.c_float(np.nan)
        self.L.orc_minmax_serial(_ptr(x, _f32p), x.size, C.byref(mn), C.byref(mx))
        return np.float32(mn.value), np.float32(mx.value)

    def minmax_seeded(self, x):
        x = _c(x, np.float32).ravel()
        mn, mx = C.c_float(), C.c_float()
        self.L.orc_minmax_seeded(_ptr(x, _f32p), x.size, C.byref(mn), C.byref(mx))
        return np.float32(mn.value), np.float32(mx.value)

    def scale_symmetric(self, mn, mx):
        return np.float32(self.L.orc_scale_symmetric(float(mn), float(mx)))

    def params_asymmetric(self, mn, mx):
        s, z = C.c_float(), C.c_int32()
        self.L.orc_params_asymmetric(float(mn), float(mx), C.byref(s), C.byref(z))
        return np.float32(s.value), int(z.value)

    def quantize(self, x, scale, zp=0):
        x = _c(x, np.float32)
        q = np.empty(x.shape, np.int8)
        self.L.orc_quantize_i8(_ptr(x, _f32p), _ptr(q, _i8p), x.size, float(scale), int(zp))
        return q

    def quantize_symmetric(self, x):
        x = _c(x, np.float32)
        q = np.empty(x.shape, np.int8)
        s = self.L.orc_quantize_symmetric(_ptr(x, _f32p), _ptr(q, _i8p), x.size)
        return q, np.float32(s)

    def quantize_asymmetric(self, x):
        x = _c(x, np.float32)
        q = np.empty(x.shape, np.int8)
        s, z = C.c_float(), C.c_int32()
        self.L.orc_quantize_asymmetric(_ptr(x, _f32p), _ptr(q, _i8p), x.size, C.byref(s), C.byref(z))
        return q, np.float32(s.value), int(z.value)

    def quantize_per_channel(self, x, num_channels):
        x = _c(x, np.float32)
        L = x.size // num_channels if num_channels else 0
        q = np.empty(x.shape, np.int8)
        scales = np.empty(num_channels, np.float32)
        zps = np.empty(num_channels, np.int32)
        self.L.orc_quantize_per_channel(_ptr(x, _f32p), _ptr(q, _i8p), _ptr(scales, _f32p),
                                        _ptr(zps, _i32p), num_channels, L)
        return q, scales, zps

    def dequantize(self, q, scale, zp=0):
        q = _c(q, np.int8)
        out = np.empty(q.shape, np.float32)
        self.L.orc_dequantize_i8(_ptr(q, _i8p), _ptr(out, _f32p), q.size, float(scale), int(zp))
        return out

    def dequantize_per_channel(self, q, scales):
        q = _c(q, np.int8)
        scales = _c(scales, np.float32)
        out = np.empty(q.shape, np.float32)
        self.L.orc_dequantize_per_channel(_ptr(q, _i8p), _ptr(scales, _f32p), _ptr(out, _f32p),
                                          scales.size, q.size // max(scales.size, 1))
        return out

    def gemm_requant(self, A, B, sa=1.0, sb=1.0, sc=1.0, za=0, zb=0):
        """A [M,K], B [K,N] -> int32 [M,N] (gemm_int8 semantics)."""
        A, B = _c(A, np.int8), _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.int32)
        self.L.orc_gemm_i8_requant(_ptr(A, _i8p), _ptr(B, _i8p), _ptr(out, _i32p), M, N, K,
                                   float(sa), float(sb), float(sc), int(za), int(zb))
        return out

    def linear(self, x, w, bias=None):
        """x [M,K], w [N,K], bias int8 [N] or None -> raw int32 [M,N] (linear_int8)."""
        x, w = _c(x, np.int8), _c(w, np.int8)
        M, K = x.shape
        N = w.shape[0]
        b = _c(bias, np.int8) if bias is not None else None
        out = np.empty((M, N), np.int32)
        self.L.orc_linear_i8(_ptr(x, _i8p), _ptr(w, _i8p), _ptr(b, _i8p), _ptr(out, _i32p), M, K, N)
        return out

    def linear_dequant(self, x, w, a_scale, w_scales, bias=None, relu=False):
        x, w = _c(x, np.int8), _c(w, np.int8)
        M, K = x.shape
        N = w.shape[0]
        ws = _c(w_scales, np.float32)
        b = _c(bias, np.float32) if bias is not None else None
        out = np.empty((M, N), np.float32)
        self.L.orc_linear_i8_dequant(_ptr(x, _i8p), _ptr(w, _i8p), _ptr(out, _f32p), M, K, N, N,
                                     float(a_scale), _ptr(ws, _f32p), _ptr(b, _f32p), int(bool(relu)))
        return out

    def relu(self, x):
        x = np.array(x, dtype=np.float32, copy=True)
        self.L.orc_relu_inplace(_ptr(x, _f32p), x.size)
        return x


# ---------------------------------------------------------------------------
# The compiled reference, called through its own ABI.
# ---------------------------------------------------------------------------
class RefTensor(C.Structure):
    """``Tensor`` of include/rpl.h:57-78 (sizeof 152 on x86-64)."""


RefTensor._fields_ = [
    ("data", _f32p), ("grad", _f32p), ("dims", C.c_uint32),
    ("shape", C.c_uint32 * MAX_DIMS), ("strides", C.c_uint32 * MAX_DIMS),
    ("size", C.c_uint32), ("requires_grad", C.c_bool),
    ("_allocation", C.c_void_p), ("_alloc_size", C.c_size_t),
    ("device", C.c_int), ("gpu_buffer", C.c_uint32),
    ("is_leaf", C.c_bool), ("parent1", C.c_void_p), ("parent2", C.c_void_p),
    ("backward_fn", C.c_void_p),
]


class RefQuantizedTensor(C.Structure):
    """``QuantizedTensor`` of include/rpl.h:167-174 (sizeof 56)."""
    _fields_ = [("data", _i8p), ("scale", C.c_float), ("zero_point", C.c_int32),
                ("size", C.c_uint32), ("dims", C.c_uint32), ("shape", C.c_uint32 * MAX_DIMS)]


class RefPerChannel(C.Structure):
    """``PerChannelQuantizedTensor`` of src/rpl_quantization.c:110-118."""
    _fields_ = [("data", _i8p), ("scales", _f32p), ("zero_points", _i32p),
                ("num_channels", C.c_uint32), ("channel_size", C.c_uint32),
                ("dims", C.c_uint32), ("shape", C.c_uint32 * MAX_DIMS)]


def ref_available():
    return os.path.exists(REF_SO)


class Ref:
    """The reference's own functions (scalar x86 branch), numpy in / numpy out."""

    def __init__(self):
        if not ref_available():
            raise FileNotFoundError(REF_SO)
        L = C.CDLL(REF_SO)
        TP, QP, PP = C.POINTER(RefTensor), C.POINTER(RefQuantizedTensor), C.POINTER(RefPerChannel)
        L.tensor_quantize_int8.argtypes = [TP, C.c_float, C.c_int32]
        L.tensor_quantize_int8.restype = QP
        L.tensor_quantize_int8_symmetric.argtypes = [TP]
        L.tensor_quantize_int8_symmetric.restype = QP
        L.tensor_quantize_int8_asymmetric.argtypes = [TP]
        L.tensor_quantize_int8_asymmetric.restype = QP
        L.tensor_quantize_per_channel.argtypes = [TP, C.c_uint32]
        L.tensor_quantize_per_channel.restype = PP
        L.per_channel_quantized_tensor_free.argtypes = [PP]
        L.quantized_tensor_free.argtypes = [QP]
        L.tensor_get_min_max.argtypes = [TP, _f32p, _f32p]
        L.tensor_dequantize_int8.argtypes = [QP]
        L.tensor_dequantize_int8.restype = TP
        L.tensor_free.argtypes = [TP]
        L.gemm_int8.argtypes = [_i8p, _i8p, _i32p, C.c_uint32, C.c_uint32, C.c_uint32,
                                C.c_float, C.c_float, C.c_float, C.c_int32, C.c_int32]
        L.linear_int8.argtypes = [QP, QP, QP, _i32p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.tensor_relu_inplace.argtypes = [TP]
        self.L = L

    @staticmethod
    def tensor(x):
        """A stack ``Tensor`` viewing ``x`` (kept alive by the caller)."""
        t = RefTensor()
        t.data = _ptr(x, _f32p)
        shape = x.shape if x.ndim else (1,)
        t.dims = len(shape)
        stride = 1
        for i in range(len(shape) - 1, -1, -1):
            t.shape[i] = shape[i]
            t.strides[i] = stride
            stride *= shape[i]
        t.size = x.size
        t.is_leaf = True
        return t

    @staticmethod
    def qtensor(q, scale=1.0, zp=0):
        t = RefQuantizedTensor()
        t.data = _ptr(q, _i8p)
        t.scale, t.zero_point, t.size = float(scale), int(zp), q.size
        shape = q.shape if q.ndim else (1,)
        t.dims = len(shape)
        for i, s in enumerate(shape):
            t.shape[i] = s
        return t

    def _take_qt(self, p, shape):
        qt = p.contents
        q = np.ctypeslib.as_array(qt.data, shape=(qt.size,)).copy().reshape(shape) if qt.size else np.empty(shape, np.int8)
        s, z = np.float32(qt.scale), int(qt.zero_point)
        self.L.quantized_tensor_free(p)
        return q, s, z

    def minmax(self, x):
        x = _c(x, np.float32)
        t = self.tensor(x)
        mn, mx = C.c_float(np.nan), C.c_float(np.nan)
        self.L.tensor_get_min_max(C.byref(t), C.byref(mn), C.byref(mx))
        return np.float32(mn.value), np.float32(mx.value)

    def quantize(self, x, scale, zp=0):
        x = _c(x, np.float32)
        t = self.tensor(x)
        return self._take_qt(self.L.tensor_quantize_int8(C.byref(t), float(scale), int(zp)), x.shape)[0]

    def quantize_symmetric(self, x):
        x = _c(x, np.float32)
        t = self.tensor(x)
        q, s, _ = self._take_qt(self.L.tensor_quantize_int8_symmetric(C.byref(t)), x.shape)
        return q, s

    def quantize_asymmetric(self, x):
        x = _c(x, np.float32)
        t = self.tensor(x)
        return self._take_qt(self.L.tensor_quantize_int8_asymmetric(C.byref(t)), x.shape)

    def quantize_per_channel(self, x, axis=0):
        x = _c(x, np.float32)
        t = self.tensor(x)
        p = self.L.tensor_quantize_per_channel(C.byref(t), int(axis))
        pc = p.contents
        n = pc.num_channels
        q = np.ctypeslib.as_array(pc.data, shape=(x.size,)).copy().reshape(x.shape)
        scales = np.ctypeslib.as_array(pc.scales, shape=(n,)).copy()
        zps = np.ctypeslib.as_array(pc.zero_points, shape=(n,)).copy()
        self.L.per_channel_quantized_tensor_free(p)
        return q, scales, zps

    def dequantize(self, q, scale, zp=0):
        q = _c(q, np.int8)
        qt = self.qtensor(q, scale, zp)
        p = self.L.tensor_dequantize_int8(C.byref(qt))
        out = np.ctypeslib.as_array(p.contents.data, shape=(q.size,)).copy().reshape(q.shape)
        self.L.tensor_free(p)
        return out

    def gemm_requant(self, A, B, sa=1.0, sb=1.0, sc=1.0, za=0, zb=0):
        A, B = _c(A, np.int8), _c(B, np.int8)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), np.int32)
        self.L.gemm_int8(_ptr(A, _i8p), _ptr(B, _i8p), _ptr(out, _i32p), M, N, K,
                         float(sa), float(sb), float(sc), int(za), int(zb))
        return out

    def linear(self, x, w, bias=None):
        x, w = _c(x, np.int8), _c(w, np.int8)
        M, K = x.shape
        N = w.shape[0]
        qx, qw = self.qtensor(x), self.qtensor(w)
        out = np.empty((M, N), np.int32)
        if bias is not None:
            b = _c(bias, np.int8)
            qb = self.qtensor(b)
            self.L.linear_int8(C.byref(qx), C.byref(qw), C.byref(qb), _ptr(out, _i32p), M, K, N)
        else:
            self.L.linear_int8(C.byref(qx), C.byref(qw), None, _ptr(out, _i32p), M, K, N)
        return out

    def relu(self, x):
        x = np.array(x, dtype=np.float32, copy=True)
        t = self.tensor(x)
        self.L.tensor_relu_inplace(C.byref(t))
        return x
