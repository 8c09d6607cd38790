"""The ``rplb_*`` device-level entry points over torch CUDA tensors.

torch is used here for device memory and streams only: every function passes
``data_ptr()`` values and the current CUDA stream to ``librpl.so`` and returns
without synchronising.  Nothing in this module computes on the host, and there
is no fallback: a missing library or a non-CUDA tensor is an error.
"""
import ctypes as C

import torch

from . import capi


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _need(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor (librpl has no CPU path)" % name)
    if t.dtype != dtype:
        raise TypeError("%s must be %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    return t


def launch_count():
    return int(capi.load().rplb_launch_count())


def gemm_backend(which):
    """0 automatic, 1 dp4a, 2 tcgen05 (3 = 128x256 tiles, 4 = CTA-pair 256x256 tiles, 5 = 256x256 tiles per CTA,
    6 = the kernel for few output features);
    returns the previous setting."""
    return int(capi.load().rplb_gemm_backend(int(which)))


def gemm_epilogue(which):
    """0 = four-byte outputs leave through TMA tensor stores when the output allows it, 1 = always
    stored from registers; returns the previous setting (per host thread)."""
    return int(capi.load().rplb_gemm_epilogue(int(which)))


def kernel_status(clear=True):
    return int(capi.load().rplb_kernel_status(1 if clear else 0))


# --------------------------------------------------------------------------- quantize / dequantize
def minmax(x, params=None):
    """Device ``rplb_qparams`` (8 words) of ``x``: see ``QPARAM_*`` indices."""
    _need(x, torch.float32, "x")
    if params is None:
        params = torch.empty(8, dtype=torch.float32, device=x.device)
    capi.call("rplb_minmax_f32", _p(x), x.numel(), _p(params), _stream())
    return params


def qparams_to_pair(params, pair=None):
    """(-min, max) of a device ``rplb_qparams`` as two device floats, ready for a max-reduction across ranks."""
    if pair is None:
        pair = torch.empty(2, dtype=torch.float32, device=params.device)
    capi.call("rplb_qparams_to_pair", _p(params), _p(pair), _stream())
    return pair


def qparams_from_pair(pair, params):
    """All parameters (scales, zero point) from a combined (-min, max) pair, as the min/max kernel derives them."""
    capi.call("rplb_qparams_from_pair", _p(pair), _p(params), _stream())
    return params


QPARAM_MIN, QPARAM_MAX, QPARAM_SCALE_SYM, QPARAM_SCALE_ASYM, QPARAM_ZP_ASYM = 0, 1, 2, 3, 4
QPARAM_FIRST, QPARAM_TRUE_MIN, QPARAM_TRUE_MAX = 5, 6, 7


def quantize(x, scale, zero_point=0, out=None):
    """tensor_quantize_int8 with a host scale / zero point."""
    _need(x, torch.float32, "x")
    q = out if out is not None else torch.empty(x.shape, dtype=torch.int8, device=x.device)
    capi.call("rplb_quantize_f32_i8", _p(x), _p(q), x.numel(), float(scale), int(zero_point), _stream())
    return q


def quantize_dev(x, scale_dev, zp_dev=None, out=None):
    """Same with the scale (and zero point) read from device memory."""
    _need(x, torch.float32, "x")
    q = out if out is not None else torch.empty(x.shape, dtype=torch.int8, device=x.device)
    capi.call("rplb_quantize_f32_i8_dev", _p(x), _p(q), x.numel(), _p(scale_dev), _p(zp_dev), _stream())
    return q


def quantize_symmetric(x, out=None, params=None):
    """tensor_quantize_int8_symmetric.  Returns (q, params); the scale is
    ``params[QPARAM_SCALE_SYM]`` and stays on the device."""
    _need(x, torch.float32, "x")
    q = out if out is not None else torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if params is None:
        params = torch.empty(8, dtype=torch.float32, device=x.device)
    capi.call("rplb_quantize_symmetric_f32_i8", _p(x), _p(q), x.numel(), _p(params), _stream())
    return q, params


def quantize_asymmetric(x, out=None, params=None):
    """tensor_quantize_int8_asymmetric.  Scale ``params[QPARAM_SCALE_ASYM]``,
    zero point ``params.view(torch.int32)[QPARAM_ZP_ASYM]``."""
    _need(x, torch.float32, "x")
    q = out if out is not None else torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if params is None:
        params = torch.empty(8, dtype=torch.float32, device=x.device)
    capi.call("rplb_quantize_asymmetric_f32_i8", _p(x), _p(q), x.numel(), _p(params), _stream())
    return q, params


def quantize_per_channel(x, num_channels=None, out=None):
    """tensor_quantize_per_channel: channels are contiguous blocks (rows of a 2-D weight)."""
    _need(x, torch.float32, "x")
    Cn = int(num_channels if num_channels is not None else x.shape[0])
    L = x.numel() // Cn if Cn else 0
    q = out if out is not None else torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scales = torch.empty(Cn, dtype=torch.float32, device=x.device)
    zps = torch.empty(Cn, dtype=torch.int32, device=x.device)
    capi.call("rplb_quantize_per_channel_f32_i8", _p(x), _p(q), _p(scales), _p(zps), Cn, L, _stream())
    return q, scales, zps


def dequantize(q, scale, zero_point=0, out=None):
    _need(q, torch.int8, "q")
    o = out if out is not None else torch.empty(q.shape, dtype=torch.float32, device=q.device)
    capi.call("rplb_dequantize_i8_f32", _p(q), _p(o), q.numel(), float(scale), int(zero_point), _stream())
    return o


def dequantize_per_channel(q, scales, out=None):
    _need(q, torch.int8, "q")
    _need(scales, torch.float32, "scales")
    Cn = scales.numel()
    o = out if out is not None else torch.empty(q.shape, dtype=torch.float32, device=q.device)
    capi.call("rplb_dequantize_per_channel_i8_f32", _p(q), _p(scales), _p(o), Cn, q.numel() // max(Cn, 1), _stream())
    return o


def relu_(x):
    _need(x, torch.float32, "x")
    capi.call("rplb_relu_f32_inplace", _p(x), x.numel(), _stream())
    return x


# --------------------------------------------------------------------------- contraction
def linear_i8(x, w, bias=None, out=None):
    """linear_int8: x [M,K] int8, w [N,K] int8, optional int8 bias [N] -> raw int32 [M,N]."""
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError("w must be [N, K] with K = %d" % K)
    if bias is not None:
        _need(bias, torch.int8, "bias")
    o = out if out is not None else torch.empty((M, N), dtype=torch.int32, device=x.device)
    capi.call("rplb_linear_i8_i32", _p(x), _p(w), _p(bias), _p(o), M, K, N, _stream())
    return o


def gemm_i8_requant(A, B, sa=1.0, sb=1.0, sc=1.0, za=0, zb=0, out=None):
    """gemm_int8: A [M,K], B [K,N] -> int32 [M,N] = roundf(sum*sa*sb/sc)."""
    _need(A, torch.int8, "A")
    _need(B, torch.int8, "B")
    M, K = A.shape
    N = B.shape[1]
    if B.shape[0] != K:
        raise ValueError("B must be [K, N] with K = %d" % K)
    o = out if out is not None else torch.empty((M, N), dtype=torch.int32, device=A.device)
    capi.call("rplb_gemm_i8_requant_i32", _p(A), _p(B), _p(o), M, N, K, float(sa), float(sb), float(sc),
              int(za), int(zb), _stream())
    return o


def linear_i8_dequant(x, w, a_scale, w_scales, bias=None, relu=False, out=None):
    """Fused fp32 epilogue: out = relu?(((float)acc * a_scale) * w_scales[n] + bias[n]).

    ``a_scale`` is a one-element CUDA tensor (e.g. ``params[2:3]``).  ``out`` may
    be a column block of a wider row-major matrix (its row stride is passed on).
    """
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    if not (isinstance(a_scale, torch.Tensor) and a_scale.is_cuda and a_scale.dtype == torch.float32):
        raise TypeError("a_scale must be a float32 CUDA tensor with one element")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError("w must be [N, K] with K = %d" % K)
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    else:
        if out.dtype != torch.float32 or not out.is_cuda or out.shape != (M, N) or out.stride(1) != 1:
            raise ValueError("out must be a float32 CUDA [M,N] view with unit column stride")
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    capi.call("rplb_linear_i8_dequant_f32", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales),
              _p(bias), 1 if relu else 0, _stream())
    return out


def linear_i8_dequant_peers(x, w, a_scale, w_scales, out, peer_ptrs, bias=None, relu=False):
    """``linear_i8_dequant`` whose values are also stored, at the same offsets and row
    stride, into further buffers given by raw device addresses (``peer_ptrs``: other
    ranks' outputs opened with ``rplb_ipc_open``, each advanced to this rank's first
    column).  The caller orders the ranks around the call."""
    import ctypes as C
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError("w must be [N, K] with K = %d" % K)
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out.dtype != torch.float32 or not out.is_cuda or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("out must be a float32 CUDA [M,N] view with unit column stride")
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    ptrs = (C.c_void_p * max(1, len(peer_ptrs)))(*[int(q) for q in peer_ptrs])
    capi.call("rplb_linear_i8_dequant_f32_peers", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales),
              _p(bias), 1 if relu else 0, ptrs, len(peer_ptrs), _stream())
    return out


def linear_i8_dequant_arriving(x, w, a_scale, w_scales, ready, epoch, local_first_block, local_blocks,
                               bias=None, relu=False, out=None):
    """``linear_i8_dequant`` over an activation whose 128-row blocks may still be arriving from other
    GPUs: ``ready`` is an int32/uint32 CUDA tensor with one word per block, a block is complete once its
    word has reached ``epoch``; blocks ``[local_first_block, +local_blocks)`` are complete at launch."""
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    M, K = x.shape
    N = w.shape[0]
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    capi.call("rplb_linear_i8_dequant_f32_arriving", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales),
              _p(bias), 1 if relu else 0, _p(ready), int(epoch) & 0xFFFFFFFF, int(local_first_block), int(local_blocks), _stream())
    return out


def linear_i8_dequant_absmax(x, w, a_scale, w_scales, bias=None, relu=False, out=None):
    """``linear_i8_dequant`` that also returns ``(absmax, next_scale)``: max |out| and
    absmax / 127, the per-tensor symmetric scale of ``out``, both one-element device
    tensors, so the next layer can quantize ``out`` without a min/max pass."""
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    M, K = x.shape
    N = w.shape[0]
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    stats = torch.empty(2, dtype=torch.float32, device=x.device)
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    capi.call("rplb_linear_i8_dequant_f32_absmax", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales),
              _p(bias), 1 if relu else 0, _p(stats[0:1]), _p(stats[1:2]), _stream())
    return out, stats[0:1], stats[1:2]


def quantize_linear_dequant(x, w, a_scale, w_scales, bias=None, relu=False, out=None, stats=None):
    """Quantize fused into the layer: ``x`` is fp32 ``[M,K]``, quantized with the device scalar ``a_scale`` on
    its way into the contraction; otherwise as ``linear_i8_dequant``.  With ``stats`` (a 2-element float32 CUDA
    tensor) the call also leaves max |out| and max |out| / 127 there.  Few output features only (see
    ``rplb_quantize_linear_dequant_f32``); other shapes raise ``RplError`` with code ``RPLB_E_UNSUPPORTED``."""
    _need(x, torch.float32, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError("w must be [N, K] with K = %d" % K)
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    capi.call("rplb_quantize_linear_dequant_f32", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales), _p(bias),
              1 if relu else 0, _p(stats[0:1]) if stats is not None else None, _p(stats[1:2]) if stats is not None else None,
              _stream())
    return out


def linear_i8_requant_i8(x, w, a_scale, w_scales, out_scale, out_zero_point=0, bias=None, relu=False, out=None):
    """Fused layer with int8 output: the fp32 epilogue value quantized with a given
    (calibrated) scale, as tensor_quantize_int8 would; ``out_scale`` is a one-element
    device tensor."""
    _need(x, torch.int8, "x")
    _need(w, torch.int8, "w")
    _need(w_scales, torch.float32, "w_scales")
    M, K = x.shape
    N = w.shape[0]
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=x.device)
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    capi.call("rplb_linear_i8_requant_i8", _p(x), _p(w), _p(out), M, K, N, ldo, _p(a_scale), _p(w_scales),
              _p(bias), 1 if relu else 0, _p(out_scale), int(out_zero_point), _stream())
    return out
