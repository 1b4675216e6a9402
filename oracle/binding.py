"""ctypes binding of the CPU oracle (``libgrad_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; never by the product package.
The C++ behind it restates the reference's CPU backend (src/cpu/kernels.zig, src/cpu/ops.zig,
src/gpu/math/conv.zig, src/gpu/math/bf16.zig, src/onnx/runtime.zig, src/nn/replicas.zig).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgrad_oracle.so")


def build(force: bool = False) -> str:
    """Compiles the oracle with the Makefile beside it when the library is missing or stale."""
    srcs = [os.path.join(_HERE, f) for f in ("grad_oracle.cpp", "grad_oracle.h")]
    stale = (not os.path.exists(_LIB_PATH)) or any(os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)
    return _LIB_PATH


class Dims(C.Structure):
    """src/gpu/math/conv.zig:22 ``Dims`` (n, h, w, c, k, stride, pad, dilation, groups, c_out)."""

    _fields_ = [(n, C.c_uint32) for n in ("n", "h", "w", "c", "k", "stride", "pad", "dilation", "groups", "c_out")]


@dataclass
class ConvDims:
    n: int
    h: int
    w: int
    c: int
    k: int
    stride: int = 1
    pad: int = 0
    dilation: int = 1
    groups: int = 1
    c_out: int = 0

    def c_struct(self) -> Dims:
        return Dims(self.n, self.h, self.w, self.c, self.k, self.stride, self.pad, self.dilation, self.groups, self.c_out)

    @property
    def out_h(self) -> int:
        return (self.h + 2 * self.pad - self.dilation * (self.k - 1) - 1) // self.stride + 1

    @property
    def out_w(self) -> int:
        return (self.w + 2 * self.pad - self.dilation * (self.k - 1) - 1) // self.stride + 1

    @property
    def rows(self) -> int:
        return self.n * self.out_h * self.out_w

    @property
    def taps(self) -> int:
        return self.k * self.k * self.c


_lib = None
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u16p = C.POINTER(C.c_uint16)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        z, i, f = C.c_size_t, C.c_int, C.c_float
        dp = C.POINTER(Dims)
        sig = {
            "oracle_bf16_encode": ([f], C.c_uint16),
            "oracle_bf16_decode": ([C.c_uint16], f),
            "oracle_bf16_round_array": ([_f32p, _f32p, z], None),
            "oracle_bf16_encode_array": ([_f32p, _u16p, z], None),
            "oracle_bf16_decode_array": ([_u16p, _f32p, z], None),
            "oracle_tf32_round": ([f], f),
            "oracle_tf32_round_array": ([_f32p, _f32p, z], None),
            "oracle_matmul_naive_f32": ([z, z, z, _f32p, _f32p, _f32p], None),
            "oracle_matmul_naive_f64": ([z, z, z, _f64p, _f64p, _f64p], None),
            "oracle_matmul_tiled_f32": ([z, z, z, _f32p, _f32p, _f32p, i, i, i, i], None),
            "oracle_matmul_tiled_f64": ([z, z, z, _f64p, _f64p, _f64p, i, i, i, i], None),
            "oracle_matmul_tiled_cfg_f32": ([z, z, z, _f32p, _f32p, _f32p, i, i, i, i, z, z, z, z, z], None),
            "oracle_split_for": ([z, z, z, i, C.POINTER(z), C.POINTER(z)], i),
            "oracle_out_height": ([dp], C.c_uint32),
            "oracle_out_width": ([dp], C.c_uint32),
            "oracle_im2col_elements": ([_f32p, _f32p, dp], None),
            "oracle_col2im_elements": ([_f32p, _f32p, dp], None),
            "oracle_im2col_rows": ([_f32p, _f32p, dp, z, z, i], None),
            "oracle_col2im_pixels": ([_f32p, _f32p, dp, i], None),
            "oracle_conv_forward": ([_f32p, _f32p, _f32p, dp, i], None),
            "oracle_conv_input_grad": ([_f32p, _f32p, _f32p, dp, i], None),
            "oracle_conv_weight_grad": ([_f32p, _f32p, _f32p, dp, i], None),
            "oracle_conv_grouped_forward": ([_f32p, _f32p, _f32p, dp], None),
            "oracle_conv_grouped_input_grad": ([_f32p, _f32p, _f32p, dp], None),
            "oracle_conv_grouped_weight_grad": ([_f32p, _f32p, _f32p, dp], None),
            "oracle_conv_direct_f64": ([_f32p, _f32p, _f64p, dp], None),
            "oracle_reorder_oihw": ([_f32p, _f32p, z, z, z, z], None),
            "oracle_convolve_nhwc": ([_f32p, _f32p, _f32p, _f32p, dp, i], None),
            "oracle_convolve_nchw": ([_f32p, _f32p, _f32p, _f32p, z, z, z, z, z, z, z, z, z, z, z, i], None),
            "oracle_onnx_matmul": ([_f32p, _f32p, _f32p, z, z, z, z, z, i], None),
            "oracle_onnx_gemm": ([_f32p, _f32p, _f32p, _f32p, z, z, z, i, i, f, f, i], None),
            "oracle_relu": ([_f32p, z], None),
            "oracle_bias_act": ([_f32p, _f32p, z, z, i], None),
            "oracle_average_grads": ([_f32p, z, z], None),
            "oracle_host_threads": ([], i),
            "oracle_vector_lanes": ([], i),
        }
        for name, (args, res) in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    if a is None:
        return None
    if a.dtype == np.float32:
        return a.ctypes.data_as(_f32p)
    if a.dtype == np.float64:
        return a.ctypes.data_as(_f64p)
    if a.dtype == np.uint16:
        return a.ctypes.data_as(_u16p)
    raise TypeError(a.dtype)


def host_threads() -> int:
    return int(lib().oracle_host_threads())


def vector_lanes() -> int:
    return int(lib().oracle_vector_lanes())


# ---- bf16 / tf32 ------------------------------------------------------------------------------
def bf16_encode(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_bf16_encode_array(_p(x), _p(out), x.size)
    return out


def bf16_decode(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().oracle_bf16_decode_array(_p(h), _p(out), h.size)
    return out


def bf16_round(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_bf16_round_array(_p(x), _p(out), x.size)
    return out


def tf32_round(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_tf32_round_array(_p(x), _p(out), x.size)
    return out


# ---- matmul -----------------------------------------------------------------------------------
def matmul_naive(a, b) -> np.ndarray:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), a.dtype)
    fn = lib().oracle_matmul_naive_f64 if a.dtype == np.float64 else lib().oracle_matmul_naive_f32
    fn(m, k, n, _p(a), _p(b), _p(out))
    return out


def matmul_tiled(a, b, m, k, n, trans_a=False, trans_b=False, out=None, threads=1, cfg=None) -> np.ndarray:
    """``a`` and ``b`` are the STORED operands: a is (m,k) or (k,m) when trans_a; b is (k,n) or (n,k) when trans_b.
    ``out`` given means accumulate into it (in place on a float copy of the same dtype)."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    accumulate = out is not None
    if out is None:
        out = np.full((m, n), 99, a.dtype)
    assert out.flags.c_contiguous and out.dtype == a.dtype
    if cfg is not None:
        assert a.dtype == np.float32
        lib().oracle_matmul_tiled_cfg_f32(m, k, n, _p(a), _p(b), _p(out), int(trans_a), int(trans_b), int(accumulate), threads, *cfg)
    elif a.dtype == np.float64:
        lib().oracle_matmul_tiled_f64(m, k, n, _p(a), _p(b), _p(out), int(trans_a), int(trans_b), int(accumulate), threads)
    else:
        lib().oracle_matmul_tiled_f32(m, k, n, _p(a), _p(b), _p(out), int(trans_a), int(trans_b), int(accumulate), threads)
    return out


def split_for(m, k, n, threads):
    parts, chunk = C.c_size_t(), C.c_size_t()
    axis = lib().oracle_split_for(m, k, n, threads, C.byref(parts), C.byref(chunk))
    return ("rows", "cols", "depth")[axis], parts.value, chunk.value


# ---- convolution ------------------------------------------------------------------------------
def im2col_elements(x, d: ConvDims) -> np.ndarray:
    x = _f32(x)
    col = np.empty((d.rows, d.taps), np.float32)
    ds = d.c_struct()
    lib().oracle_im2col_elements(_p(x), _p(col), C.byref(ds))
    return col


def im2col_rows(x, d: ConvDims, threads=1) -> np.ndarray:
    x = _f32(x)
    col = np.full((d.rows, d.taps), 99, np.float32)
    ds = d.c_struct()
    lib().oracle_im2col_rows(_p(x), _p(col), C.byref(ds), 0, d.rows, threads)
    return col


def col2im_elements(dcol, d: ConvDims) -> np.ndarray:
    dcol = _f32(dcol)
    dx = np.zeros((d.n, d.h, d.w, d.c), np.float32)
    ds = d.c_struct()
    lib().oracle_col2im_elements(_p(dcol), _p(dx), C.byref(ds))
    return dx


def col2im_pixels(dcol, d: ConvDims, threads=1) -> np.ndarray:
    dcol = _f32(dcol)
    dx = np.zeros((d.n, d.h, d.w, d.c), np.float32)
    ds = d.c_struct()
    lib().oracle_col2im_pixels(_p(dcol), _p(dx), C.byref(ds), threads)
    return dx


def conv_forward(x, w, d: ConvDims, threads=1) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty((d.n, d.out_h, d.out_w, d.c_out), np.float32)
    ds = d.c_struct()
    if d.groups > 1:
        lib().oracle_conv_grouped_forward(_p(x), _p(w), _p(out), C.byref(ds))
    else:
        lib().oracle_conv_forward(_p(x), _p(w), _p(out), C.byref(ds), threads)
    return out


def conv_input_grad(dy, w, d: ConvDims, threads=1, dx=None) -> np.ndarray:
    dy, w = _f32(dy), _f32(w)
    if dx is None:
        dx = np.zeros((d.n, d.h, d.w, d.c), np.float32)
    ds = d.c_struct()
    if d.groups > 1:
        lib().oracle_conv_grouped_input_grad(_p(dy), _p(w), _p(dx), C.byref(ds))
    else:
        lib().oracle_conv_input_grad(_p(dy), _p(w), _p(dx), C.byref(ds), threads)
    return dx


def conv_weight_grad(x, dy, d: ConvDims, threads=1, dw=None) -> np.ndarray:
    x, dy = _f32(x), _f32(dy)
    if dw is None:
        dw = np.zeros((d.k * d.k * (d.c // d.groups), d.c_out), np.float32)
    ds = d.c_struct()
    if d.groups > 1:
        lib().oracle_conv_grouped_weight_grad(_p(x), _p(dy), _p(dw), C.byref(ds))
    else:
        lib().oracle_conv_weight_grad(_p(x), _p(dy), _p(dw), C.byref(ds), threads)
    return dw


def conv_direct_f64(x, w, d: ConvDims) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty((d.n, d.out_h, d.out_w, d.c_out), np.float64)
    ds = d.c_struct()
    lib().oracle_conv_direct_f64(_p(x), _p(w), _p(out), C.byref(ds))
    return out


def reorder_oihw(w) -> np.ndarray:
    w = _f32(w)
    m, c, kh, kw = w.shape
    wt = np.empty((kh * kw * c, m), np.float32)
    lib().oracle_reorder_oihw(_p(w), _p(wt), m, c, kh, kw)
    return wt


def convolve_nhwc(x, w_oihw, bias, d: ConvDims, threads=1) -> np.ndarray:
    x, w = _f32(x), _f32(w_oihw)
    b = None if bias is None else _f32(bias)
    out = np.empty((d.n, d.out_h, d.out_w, d.c_out), np.float32)
    ds = d.c_struct()
    lib().oracle_convolve_nhwc(_p(x), _p(w), _p(b) if b is not None else None, _p(out), C.byref(ds), threads)
    return out


def convolve_nchw(x, w_oihw, bias=None, groups=1, stride=1, pad=0, dilation=1, threads=1) -> np.ndarray:
    x, w = _f32(x), _f32(w_oihw)
    n, c, h, width = x.shape
    m, _, kh, kw = w.shape
    oh = (h + 2 * pad - dilation * (kh - 1) - 1) // stride + 1
    ow = (width + 2 * pad - dilation * (kw - 1) - 1) // stride + 1
    b = None if bias is None else _f32(bias)
    out = np.empty((n, m, oh, ow), np.float32)
    lib().oracle_convolve_nchw(_p(x), _p(w), _p(b) if b is not None else None, _p(out), n, c, h, width, m, kh, kw,
                               groups, stride, pad, dilation, threads)
    return out


def onnx_matmul(x, y, threads=1) -> np.ndarray:
    x, y = _f32(x), _f32(y)
    m, k = x.shape[-2:]
    n = y.shape[-1]
    batch = int(np.prod(x.shape[:-2], dtype=np.int64)) if x.ndim > 2 else 1
    wb = int(np.prod(y.shape[:-2], dtype=np.int64)) if y.ndim > 2 else 1
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    lib().oracle_onnx_matmul(_p(x), _p(y), _p(out), batch, wb, m, k, n, threads)
    return out


def onnx_gemm(x, y, c=None, trans_a=False, trans_b=False, alpha=1.0, beta=1.0, threads=1) -> np.ndarray:
    x, y = _f32(x), _f32(y)
    m, k = (x.shape[1], x.shape[0]) if trans_a else x.shape
    n = y.shape[0] if trans_b else y.shape[1]
    cc = None if c is None else _f32(c)
    out = np.empty((m, n), np.float32)
    lib().oracle_onnx_gemm(_p(x), _p(y), _p(cc) if cc is not None else None, _p(out), m, k, n, int(trans_a), int(trans_b),
                           alpha, beta, threads)
    return out


def relu(v) -> np.ndarray:
    v = _f32(v).copy()
    lib().oracle_relu(_p(v), v.size)
    return v


def bias_act(out, bias, relu_flag: bool) -> np.ndarray:
    out = _f32(out).copy()
    rows, cols = out.reshape(-1, out.shape[-1]).shape
    b = None if bias is None else _f32(bias)
    lib().oracle_bias_act(_p(out), _p(b) if b is not None else None, rows, cols, int(relu_flag))
    return out


def average_grads(grads) -> np.ndarray:
    g = _f32(grads).copy()
    replicas, length = g.shape
    lib().oracle_average_grads(_p(g), replicas, length)
    return g
