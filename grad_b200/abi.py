"""ctypes declarations of every entry point in include/gradb200.h.

This is the Python twin of the binding a grad maintainer would add in Zig (an ``Api`` struct of
``*const fn (...) callconv(.c)`` filled by ``dynlib.Library.bind``, as src/gpu/cudnn.zig:22-86 does for
cuDNN).  Loading fails loudly: a missing library or symbol raises, nothing falls back to another path.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))

F32, BF16 = 0, 1
MATH_F32, MATH_TF32, MATH_BF16 = 0, 1, 2
ACT_NONE, ACT_RELU = 0, 1
EPILOGUE_ROUND_TF32 = 1
PASS_FPROP, PASS_DGRAD, PASS_WGRAD = 0, 1, 2
WEIGHTS_PLAIN, WEIGHTS_ROWS = 0, 1

STATUS_NAMES = {0: "GB_OK", 1: "GB_ERR_INVALID", 2: "GB_ERR_CUDA", 3: "GB_ERR_WORKSPACE", 4: "GB_ERR_UNSUPPORTED",
                5: "GB_ERR_TIMEOUT", 6: "GB_ERR_NCCL", 7: "GB_ERR_NO_DEVICE"}


class GbError(RuntimeError):
    """A nonzero gb_status; mirrors the closed error set `gpu.Error` (src/gpu/gpu.zig:14)."""

    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {STATUS_NAMES.get(status, status)} ({error_string(status)})")


class BnStats(C.Structure):
    _fields_ = [("shift", C.c_void_p), ("sums", C.c_void_p), ("ordered", C.c_uint32), ("reserved", C.c_uint32)]


class DxStats(C.Structure):
    _fields_ = [("x", C.c_void_p), ("mean", C.c_void_p), ("inv_std", C.c_void_p), ("gamma", C.c_void_p), ("beta", C.c_void_p),
                ("sums", C.c_void_p), ("ordered", C.c_uint32), ("reserved", C.c_uint32)]


class AffineInput(C.Structure):
    _fields_ = [("mean", C.c_void_p), ("inv_std", C.c_void_p), ("gamma", C.c_void_p), ("beta", C.c_void_p)]


class Epilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("activation", C.c_int32), ("flags", C.c_int32), ("bn_stats", C.POINTER(BnStats))]


class GemmDesc(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("batch", C.c_uint32),
                ("stride_a", C.c_uint64), ("stride_b", C.c_uint64), ("stride_c", C.c_uint64),
                ("lda", C.c_uint32), ("ldb", C.c_uint32), ("ldc", C.c_uint32),
                ("trans_a", C.c_uint8), ("trans_b", C.c_uint8), ("accumulate", C.c_uint8), ("transpose_out", C.c_uint8),
                ("dtype_a", C.c_uint8), ("dtype_b", C.c_uint8), ("dtype_c", C.c_uint8), ("math", C.c_uint8),
                ("deterministic", C.c_uint8), ("reserved", C.c_uint8 * 3),
                ("batch_outer", C.c_uint32), ("reserved2", C.c_uint32),
                ("stride_a_outer", C.c_uint64), ("stride_b_outer", C.c_uint64), ("stride_c_outer", C.c_uint64)]


class ConvGeometryC(C.Structure):
    """Field-for-field `ConvGeometry` (src/gpu/args.zig:78)."""

    _fields_ = [(n, C.c_uint32) for n in ("n", "h", "w", "c", "k", "stride", "pad", "out_h", "out_w", "positions", "c_out",
                                          "dilation", "c_step", "subsample")]


class ConvDesc(C.Structure):
    _fields_ = [("geo", ConvGeometryC), ("dtype_x", C.c_uint8), ("dtype_w", C.c_uint8), ("dtype_y", C.c_uint8), ("math", C.c_uint8),
                ("accumulate", C.c_uint8), ("deterministic", C.c_uint8), ("w_layout", C.c_uint8), ("reserved", C.c_uint8), ("groups", C.c_uint32)]


class PlanInfo(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("tensor_path", "a_kind", "b_kind", "tile_m", "tile_n", "stages", "splits", "k_blocks",
                                          "work_items", "kernel_launches")]


# name -> (argtypes, restype): exactly the declarations of include/gradb200.h
SIGNATURES = {
    "gb_create": ([C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "gb_destroy": ([C.c_void_p], None),
    "gb_abi_version": ([], C.c_int),
    "gb_error_string": ([C.c_int], C.c_char_p),
    "gb_last_cuda_error": ([C.c_void_p], C.c_int),
    "gb_last_status": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)], C.c_int),
    "gb_sm_count": ([C.c_void_p], C.c_int),
    "gb_last_plan": ([C.c_void_p, C.POINTER(PlanInfo)], C.c_int),
    "gb_plan_cache_hits": ([C.c_void_p], C.c_uint64),
    "gb_weights_bytes": ([C.c_uint32, C.c_uint32, C.c_int], C.c_size_t),
    "gb_prepare_weights": ([C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)], C.c_int),
    "gb_refresh_weights": ([C.c_void_p, C.c_void_p], C.c_int),
    "gb_weights_data": ([C.c_void_p], C.c_void_p),
    "gb_weights_destroy": ([C.c_void_p], None),
    "gb_gemm_workspace": ([C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_size_t)], C.c_int),
    "gb_gemm": ([C.c_void_p, C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Epilogue), C.c_void_p,
                 C.c_size_t], C.c_int),
    "gb_gemm_static_scratch": ([C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Epilogue)], C.c_int),
    "gb_static_last_status": ([C.c_void_p, C.POINTER(C.c_uint32)], C.c_int),
    "gb_conv_workspace": ([C.c_void_p, C.c_int, C.POINTER(ConvDesc), C.POINTER(C.c_size_t)], C.c_int),
    "gb_conv_fprop": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Epilogue),
                       C.c_void_p, C.c_size_t], C.c_int),
    "gb_conv_dgrad": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t],
                      C.c_int),
    "gb_conv_fprop_affine": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Epilogue),
                              C.POINTER(AffineInput), C.c_void_p, C.c_size_t], C.c_int),
    "gb_conv_wgrad_affine": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(AffineInput), C.c_void_p,
                              C.c_size_t], C.c_int),
    "gb_conv_dgrad_stats": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(DxStats), C.c_void_p,
                             C.c_size_t], C.c_int),
    "gb_conv_wgrad": ([C.c_void_p, C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t],
                      C.c_int),
    "gb_pool2d": ([C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p] + [C.c_uint32] * 7, C.c_int),
    "gb_elementwise": ([C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint32], C.c_int),
    "gb_cast": ([C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t], C.c_int),
    "gb_reorder_oihw": ([C.c_void_p, C.c_int, C.c_void_p, C.c_void_p] + [C.c_uint32] * 4, C.c_int),
    "gb_reorder_oihw_rows": ([C.c_void_p, C.c_int, C.c_void_p, C.c_void_p] + [C.c_uint32] * 4, C.c_int),
    "gb_permute_layout": ([C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p] + [C.c_uint32] * 4, C.c_int),
    "gb_comm_unique_id": ([C.c_void_p], C.c_int),
    "gb_comm_create": ([C.c_int, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "gb_allreduce_mean": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t], C.c_int),
    "gb_comm_set_timeout": ([C.c_void_p, C.c_uint32], C.c_int),
    "gb_comm_finish": ([C.c_void_p, C.c_void_p], C.c_int),
    "gb_comm_abort": ([C.c_void_p], C.c_int),
    "gb_comm_destroy": ([C.c_void_p], None),
}

_lib = None


def library_path() -> str:
    """The library next to this file, or the one GB_LIBRARY names (a build with other compile-time options)."""
    return os.environ.get("GB_LIBRARY") or os.path.join(HERE, "libgradb200.so")


def library() -> C.CDLL:
    """dlopen + bind every symbol; raises when the library or a symbol is missing."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built: run `python -m grad_b200.build` (needs nvcc); there is no fallback path")
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (args, res) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError = error.MissingSymbol
            fn.argtypes = args
            fn.restype = res
        _lib = lib
    return _lib


def abi_version() -> int:
    return int(library().gb_abi_version())


def error_string(status: int) -> str:
    return library().gb_error_string(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != 0:
        raise GbError(status, where)
