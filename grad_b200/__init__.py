"""grad_b200: the dense-contraction path of hyunjun3952/grad (matmul family, implicit-GEMM conv2d,
gradient allreduce) as hand-written sm_100a CUDA behind a C ABI (``libgradb200.so``).

The Python layer is a host-side mirror of grad's ``Gpu`` wrappers (src/gpu/gpu.zig) used by the tests
and the benchmark; PyTorch only provides device memory and streams.  There is no CPU fallback: every
compute call goes through the C ABI and fails loudly when the CUDA library is missing.
"""
from .abi import (ACT_NONE, ACT_RELU, BF16, F32, MATH_BF16, MATH_F32, MATH_TF32, GbError, abi_version, error_string, library,
                  library_path)
from .gpu import ConvGeometry, Epilogue, Gpu, MatmulOpts, MatmulShape, PreparedWeights, conv_geometry

__all__ = ["ACT_NONE", "ACT_RELU", "BF16", "F32", "MATH_BF16", "MATH_F32", "MATH_TF32", "GbError", "abi_version", "error_string",
           "library", "library_path", "ConvGeometry", "Epilogue", "Gpu", "MatmulOpts", "MatmulShape", "PreparedWeights", "conv_geometry"]
