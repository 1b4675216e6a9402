"""gb_gemm_static_scratch: the split-K product for callers that may not allocate device memory.

A host on a fixed device-memory budget, or one whose arena is closed after start-up, cannot call cudaMalloc and so
can neither create a handle nor bring a workspace.  This entry point keeps its split-K partial sums in a
fixed array inside the library instead.  The test drives it through the C ABI on a shape that splits K,
twice in a row with different operands (the shared array keeps the first call's partials), and expects the
same bits as gb_gemm with a caller-owned workspace, which runs the identical plan.  It is collected last so
that a failure here cannot hide any other test under `-x`.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _desc(abi, m, n, k):
    d = abi.GemmDesc()
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.dtype_a = d.dtype_b = abi.BF16
    d.dtype_c = abi.F32
    d.math = abi.MATH_BF16
    return d


def test_static_scratch_matches_workspace_gemm_on_two_calls_in_a_row():
    import torch

    import grad_b200
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape, abi

    gpu = grad_b200.Gpu(0)
    lib = gpu.lib
    m, n, k = 256, 320, 4096            # 6 tiles on 148 SMs: the planner splits K
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(7)
    for call in range(2):
        a = torch.randn((m, k), generator=gen, device="cuda").bfloat16()
        b = torch.randn((k, n), generator=gen, device="cuda").bfloat16()
        bias = torch.randn(n, generator=gen, device="cuda")
        want = torch.empty((m, n), device="cuda")
        gpu.matmul(a, b, want, MatmulShape(m, n, k), MatmulOpts(), epilogue=Epilogue(bias, None, True))
        assert gpu.last_plan()["splits"] > 1, "the shape must exercise the scratch memory"
        got = torch.full((m, n), -1.0, device="cuda")
        d = _desc(abi, m, n, k)
        ep = abi.Epilogue(bias.data_ptr(), None, abi.ACT_RELU, 0)
        torch.cuda.synchronize()
        # Free bytes as the driver counts them (cudaMemGetInfo): a cudaMalloc inside the library would lower this,
        # whereas torch's own counters only see torch's caching allocator.  The first call may make the driver load
        # the kernels lazily, so the comparison brackets the second call.
        before = torch.cuda.mem_get_info()[0]
        rc = lib.gb_gemm_static_scratch(stream, C.byref(d), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()),
                                        C.c_void_p(got.data_ptr()), C.byref(ep))
        assert rc == 0, abi.error_string(rc)
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == before
        word = C.c_uint32(7)
        assert lib.gb_static_last_status(stream, C.byref(word)) == 0 and word.value == 0
        assert torch.equal(got, want), f"call {call}: max abs diff {(got - want).abs().max().item()}"
        ref = torch.relu(a.float() @ b.float() + bias)
        assert ((got - ref).norm() / ref.norm()).item() <= 2e-2
    gpu.check_status()
    gpu.close()


def test_static_scratch_on_the_strict_f32_split_path():
    """The strict-f32 kernels split K too (few tiles, long K) and their partial sums use the same fixed array."""
    import torch

    import grad_b200
    from grad_b200 import MatmulOpts, MatmulShape, abi

    gpu = grad_b200.Gpu(0)
    lib = gpu.lib
    m, n, k = 64, 128, 784              # the MLP's first product: two 64 x 64 tiles, K split three ways
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(11)
    for call in range(2):
        a = torch.randn((m, k), generator=gen, device="cuda")
        b = torch.randn((k, n), generator=gen, device="cuda")
        want = torch.empty((m, n), device="cuda")
        gpu.matmul(a, b, want, MatmulShape(m, n, k), MatmulOpts(), math=abi.MATH_F32)
        plan = gpu.last_plan()
        assert plan["tensor_path"] == 0 and plan["splits"] > 1, plan
        got = torch.full((m, n), -1.0, device="cuda")
        d = _desc(abi, m, n, k)
        d.dtype_a = d.dtype_b = abi.F32
        d.math = abi.MATH_F32
        rc = lib.gb_gemm_static_scratch(stream, C.byref(d), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(got.data_ptr()), None)
        assert rc == 0, abi.error_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: max abs diff {(got - want).abs().max().item()}"
        ref = a.double() @ b.double()
        assert ((got.double() - ref).norm() / ref.norm()).item() <= 1e-5
    gpu.check_status()
    gpu.close()


def test_static_scratch_rejects_partials_beyond_the_fixed_array():
    import torch

    import grad_b200
    from grad_b200 import abi

    lib = grad_b200.library()
    torch.cuda.set_device(0)
    # 74 row tiles of 128 x 64 (B is stored (K, N), so 64 is the narrowest tile) leave half of the 148 SMs idle, and
    # the planner splits K in two: 2 * 9472 * 64 * 4 bytes = 4.6 MiB of partials, more than the 4 MiB array.  The
    # ordinary entry point states that need, so the case stays honest when the planner changes.
    m, n, k = 9472, 64, 8192
    gpu = grad_b200.Gpu(0)
    need = C.c_size_t(0)
    assert lib.gb_gemm_workspace(gpu.handle, C.byref(_desc(abi, m, n, k)), C.byref(need)) == 0
    gpu.close()
    assert need.value > 4 << 20, need.value
    a = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((k, n), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((m, n), device="cuda")
    d = _desc(abi, m, n, k)
    rc = lib.gb_gemm_static_scratch(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(d), C.c_void_p(a.data_ptr()),
                                    C.c_void_p(b.data_ptr()), C.c_void_p(c.data_ptr()), None)
    assert rc == 3, rc                   # GB_ERR_WORKSPACE
    assert "workspace" in abi.error_string(rc)
    d.trans_a = d.trans_b = 1
    assert lib.gb_gemm_static_scratch(None, C.byref(d), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(c.data_ptr()), None) == 1
