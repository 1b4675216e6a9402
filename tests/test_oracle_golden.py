"""Pins the CPU oracle to the reference's own known-answer tests and exact-equality properties.

Each test names the reference test it replays (paths are within hyunjun3952/grad).  The reference
cannot be built here (it is Zig), so these vectors and properties are what makes the oracle's
parity "pinned" rather than asserted.
"""
import numpy as np
import pytest

from oracle import binding as orc
from oracle.binding import ConvDims


def _pattern(count, mod, shift, dtype=np.float32):
    return ((np.arange(count) % mod) - shift).astype(dtype)


# ---- tests/tensor.zig:32-43, 91-104 -------------------------------------------------------------
def test_known_answer_2x3_times_3x2():
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    assert orc.matmul_tiled(a, b, 2, 3, 2).ravel().tolist() == [58, 64, 139, 154]
    assert orc.matmul_naive(a, b).ravel().tolist() == [58, 64, 139, 154]
    out = np.ones((2, 2), np.float32)
    orc.matmul_tiled(a, b, 2, 3, 2, out=out)
    assert out.ravel().tolist() == [59, 65, 140, 155]
    assert orc.matmul_tiled(a, b, 2, 3, 2).ravel().tolist() == [58, 64, 139, 154]


# ---- tests/tensor.zig:45-114 (inputs i%7, i%5 on the STORED operands) ---------------------------
@pytest.mark.parametrize("m,k,n", [(7, 5, 3), (50, 64, 33), (190, 192, 191), (200, 193, 197), (257, 130, 100), (1, 9, 1)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_tiled_equals_naive_on_stored_patterns(m, k, n, ta, tb):
    a = _pattern(m * k, 7, 0).reshape((k, m) if ta else (m, k))
    b = _pattern(k * n, 5, 0).reshape((n, k) if tb else (k, n))
    la = a.T.copy() if ta else a
    lb = b.T.copy() if tb else b
    want = orc.matmul_naive(la, lb)
    got = orc.matmul_tiled(a, b, m, k, n, ta, tb)
    assert np.array_equal(want, got)


# ---- tests/kernels.zig:27-85, 142-148 -----------------------------------------------------------
def _expect_same_result(dtype, threads, m, k, n):
    a = _pattern(m * k, 7, 3, dtype).reshape(m, k)
    b = _pattern(k * n, 5, 2, dtype).reshape(k, n)
    want = orc.matmul_naive(a, b)
    at, bt = a.T.copy(), b.T.copy()
    lanes = orc.vector_lanes()
    cfgs = [None]
    if dtype == np.float32:
        cfgs.append((4, 2, 8, 5, 4 * lanes))   # the "small" TileConfig of tests/kernels.zig:60
    for cfg in cfgs:
        for ta, tb in [(False, False), (True, False), (False, True), (True, True)]:
            got = orc.matmul_tiled(at if ta else a, bt if tb else b, m, k, n, ta, tb, threads=threads, cfg=cfg)
            assert np.array_equal(want, got), (m, k, n, ta, tb, cfg)


def test_split_directions_match_reference_expectations():
    assert orc.split_for(200, 193, 197, 4)[0] == "rows" and orc.split_for(200, 193, 197, 4)[1] > 1
    assert orc.split_for(150, 200, 260, 4)[0] == "cols" and orc.split_for(150, 200, 260, 4)[1] > 1
    assert orc.split_for(12, 40000, 10, 4)[0] == "depth" and orc.split_for(12, 40000, 10, 4)[1] > 1


@pytest.mark.parametrize("dtype,m,k,n", [(np.float32, 200, 193, 197), (np.float32, 150, 200, 260), (np.float64, 120, 150, 140),
                                         (np.float32, 12, 40000, 10), (np.float64, 6, 200001, 4)])
def test_parallel_tiled_matches_in_every_split_direction(dtype, m, k, n):
    _expect_same_result(dtype, 4, m, k, n)


def test_depth_split_accumulates():
    m, k, n = 12, 40000, 10
    a = _pattern(m * k, 7, 3).reshape(m, k)
    b = _pattern(k * n, 5, 2).reshape(k, n)
    want = orc.matmul_naive(a, b) + 1
    got = np.ones((m, n), np.float32)
    orc.matmul_tiled(a, b, m, k, n, out=got, threads=4)
    assert np.array_equal(want, got)


@pytest.mark.parametrize("shape", [(5, 7, 11), (3, 1, 9), (1, 4, 1), (16, 16, 16), (17, 33, 65), (6, 5, 16), (12, 12, 32),
                                   (13, 9, 40), (7, 3, 17), (24, 10, 48), (50, 70, 90)])
def test_odd_shapes_single_thread(shape):
    _expect_same_result(np.float32, 1, *shape)


def test_odd_shapes_f64():
    _expect_same_result(np.float64, 1, 9, 5, 13)
    _expect_same_result(np.float64, 1, 33, 21, 29)


def test_pool_survives_many_cycles():
    for i in range(20):
        _expect_same_result(np.float32, 6, 110 + i % 7, 130, 120 + i % 5)


# ---- tests/bf16.zig:6-15 ------------------------------------------------------------------------
def test_bf16_round_to_nearest_even():
    L = orc.lib()
    assert L.oracle_bf16_decode(L.oracle_bf16_encode(1.0)) == 1.0
    assert L.oracle_bf16_decode(L.oracle_bf16_encode(-2.5)) == -2.5
    assert L.oracle_bf16_encode(1.0) == 0x3F80
    assert L.oracle_bf16_encode(1.00195312) == 0x3F80
    assert L.oracle_bf16_encode(1.01171875) == 0x3F82
    assert abs(L.oracle_bf16_decode(L.oracle_bf16_encode(1e-30)) / 1e-30 - 1) < 1e-2
    assert abs(L.oracle_bf16_decode(L.oracle_bf16_encode(3e38)) / 3e38 - 1) < 1e-2
    assert np.isinf(L.oracle_bf16_decode(L.oracle_bf16_encode(float("inf"))))


def test_bf16_matches_torch_rne():
    import torch

    rng = np.random.default_rng(0)
    x = rng.standard_normal(4096).astype(np.float32) * np.float32(10.0) ** rng.integers(-20, 20, 4096).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.bf16_encode(x), want)


# ---- tests/runtime.zig:62-84 --------------------------------------------------------------------
def test_grouped_and_dilated_known_answers():
    x = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 1, 0, 1, 0, 1, 0, 1, 0, 1], np.float32).reshape(1, 2, 3, 3)
    w = np.array([1, 0, 0, 1, 1, 1, 1, 1], np.float32).reshape(2, 1, 2, 2)
    grouped = orc.convolve_nchw(x, w, groups=2)
    assert grouped.shape == (1, 2, 2, 2)
    assert grouped.ravel().tolist() == [6, 8, 12, 14, 2, 2, 2, 2]
    dilated = orc.convolve_nchw(x[:, :1], np.ones((1, 1, 2, 2), np.float32), dilation=2, pad=1)
    assert dilated.shape == (1, 1, 3, 3)
    assert dilated.ravel().tolist() == [5, 10, 5, 10, 20, 10, 5, 10, 5]
    # The same dilated case through the NHWC path the exported graphs use (tests/runtime.zig:370-418).
    d = ConvDims(n=1, h=3, w=3, c=1, k=2, pad=1, dilation=2, c_out=1)
    nhwc = orc.convolve_nhwc(x[:, :1].transpose(0, 2, 3, 1), np.ones((1, 1, 2, 2), np.float32), None, d)
    assert nhwc.ravel().tolist() == [5, 10, 5, 10, 20, 10, 5, 10, 5]


def test_convolve_nhwc_equals_transposed_nchw():
    rng = np.random.default_rng(3)
    for (n, h, w, c, m, k, s, p, dil) in [(2, 9, 8, 3, 5, 3, 2, 1, 2), (1, 6, 6, 4, 8, 3, 1, 1, 1), (2, 5, 5, 2, 3, 1, 1, 0, 1)]:
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
        wt = rng.standard_normal((m, c, k, k)).astype(np.float32)
        bias = rng.standard_normal(m).astype(np.float32)
        want = orc.convolve_nchw(x, wt, bias, stride=s, pad=p, dilation=dil).transpose(0, 2, 3, 1)
        d = ConvDims(n=n, h=h, w=w, c=c, k=k, stride=s, pad=p, dilation=dil, c_out=m)
        got = orc.convolve_nhwc(x.transpose(0, 2, 3, 1), wt, bias, d)
        np.testing.assert_allclose(got, want, atol=1e-4)


# ---- tests/cpu_ops.zig:14-57 --------------------------------------------------------------------
CPU_OPS_DIMS = [ConvDims(2, 6, 7, 1, 3, 1, 0), ConvDims(2, 6, 7, 3, 3, 1, 1), ConvDims(1, 9, 8, 4, 5, 2, 2),
                ConvDims(3, 5, 5, 16, 1, 1, 0), ConvDims(2, 8, 8, 2, 3, 2, 1)]


@pytest.mark.parametrize("d", CPU_OPS_DIMS)
def test_rowwise_im2col_col2im_equal_per_element(d):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((d.n, d.h, d.w, d.c)).astype(np.float32)
    want = orc.im2col_elements(x, d)
    got = orc.im2col_rows(x, d, threads=3)
    assert np.array_equal(want, got)
    dcol = rng.standard_normal(want.shape).astype(np.float32)
    np.testing.assert_allclose(orc.col2im_pixels(dcol, d, threads=3), orc.col2im_elements(dcol, d), atol=1e-6)


# ---- tests/cpu_ops.zig:59-117 -------------------------------------------------------------------
@pytest.mark.parametrize("threads", [1, 3])
@pytest.mark.parametrize("d", [ConvDims(3, 12, 11, 1, 5, c_out=16), ConvDims(2, 13, 12, 1, 3, stride=2, c_out=32),
                               ConvDims(1, 6, 6, 1, 1, c_out=16), ConvDims(2, 8, 8, 1, 3, pad=1, c_out=16),
                               ConvDims(2, 8, 8, 3, 3, c_out=16), ConvDims(2, 9, 9, 1, 3, c_out=6)])
def test_conv_forward_and_weight_grad_vs_f64_im2col_product(d, threads):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((d.n, d.h, d.w, d.c)).astype(np.float32)
    w = rng.standard_normal((d.taps, d.c_out)).astype(np.float32)
    col = orc.im2col_elements(x, d).astype(np.float64)
    want = (col @ w.astype(np.float64)).astype(np.float32)
    got = orc.conv_forward(x, w, d, threads).reshape(d.rows, d.c_out)
    np.testing.assert_allclose(got, want, atol=1e-4)
    up = rng.standard_normal((d.rows, d.c_out)).astype(np.float32)
    start = rng.standard_normal((d.taps, d.c_out)).astype(np.float32)
    want_dw = (start.astype(np.float64) + col.T @ up.astype(np.float64)).astype(np.float32)
    got_dw = orc.conv_weight_grad(x, up, d, threads, dw=start.copy())
    np.testing.assert_allclose(got_dw, want_dw, atol=1e-3)


# ---- tests/autograd.zig:683-735 (direct 7-loop convolution) and :1843-1913 (chunked, threads) ---
@pytest.mark.parametrize("d", [ConvDims(2, 7, 6, 3, 3, 1, 1, c_out=4), ConvDims(2, 8, 8, 2, 3, 2, 1, c_out=5),
                               ConvDims(1, 9, 9, 4, 3, 3, 2, c_out=3), ConvDims(1, 10, 10, 2, 3, 1, 2, 2, c_out=4),
                               ConvDims(3, 5, 5, 8, 1, 1, 0, c_out=6)])
def test_conv_forward_matches_direct_convolution(d):
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, (d.n, d.h, d.w, d.c)).astype(np.float32)
    w = rng.uniform(-1, 1, (d.taps, d.c_out)).astype(np.float32)
    want = orc.conv_direct_f64(x, w, d)
    got = orc.conv_forward(x, w, d)
    np.testing.assert_allclose(got, want, atol=1e-6 * d.k * d.k * d.c * 4)


def test_chunked_conv_with_threads_is_bit_identical_and_matches_f64():
    d = ConvDims(30, 28, 28, 4, 3, 1, 1, c_out=8)   # more rows than one 2 MiB chunk holds
    rng = np.random.default_rng(11)
    x = rng.standard_normal((d.n, d.h, d.w, d.c)).astype(np.float32)
    w = rng.standard_normal((d.taps, d.c_out)).astype(np.float32)
    y1 = orc.conv_forward(x, w, d, 1)
    y4 = orc.conv_forward(x, w, d, 4)
    assert np.array_equal(y1, y4)
    np.testing.assert_allclose(y1, orc.conv_direct_f64(x, w, d), atol=1e-4)
    dy = rng.standard_normal(y1.shape).astype(np.float32)
    dx1 = orc.conv_input_grad(dy, w, d, 1)
    dx4 = orc.conv_input_grad(dy, w, d, 4)
    assert np.array_equal(dx1, dx4)
    # dX against the definition: the adjoint of the forward map (f64).
    col = orc.im2col_elements(np.zeros_like(x), d)   # shape only
    dcol = dy.reshape(d.rows, d.c_out).astype(np.float64) @ w.astype(np.float64).T
    want_dx = orc.col2im_elements(dcol.astype(np.float32), d)
    np.testing.assert_allclose(dx1, want_dx, atol=1e-3)
    assert col.shape == (d.rows, d.taps)


# ---- grouped per-element convolution (src/gpu/math/conv.zig:259-340) against the dense one -------
def test_grouped_convolution_equals_block_diagonal_dense():
    rng = np.random.default_rng(13)
    d = ConvDims(2, 6, 6, 4, 3, 1, 1, 1, groups=2, c_out=6)
    cg, og = d.c // d.groups, d.c_out // d.groups
    x = rng.standard_normal((d.n, d.h, d.w, d.c)).astype(np.float32)
    w = rng.standard_normal((d.k * d.k * cg, d.c_out)).astype(np.float32)
    dense_w = np.zeros((d.k * d.k, d.c, d.c_out), np.float32)
    for g in range(d.groups):
        dense_w[:, g * cg:(g + 1) * cg, g * og:(g + 1) * og] = w.reshape(d.k * d.k, cg, d.c_out)[:, :, g * og:(g + 1) * og]
    dd = ConvDims(d.n, d.h, d.w, d.c, d.k, d.stride, d.pad, d.dilation, 1, d.c_out)
    want = orc.conv_direct_f64(x, dense_w.reshape(-1, d.c_out), dd)
    np.testing.assert_allclose(orc.conv_forward(x, w, d), want, atol=1e-4)
    dy = rng.standard_normal(want.shape).astype(np.float32)
    np.testing.assert_allclose(orc.conv_input_grad(dy, w, d), orc.conv_input_grad(dy, dense_w.reshape(-1, d.c_out), dd), atol=1e-4)
    dw_dense = orc.conv_weight_grad(x, dy, dd).reshape(d.k * d.k, d.c, d.c_out)
    dw = orc.conv_weight_grad(x, dy, d).reshape(d.k * d.k, cg, d.c_out)
    for g in range(d.groups):
        np.testing.assert_allclose(dw[:, :, g * og:(g + 1) * og], dw_dense[:, g * cg:(g + 1) * cg, g * og:(g + 1) * og], atol=1e-4)


# ---- src/onnx/runtime.zig:621-664 ---------------------------------------------------------------
def test_onnx_gemm_and_matmul():
    rng = np.random.default_rng(17)
    x = rng.standard_normal((5, 7)).astype(np.float32)
    y = rng.standard_normal((7, 3)).astype(np.float32)
    c = rng.standard_normal(3).astype(np.float32)
    np.testing.assert_allclose(orc.onnx_gemm(x, y, c, alpha=0.5, beta=2.0), 0.5 * (x @ y) + 2 * c, atol=1e-5)
    np.testing.assert_allclose(orc.onnx_gemm(x.T.copy(), y.T.copy(), c, trans_a=True, trans_b=True), x @ y + c, atol=1e-5)
    xb = rng.standard_normal((4, 5, 7)).astype(np.float32)
    np.testing.assert_allclose(orc.onnx_matmul(xb, y), xb @ y, atol=1e-5)


# ---- src/nn/replicas.zig:57-91; tests/replicas.zig:76 -------------------------------------------
def test_average_grads_is_ordered_mean_and_identical_on_all_replicas():
    rng = np.random.default_rng(19)
    g = rng.standard_normal((3, 1000)).astype(np.float32)
    out = orc.average_grads(g)
    want = ((g[0] + g[1]) + g[2]) * np.float32(1.0 / 3.0)
    assert np.array_equal(out[0], want)
    assert np.array_equal(out[0], out[1]) and np.array_equal(out[0], out[2])


def test_tf32_rounding_is_rna_to_10_bits():
    L = orc.lib()
    assert L.oracle_tf32_round(1.0) == 1.0
    assert L.oracle_tf32_round(1.0 + 2.0 ** -11) == 1.0 + 2.0 ** -10   # tie rounds away from zero
    assert L.oracle_tf32_round(1.0 + 2.0 ** -12) == 1.0
    assert L.oracle_tf32_round(-(1.0 + 2.0 ** -11)) == -(1.0 + 2.0 ** -10)
