"""GPU parity of the implicit-GEMM convolution (forward, input gradient, weight gradient) against the CPU
oracle, through the C ABI.

Geometries follow the reference's conv tests (tests/autograd.zig:2002-2072: 2x5x5 inputs, k in {1,2,3},
stride {1,2,3}, pad {0,1,2}, dilation 2, channels 2..128) plus the ResNet-14 layer shapes of the benchmark
configuration at a reduced batch.  Tolerances: relative Frobenius error <= 1e-5 (strict f32), 5e-3 (TF32),
2e-2 (bf16) against the f32 oracle on the same seeded inputs.
"""
import numpy as np
import pytest

from tests.util import TOL_BF16, TOL_F32, TOL_TF32, rel_fro, seeded, to_dev, to_host

pytestmark = pytest.mark.gpu

# (n, h, w, c, k, c_out, stride, pad, dilation)
SMALL = [
    (2, 5, 5, 2, 3, 3, 1, 0, 1), (2, 5, 5, 4, 3, 8, 1, 1, 1), (2, 5, 5, 8, 3, 4, 2, 1, 1), (2, 5, 5, 2, 3, 3, 2, 0, 1),
    (2, 5, 5, 3, 3, 4, 1, 2, 2), (2, 5, 5, 2, 2, 4, 1, 0, 2), (2, 5, 5, 3, 1, 4, 1, 1, 1), (2, 5, 5, 64, 3, 32, 1, 1, 1),
    (2, 5, 5, 64, 3, 64, 1, 0, 1), (2, 5, 5, 128, 3, 64, 1, 1, 1), (2, 5, 5, 64, 1, 128, 1, 0, 1), (2, 7, 6, 5, 3, 7, 3, 1, 1),
    (1, 9, 8, 4, 5, 6, 2, 2, 1),
]
# ResNet-14 layer shapes (examples/cifar/main.zig:15-34) at batch 4, plus the strided transition variants.
RESNET = [
    (4, 32, 32, 3, 3, 64, 1, 1, 1),      # stem: K = 27
    (4, 32, 32, 64, 3, 64, 1, 1, 1),
    (4, 16, 16, 64, 3, 128, 1, 1, 1),
    (4, 16, 16, 128, 3, 128, 1, 1, 1),
    (4, 16, 16, 64, 1, 128, 1, 0, 1),    # 1x1 shortcut
    (4, 8, 8, 128, 3, 256, 1, 1, 1),
    (4, 8, 8, 256, 3, 256, 1, 1, 1),
    (4, 32, 32, 64, 3, 128, 2, 1, 1),    # strided transition
    (4, 32, 32, 64, 1, 128, 2, 0, 1),    # strided shortcut
    (3, 16, 16, 128, 3, 256, 2, 1, 1),
    (2, 16, 16, 64, 3, 64, 1, 2, 2),     # dilation 2: column-patch stages step two image rows per tap
    (2, 16, 16, 64, 5, 64, 1, 2, 1),     # 5x5: five taps per column-patch stage
    (2, 32, 32, 128, 3, 32, 1, 1, 1),    # two channel blocks per tap, narrow output
]


@pytest.fixture(scope="module")
def gpu():
    import grad_b200

    g = grad_b200.Gpu(0)
    yield g
    g.check_status()
    g.close()


def _dims(case):
    from oracle.binding import ConvDims

    n, h, w, c, k, c_out, s, p, d = case
    return ConvDims(n=n, h=h, w=w, c=c, k=k, stride=s, pad=p, dilation=d, c_out=c_out)


def _geo(case):
    from grad_b200 import conv_geometry

    n, h, w, c, k, c_out, s, p, d = case
    return conv_geometry(n, h, w, c, k, c_out, s, p, d)


def _inputs(case, seed):
    d = _dims(case)
    x = seeded(seed, d.n, d.h, d.w, d.c)
    w = (seeded(seed + 1, d.taps, d.c_out) * np.float32(np.sqrt(2.0 / d.taps))).astype(np.float32)   # He-normal
    dy = seeded(seed + 2, d.n, d.out_h, d.out_w, d.c_out)
    return d, x, w, dy


def _run_all(gpu, case, math, tol, bf16_storage=False, seed=100):
    import torch
    from oracle import binding as orc

    d, x, w, dy = _inputs(case, seed)
    geo = _geo(case)
    threads = orc.host_threads()
    want_y = orc.conv_forward(x, w, d, threads)
    want_dx = orc.conv_input_grad(dy, w, d, threads)
    want_dw = orc.conv_weight_grad(x, dy, d, threads)
    act = torch.bfloat16 if bf16_storage else torch.float32
    dx_, dw_ = to_dev(x, bf16_storage), to_dev(w)   # weights stay f32 masters (src/autograd/autograd.zig:955)
    ddy = to_dev(dy, bf16_storage)
    y = torch.full((d.n, d.out_h, d.out_w, d.c_out), 5.0, dtype=act, device="cuda")
    gpu.convForward(dx_, dw_, y, geo, math=math)
    gx = torch.zeros((d.n, d.h, d.w, d.c), dtype=act, device="cuda")
    gpu.convInputGrad(ddy, dw_, gx, geo, accumulate=True, math=math)
    gw = torch.zeros((d.taps, d.c_out), dtype=torch.float32, device="cuda")
    gpu.convWeightGrad(ddy, dx_, gw, geo, math=math)
    torch.cuda.synchronize()
    errs = (rel_fro(to_host(y), want_y), rel_fro(to_host(gx), want_dx), rel_fro(to_host(gw), want_dw))
    assert max(errs) <= tol, (case, math, bf16_storage, errs)
    return errs


@pytest.mark.parametrize("case", SMALL)
def test_small_geometries_strict_f32(gpu, case):
    _run_all(gpu, case, 0, TOL_F32)


@pytest.mark.parametrize("case", SMALL)
def test_small_geometries_tf32(gpu, case):
    _run_all(gpu, case, 1, TOL_TF32)


@pytest.mark.parametrize("case", SMALL)
def test_small_geometries_bf16_math_on_f32_storage(gpu, case):
    _run_all(gpu, case, 2, TOL_BF16)


@pytest.mark.parametrize("case", SMALL)
def test_small_geometries_bf16_storage(gpu, case):
    _run_all(gpu, case, 2, TOL_BF16, bf16_storage=True)


@pytest.mark.parametrize("case", RESNET)
@pytest.mark.parametrize("math,tol,half", [(0, TOL_F32, False), (1, TOL_TF32, False), (2, TOL_BF16, False), (2, TOL_BF16, True)])
def test_resnet_layer_shapes(gpu, case, math, tol, half):
    _run_all(gpu, case, math, tol, bf16_storage=half, seed=200)


# 3-channel 3x3 stride-1 layers over a bf16 map: the tensor kernel's gather warps build their window lines with a routine of
# their own.  Odd widths make neighbouring positions straddle rows and images, the position count is no multiple of a
# tile, padding 0 and 2 move the window's corner off the default.
STEM_LIKE = [(3, 31, 29, 3, 3, 64, 1, 1, 1), (2, 9, 7, 3, 3, 32, 1, 0, 1), (1, 6, 6, 3, 3, 64, 1, 2, 1), (5, 8, 33, 3, 3, 128, 1, 1, 1)]


@pytest.mark.parametrize("case", STEM_LIKE)
def test_three_channel_window_lines_against_the_oracle(gpu, case):
    _run_all(gpu, case, 2, TOL_BF16, bf16_storage=True, seed=300)
    plan = gpu.last_plan()   # of the weight gradient, the last of the three passes
    assert plan["tensor_path"] == 1 and plan["a_kind"] == 5, plan   # 5: the gathered operand of the tensor kernel


def test_bf16_conv_agrees_with_f32_conv_within_reference_bounds(gpu):
    """tests/autograd.zig:1309-1359: 2x8x8x64 -> 32, pad 1; y, dX, dW element-wise bounds."""
    import torch
    from oracle import binding as orc

    case = (2, 8, 8, 64, 3, 32, 1, 1, 1)
    d = _dims(case)
    geo = _geo(case)
    x, w, g = seeded(37, 2, 8, 8, 64), seeded(38, 576, 32) * np.float32(0.05), seeded(39, 2, 8, 8, 32)
    wide_y = orc.conv_forward(x, w, d)
    wide_dx = orc.conv_input_grad(g, w, d)
    wide_dw = orc.conv_weight_grad(x, g, d)
    hx, hg, dw_ = to_dev(x, True), to_dev(g, True), to_dev(w)
    y = torch.empty((2, 8, 8, 32), dtype=torch.bfloat16, device="cuda")
    gx = torch.zeros((2, 8, 8, 64), dtype=torch.bfloat16, device="cuda")
    gw = torch.zeros((576, 32), dtype=torch.float32, device="cuda")
    gpu.convForward(hx, dw_, y, geo)
    gpu.convInputGrad(hg, dw_, gx, geo)
    gpu.convWeightGrad(hg, hx, gw, geo)
    torch.cuda.synchronize()
    assert np.all(np.abs(wide_y - to_host(y)) <= 0.08 + 0.02 * np.abs(wide_y))
    assert np.all(np.abs(wide_dx - to_host(gx)) <= 0.25 + 0.03 * np.abs(wide_dx))
    assert np.all(np.abs(wide_dw - to_host(gw)) <= 0.6 + 0.03 * np.abs(wide_dw))


@pytest.mark.parametrize("case", [(3, 16, 16, 64, 3, 128, 1, 1, 1),     # TMA patch boxes, column-patch stages, TMA stores
                                  (3, 32, 32, 3, 3, 64, 1, 1, 1),       # the stem: direct FMA kernel
                                  (2, 9, 9, 3, 3, 32, 2, 1, 1),         # strided stem-like layer, odd image
                                  (2, 16, 16, 64, 3, 72, 1, 1, 1)])     # a ragged last 32-column chunk beside TMA-stored ones
@pytest.mark.parametrize("math,tol,half", [(0, TOL_F32, False), (1, TOL_TF32, False), (2, TOL_BF16, True)])
def test_fused_bias_residual_relu_epilogue(gpu, case, math, tol, half):
    """Conv + bias -> Add(residual) -> Relu in one launch == the executor's separate nodes (src/onnx/gpu.zig:608, 372-377)."""
    import torch
    from oracle import binding as orc

    d, x, w, _ = _inputs(case, 300)
    geo = _geo(case)
    bias = seeded(303, d.c_out) * np.float32(0.1)
    res = seeded(304, d.n, d.out_h, d.out_w, d.c_out)
    if half:
        res = orc.bf16_round(res)
    want = orc.conv_forward(x, w, d, orc.host_threads())
    want = orc.relu(orc.bias_act(want, bias, False) + res)
    act = torch.bfloat16 if half else torch.float32
    y = torch.empty((d.n, d.out_h, d.out_w, d.c_out), dtype=act, device="cuda")
    from grad_b200 import Epilogue

    gpu.convForward(to_dev(x, half), to_dev(w, half), y, geo, epilogue=Epilogue(to_dev(bias), to_dev(res, half), True), math=math)
    torch.cuda.synchronize()
    got = to_host(y)
    assert rel_fro(got, want) <= tol
    assert (got >= 0).all()


def test_accumulate_semantics(gpu):
    """Gradients are `+=` into caller-zeroed buffers (autograd.zig:49-50): two calls add up; forward stores."""
    import torch

    case = (2, 8, 8, 64, 3, 64, 1, 1, 1)
    d, x, w, dy = _inputs(case, 400)
    geo = _geo(case)
    for math in (0, 2):
        gw = torch.zeros((d.taps, d.c_out), device="cuda")
        gpu.convWeightGrad(to_dev(dy), to_dev(x), gw, geo, math=math)
        once = to_host(gw).copy()
        gpu.convWeightGrad(to_dev(dy), to_dev(x), gw, geo, math=math)
        torch.cuda.synchronize()
        assert rel_fro(to_host(gw), 2 * once) <= 1e-6
        gx = torch.zeros((d.n, d.h, d.w, d.c), device="cuda")
        gpu.convInputGrad(to_dev(dy), to_dev(w), gx, geo, accumulate=True, math=math)
        first = to_host(gx).copy()
        gpu.convInputGrad(to_dev(dy), to_dev(w), gx, geo, accumulate=False, math=math)
        torch.cuda.synchronize()
        assert rel_fro(to_host(gx), first) <= 1e-6


@pytest.mark.parametrize("case", [(128, 32, 32, 64, 3, 64, 1, 1, 1), (128, 16, 16, 128, 3, 128, 1, 1, 1), (128, 8, 8, 256, 3, 256, 1, 1, 1),
                                  (128, 32, 32, 64, 3, 128, 2, 1, 1), (128, 32, 32, 3, 3, 64, 1, 1, 1)])
def test_full_size_adjoint_identity(gpu, case):
    """At the benchmark's batch 128 the oracle is too slow, but the three passes are adjoints of one another:
    <conv(x, w), dy> == <x, dgrad(dy, w)> == <w, wgrad(x, dy)>.  Checked in bf16 with f32 sums on the device."""
    import torch

    n, h, w_, c, k, c_out, s, p, dil = case
    geo = _geo(case)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    x = torch.randn((n, h, w_, c), generator=gen, device="cuda").bfloat16()
    w = (torch.randn((k * k * c, c_out), generator=gen, device="cuda") * (2.0 / (k * k * c)) ** 0.5).bfloat16()
    dy = torch.randn((n, geo.out_h, geo.out_w, c_out), generator=gen, device="cuda").bfloat16()
    y = torch.empty_like(dy, dtype=torch.float32)
    gx = torch.zeros(x.shape, dtype=torch.float32, device="cuda")
    gw = torch.zeros(w.shape, dtype=torch.float32, device="cuda")
    gpu.convForward(x, w, y, geo)
    gpu.convInputGrad(dy, w, gx, geo)
    gpu.convWeightGrad(dy, x, gw, geo)
    torch.cuda.synchronize()
    a = (y.double() * dy.double()).sum().item()
    b = (gx.double() * x.double()).sum().item()
    c_ = (gw.double() * w.double()).sum().item()
    scale = (y.double().norm() * dy.double().norm()).item()
    assert abs(a - b) <= 1e-4 * scale and abs(a - c_) <= 1e-4 * scale, (a, b, c_, scale)


# Every convolution layer of the two benchmark networks at the benchmark's batch of 128: the ResNet-14 64-128-256
# stack (examples/cifar/main.zig:15-34: stem, residual 3x3 layers, the widening 3x3 layers applied after the pool,
# the 1x1 shortcuts) with the strided variants of the four transition convolutions, and the 64-192-384 widths of the
# ONNX inference graph (192 columns take a 256-wide pair tile that overhangs n; 192 channels are three channel
# blocks per tap).  The CPU oracle finishes a batch-128 layer in a fraction of a second, so all three passes are
# compared in full, not by the adjoint identity alone.
FULL_BATCH = [
    (128, 32, 32, 3, 3, 64, 1, 1, 1), (128, 32, 32, 64, 3, 64, 1, 1, 1),
    (128, 16, 16, 64, 3, 128, 1, 1, 1), (128, 16, 16, 128, 3, 128, 1, 1, 1), (128, 16, 16, 64, 1, 128, 1, 0, 1),
    (128, 8, 8, 128, 3, 256, 1, 1, 1), (128, 8, 8, 256, 3, 256, 1, 1, 1), (128, 8, 8, 128, 1, 256, 1, 0, 1),
    (128, 32, 32, 64, 3, 128, 2, 1, 1), (128, 32, 32, 64, 1, 128, 2, 0, 1),
    (128, 16, 16, 128, 3, 256, 2, 1, 1), (128, 16, 16, 128, 1, 256, 2, 0, 1),
    (128, 16, 16, 64, 3, 192, 1, 1, 1), (128, 16, 16, 192, 3, 192, 1, 1, 1), (128, 16, 16, 64, 1, 192, 1, 0, 1),
    (128, 8, 8, 192, 3, 384, 1, 1, 1), (128, 8, 8, 384, 3, 384, 1, 1, 1), (128, 8, 8, 192, 1, 384, 1, 0, 1),
    (128, 32, 32, 64, 3, 192, 2, 1, 1), (128, 32, 32, 64, 1, 192, 2, 0, 1),
    (128, 16, 16, 192, 3, 384, 2, 1, 1), (128, 16, 16, 192, 1, 384, 2, 0, 1),
]


@pytest.mark.parametrize("case", FULL_BATCH)
@pytest.mark.parametrize("math,tol,half", [(1, TOL_TF32, False), (2, TOL_BF16, True)])
def test_benchmark_layers_at_batch_128_against_the_oracle(gpu, case, math, tol, half):
    """All three passes of every benchmark layer at batch 128, bf16 storage and TF32, every element; the filters are
    passed in the activations' type (the bench's configuration), so every operand takes its TMA path."""
    import torch
    from oracle import binding as orc

    d, x, w, dy = _inputs(case, 900)
    geo = _geo(case)
    if half:
        x, w, dy = orc.bf16_round(x), orc.bf16_round(w), orc.bf16_round(dy)
    threads = orc.host_threads()
    want_y = orc.conv_forward(x, w, d, threads)
    want_dx = orc.conv_input_grad(dy, w, d, threads)
    want_dw = orc.conv_weight_grad(x, dy, d, threads)
    act = torch.bfloat16 if half else torch.float32
    tx, tw, tdy = to_dev(x, half), to_dev(w, half), to_dev(dy, half)
    y = torch.full((d.n, d.out_h, d.out_w, d.c_out), 5.0, dtype=act, device="cuda")
    gx = torch.full((d.n, d.h, d.w, d.c), 5.0, dtype=act, device="cuda")
    gw = torch.zeros((d.taps, d.c_out), dtype=torch.float32, device="cuda")
    gpu.convForward(tx, tw, y, geo, math=math)
    gpu.convInputGrad(tdy, tw, gx, geo, accumulate=False, math=math)
    gpu.convWeightGrad(tdy, tx, gw, geo, math=math)
    torch.cuda.synchronize()
    errs = (rel_fro(to_host(y), want_y), rel_fro(to_host(gx), want_dx), rel_fro(to_host(gw), want_dw))
    assert max(errs) <= tol, (case, math, errs)
    # per image, so that one mis-addressed image cannot hide in the norm of the other 127
    gy, wy = to_host(y).reshape(d.n, -1), want_y.reshape(d.n, -1)
    per_image = np.linalg.norm(gy - wy, axis=1) / np.maximum(np.linalg.norm(wy, axis=1), 1e-30)
    assert per_image.max() <= tol, (case, math, int(per_image.argmax()), float(per_image.max()))
    gxi, wxi = to_host(gx).reshape(d.n, -1), want_dx.reshape(d.n, -1)
    per_image = np.linalg.norm(gxi - wxi, axis=1) / np.maximum(np.linalg.norm(wxi, axis=1), 1e-30)
    assert per_image.max() <= tol, (case, math, int(per_image.argmax()), float(per_image.max()))


@pytest.mark.parametrize("case", [RESNET[1], RESNET[2], RESNET[0], RESNET[7], SMALL[7]])
@pytest.mark.parametrize("math,tol,half", [(0, TOL_F32, False), (1, TOL_TF32, False), (2, TOL_BF16, True)])
def test_forward_with_prepared_filter_rows(gpu, case, math, tol, half):
    """gb_conv_desc.w_layout = 1: the filters as (c_out, k*k*c), the copy the executor prepares once per weight."""
    import torch
    from oracle import binding as orc

    d, x, w, _ = _inputs(case, 500)
    geo = _geo(case)
    want = orc.conv_forward(x, w, d, orc.host_threads())
    y = torch.empty((d.n, d.out_h, d.out_w, d.c_out), dtype=torch.bfloat16 if half else torch.float32, device="cuda")
    gpu.convForward(to_dev(x, half), to_dev(np.ascontiguousarray(w.T), half), y, geo, math=math, w_rows=True)
    torch.cuda.synchronize()
    assert rel_fro(to_host(y), want) <= tol


STRIDED = [
    ((4, 32, 32, 64, 3, 128, 2, 1, 1), True),     # ResNet transition: four classes of 1, 2, 2 and 4 taps
    ((4, 32, 32, 64, 1, 128, 2, 0, 1), True),     # 1x1 shortcut: three of the four classes have no tap and are zero
    ((3, 16, 16, 128, 3, 256, 2, 1, 1), True),
    ((2, 16, 16, 64, 3, 64, 2, 1, 2), True),      # dilation 2 under stride 2: all taps fall into one class per axis
    ((2, 24, 24, 64, 3, 64, 3, 1, 1), True),      # stride 3: nine classes of one tap each
    ((2, 16, 16, 64, 5, 64, 2, 2, 1), True),      # 5x5: classes of 3 and 2 taps per axis
    ((2, 15, 15, 64, 3, 64, 2, 1, 1), False),     # odd image: a 7-wide class grid is no whole-row box -> gathered product
]


@pytest.mark.parametrize("case,by_classes", STRIDED)
@pytest.mark.parametrize("math,tol,half", [(1, TOL_TF32, False), (2, TOL_BF16, True)])
def test_strided_input_gradient_by_parity_classes(gpu, case, by_classes, math, tol, half):
    """The input gradient of a strided layer runs as one patch product per parity class of input pixels when
    dy and the filters are stored in the tile's type; it must equal the reference's single product
    (src/gpu/math/conv.zig:105-130) on overwrite (stale contents, empty classes zeroed) and on accumulate."""
    import torch
    from oracle import binding as orc

    d, x, w, dy = _inputs(case, 700)
    geo = _geo(case)
    w_used = to_host(to_dev(w, half)).astype(np.float32)     # the filters as the device sees them
    dy_used = to_host(to_dev(dy, half)).astype(np.float32)
    want = orc.conv_input_grad(dy_used, w_used, d, orc.host_threads())
    act = torch.bfloat16 if half else torch.float32
    gx = torch.full((d.n, d.h, d.w, d.c), 5.0, dtype=act, device="cuda")
    gpu.convInputGrad(to_dev(dy, half), to_dev(w, half), gx, geo, accumulate=False, math=math)
    plan = gpu.last_plan()
    torch.cuda.synchronize()
    assert rel_fro(to_host(gx), want) <= tol, (case, math, rel_fro(to_host(gx), want))
    assert (plan["a_kind"] == 2) == by_classes, plan     # 2 = TMA patch boxes, 5 = gathered
    gx32 = torch.full((d.n, d.h, d.w, d.c), 1.0, dtype=torch.float32, device="cuda")
    if not half:
        gpu.convInputGrad(to_dev(dy, half), to_dev(w, half), gx32, geo, accumulate=True, math=math)
        torch.cuda.synchronize()
        assert rel_fro(to_host(gx32) - 1.0, want) <= tol


def test_strict_f32_convolution_with_more_than_65535_row_tiles(gpu):
    """4096 images of 32 x 32 outputs are 65536 row tiles of 64 positions: the strict-f32 kernels index their tiles
    on grid.x (grid.y and grid.z stop at 65535).  First, middle and last image against the oracle."""
    import torch
    from oracle import binding as orc

    n, hw, c, co = 4096, 32, 8, 8
    geo = _geo((n, hw, hw, c, 3, co, 1, 1, 1))
    gen = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn((n, hw, hw, c), generator=gen, device="cuda")
    w = torch.randn((9 * c, co), generator=gen, device="cuda") * (2.0 / (9 * c)) ** 0.5
    y = torch.full((n, hw, hw, co), 3.0, device="cuda")
    gpu.convForward(x, w, y, geo, math=0)
    torch.cuda.synchronize()
    assert gpu.last_plan()["tensor_path"] == 0
    for img in (0, n // 2 - 1, n - 1):
        d = _dims((1, hw, hw, c, 3, co, 1, 1, 1))
        want = orc.conv_forward(to_host(x[img:img + 1]), to_host(w), d)
        assert rel_fro(to_host(y[img:img + 1]), want) <= TOL_F32, img


def test_prepared_weights_replace_the_per_call_filter_cast(gpu):
    """`gb_prepare_weights` / `gb_refresh_weights`: a bf16 copy of the f32 master filters made once per optimizer step
    instead of on every use (the reference's per-call `packMatrix`, src/autograd/autograd.zig:955, 1226, 1345).  The
    forward pass and the input gradient on the prepared copy launch no cast and give the bits of the per-call path;
    the rows layout feeds `w_layout = 1`; after the master changes, `refresh` brings the copy up to date."""
    import torch
    from oracle import binding as orc

    case = (4, 16, 16, 64, 3, 128, 1, 1, 1)
    d, x, w, dy = _inputs(case, 1100)
    geo = _geo(case)
    tx, tdy, master = to_dev(x, True), to_dev(dy, True), to_dev(w)
    y_ref = torch.empty((d.n, d.out_h, d.out_w, d.c_out), dtype=torch.bfloat16, device="cuda")
    gpu.convForward(tx, master, y_ref, geo)                       # f32 masters: cast launch + product
    assert gpu.last_plan()["kernel_launches"] == 2
    gx_ref = torch.zeros((d.n, d.h, d.w, d.c), dtype=torch.bfloat16, device="cuda")
    gpu.convInputGrad(tdy, master, gx_ref, geo, accumulate=False)
    plain, rows = gpu.prepareWeights(master), gpu.prepareWeights(master, rows_layout=True)
    assert plain.tensor.shape == (d.taps, d.c_out) and rows.tensor.shape == (d.c_out, d.taps)
    y, y_rows = torch.empty_like(y_ref), torch.empty_like(y_ref)
    gpu.convForward(tx, plain.tensor, y, geo)
    assert gpu.last_plan()["kernel_launches"] == 1
    gpu.convForward(tx, rows.tensor, y_rows, geo, w_rows=True)
    gx = torch.zeros_like(gx_ref)
    gpu.convInputGrad(tdy, plain.tensor, gx, geo, accumulate=False)
    assert gpu.last_plan()["kernel_launches"] == 1
    torch.cuda.synchronize()
    assert torch.equal(y, y_ref) and torch.equal(gx, gx_ref)
    want = orc.conv_forward(x, w, d, orc.host_threads())
    assert rel_fro(to_host(y_rows), want) <= TOL_BF16
    master.mul_(-2.0)                                              # the optimizer step
    plain.refresh(gpu._stream())
    gpu.convForward(tx, plain.tensor, y, geo)
    torch.cuda.synchronize()
    assert rel_fro(to_host(y), -2.0 * want) <= TOL_BF16
    plain.close(); rows.close()


def test_repeated_calls_are_served_from_the_plan_cache(gpu):
    """A call with the same descriptor, addresses, epilogue and workspace reuses its prepared plan (tile choice and
    tensor maps) and must give the same bits; a changed address plans anew."""
    import torch

    case = (4, 16, 16, 64, 3, 64, 1, 1, 1)
    d, x, w, dy = _inputs(case, 1200)
    geo = _geo(case)
    tx, tw = to_dev(x, True), to_dev(w, True)
    y1 = torch.empty((d.n, d.out_h, d.out_w, d.c_out), dtype=torch.bfloat16, device="cuda")
    gpu.convForward(tx, tw, y1, geo)
    hits = gpu.plan_cache_hits()
    first = y1.clone()
    for _ in range(3):
        gpu.convForward(tx, tw, y1, geo)
    assert gpu.plan_cache_hits() >= hits + 3
    y2 = torch.empty_like(y1)
    gpu.convForward(tx, tw, y2, geo)                               # another result buffer: a new plan, same values
    torch.cuda.synchronize()
    assert torch.equal(y1, first) and torch.equal(y2, first)


@pytest.mark.parametrize("n,side,c_in,c_out,seed", [(5, 16, 64, 96, 51), (12, 32, 64, 128, 52), (6, 8, 128, 256, 53), (3, 16, 64, 32, 54)])
def test_forward_epilogue_accumulates_batch_norm_sums(gpu, n, side, c_in, c_out, seed):
    """tests/gpu.zig:170-241 (`runEpilogueStats`): the forward pass with statistics in its epilogue stores the very bits
    of the plain forward pass, and its sums of (v - shift) and (v - shift)^2 per channel match a host reduction (f64) of
    the stored output within the reference's bounds; the ordered mode gives identical bits on repeated runs and stays
    close to the atomic sums."""
    import torch
    from grad_b200 import Epilogue

    geo = _geo((n, side, side, c_in, 3, c_out, 1, 1, 1))
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, side, side, c_in), dtype=np.float32) * 2 + 0.5).astype(np.float32)
    w = (rng.standard_normal((9 * c_in, c_out), dtype=np.float32) * 0.05).astype(np.float32)
    shift = (rng.standard_normal(c_out, dtype=np.float32) * 0.4).astype(np.float32)
    tx, tw, tshift = to_dev(x, True), to_dev(w, True), to_dev(shift)
    plain = torch.empty((n, side, side, c_out), dtype=torch.bfloat16, device="cuda")
    gpu.convForward(tx, tw, plain, geo)
    out = torch.empty_like(plain)
    sums = torch.zeros(2 * c_out, device="cuda")
    gpu.convForward(tx, tw, out, geo, epilogue=Epilogue(stats_shift=tshift, stats_sums=sums))
    torch.cuda.synchronize()
    assert gpu.last_plan()["tile_n"] >= c_out
    assert torch.equal(plain, out)                                   # tests/gpu.zig:205
    stored = out.double().cpu().numpy().reshape(-1, c_out) - shift.astype(np.float64)
    want_s, want_q = stored.sum(0), (stored * stored).sum(0)
    got = sums.cpu().numpy()
    assert np.all(np.abs(got[:c_out] - want_s) <= 0.05 + 1e-5 * np.abs(want_s)), float(np.abs(got[:c_out] - want_s).max())
    assert np.all(np.abs(got[c_out:] - want_q) <= 0.05 + 1e-4 * want_q), float(np.abs(got[c_out:] - want_q).max())
    det = []
    for _ in range(2):
        s2 = torch.zeros(2 * c_out, device="cuda")
        gpu.convForward(tx, tw, out, geo, epilogue=Epilogue(stats_shift=tshift, stats_sums=s2, stats_ordered=True))
        torch.cuda.synchronize()
        det.append(s2.cpu().numpy())
    assert np.array_equal(det[0], det[1])
    assert np.all(np.abs(det[0] - got) <= 0.05 + 1e-4 * np.abs(got))
    assert torch.equal(plain, out)


def test_statistics_accumulate_and_reject_what_the_epilogue_cannot_sum(gpu):
    """`sums` is added to (two calls double it); f32 results are summed unrounded; a product wider than one 256-column
    tile, or with a ragged last chunk, is refused with GB_ERR_UNSUPPORTED before anything is launched."""
    import torch
    from grad_b200 import Epilogue, GbError, MatmulOpts, MatmulShape

    m, n, k = 300, 64, 192
    a, b = seeded(61, m, k), seeded(62, k, n)
    out = torch.empty((m, n), device="cuda")
    sums = torch.zeros(2 * n, device="cuda")
    shift = to_dev(np.zeros(n, np.float32))
    for _ in range(2):
        gpu.matmul(to_dev(a, True), to_dev(b, True), out, MatmulShape(m, n, k), MatmulOpts(), epilogue=Epilogue(stats_shift=shift, stats_sums=sums))
    torch.cuda.synchronize()
    stored = out.double().cpu().numpy()
    got = sums.cpu().numpy()
    assert np.allclose(got[:n], 2 * stored.sum(0), rtol=1e-4, atol=0.05) and np.allclose(got[n:], 2 * (stored * stored).sum(0), rtol=1e-4, atol=0.05)
    for bad_n in (320, 72):
        wide = torch.empty((m, bad_n), device="cuda")
        with pytest.raises(GbError) as err:
            gpu.matmul(to_dev(a, True), to_dev(seeded(63, k, bad_n), True), wide, MatmulShape(m, bad_n, k), MatmulOpts(),
                       epilogue=Epilogue(stats_shift=to_dev(np.zeros(bad_n, np.float32)), stats_sums=torch.zeros(2 * bad_n, device="cuda")))
        assert err.value.status == 4


@pytest.mark.parametrize("n,side,c_in,c_out,seed", [(6, 16, 64, 128, 71), (5, 8, 128, 128, 72), (3, 32, 64, 64, 73)])
def test_input_gradient_epilogue_accumulates_batch_norm_backward_sums(gpu, n, side, c_in, c_out, seed):
    """`convImplicitForwardDxStats` (src/gpu/gpu.zig:964-972, device.zig:1537-1580): the input gradient with the masked
    batch-norm gradient sums in its epilogue stores the bits of the plain input gradient, and its sums of g and g * x_hat
    per channel match a host evaluation of the definition on the stored gradient; the ordered mode repeats bit for bit."""
    import torch

    geo = _geo((n, side, side, c_in, 3, c_out, 1, 1, 1))
    rng = np.random.default_rng(seed)
    dy = rng.standard_normal((n, side, side, c_out), dtype=np.float32)
    w = (rng.standard_normal((9 * c_in, c_out), dtype=np.float32) * 0.05).astype(np.float32)
    x_bn = (rng.standard_normal((n, side, side, c_in), dtype=np.float32) * 1.5 + 0.3).astype(np.float32)
    mean = (rng.standard_normal(c_in, dtype=np.float32) * 0.3).astype(np.float32)
    inv_std = (0.5 + rng.random(c_in, dtype=np.float32)).astype(np.float32)
    gamma = (0.5 + rng.random(c_in, dtype=np.float32)).astype(np.float32)
    beta = (rng.standard_normal(c_in, dtype=np.float32) * 0.2).astype(np.float32)
    tdy, tw, tx = to_dev(dy, True), to_dev(w, True), to_dev(x_bn, True)
    plain = torch.empty((n, side, side, c_in), dtype=torch.bfloat16, device="cuda")
    gpu.convInputGrad(tdy, tw, plain, geo, accumulate=False)
    dx = torch.empty_like(plain)
    sums = torch.zeros(2 * c_in, device="cuda")
    args = (tx, to_dev(mean), to_dev(inv_std), to_dev(gamma), to_dev(beta))
    gpu.convInputGradDxStats(tdy, tw, dx, geo, *args, sums)
    torch.cuda.synchronize()
    assert torch.equal(plain, dx)
    stored = dx.float().cpu().numpy().reshape(-1, c_in)
    xs = tx.float().cpu().numpy().reshape(-1, c_in)
    xh = ((xs - mean) * inv_std).astype(np.float32)                    # one rounding per operation, as on the device
    mask = ((gamma * xh).astype(np.float32) + beta).astype(np.float32) > 0
    g = np.where(mask, stored, np.float32(0)).astype(np.float64)
    want_s, want_q = g.sum(0), (np.where(mask, (stored * xh).astype(np.float32), np.float32(0)).astype(np.float64)).sum(0)
    got = sums.cpu().numpy()
    assert np.all(np.abs(got[:c_in] - want_s) <= 0.05 + 1e-4 * np.abs(want_s)), float(np.abs(got[:c_in] - want_s).max())
    assert np.all(np.abs(got[c_in:] - want_q) <= 0.05 + 1e-4 * np.abs(want_q)), float(np.abs(got[c_in:] - want_q).max())
    det = []
    for _ in range(2):
        s2 = torch.zeros(2 * c_in, device="cuda")
        gpu.convInputGradDxStats(tdy, tw, dx, geo, *args, s2, ordered=True)
        torch.cuda.synchronize()
        det.append(s2.cpu().numpy())
    assert np.array_equal(det[0], det[1])
    assert np.all(np.abs(det[0] - got) <= 0.05 + 1e-4 * np.abs(got))


def _virtual_map(x_bf16, mean, inv_std, gamma, beta):
    """relu(s * x + t) with s = bf16(gamma * inv_std), t = bf16(beta - mean * (gamma * inv_std)) and ONE rounding of the
    product-and-sum to bf16 (`affineExpand` / `affinePair`, src/gpu/device.zig:1774-1783, 1604-1612), evaluated in f64."""
    from oracle import binding as orc

    s32 = (gamma * inv_std).astype(np.float32)
    s = orc.bf16_round(s32)
    t = orc.bf16_round((beta - (mean * s32).astype(np.float32)).astype(np.float32))
    exact = x_bf16.astype(np.float64) * s.astype(np.float64) + t.astype(np.float64)
    return np.maximum(orc.bf16_round(exact.astype(np.float32)), np.float32(0))


@pytest.mark.parametrize("case", [(3, 16, 16, 64, 3, 64, 1, 1, 1), (2, 8, 8, 128, 3, 96, 1, 1, 1), (2, 9, 9, 64, 3, 32, 2, 1, 1)])
def test_forward_and_weight_gradient_over_a_virtual_normalised_input(gpu, case):
    """`convImplicitForwardAffineStats` and the `Affine` weight gradient (src/gpu/gpu.zig:951-959, 983-1022): a layer whose
    input is relu(batch_norm(x)) that was never written out must give what the same layer gives on the written-out map
    -- padding taps included, where relu(s * 0 + t) would be wrong -- and the statistics of its result ride along."""
    import torch
    from grad_b200 import Epilogue
    from oracle import binding as orc

    d, x, w, dy = _inputs(case, 1300)
    geo = _geo(case)
    rng = np.random.default_rng(1301)
    mean = (rng.standard_normal(d.c, dtype=np.float32) * 0.3).astype(np.float32)
    inv_std = (0.5 + rng.random(d.c, dtype=np.float32)).astype(np.float32)
    gamma = (0.5 + rng.random(d.c, dtype=np.float32)).astype(np.float32)
    beta = (0.3 + rng.standard_normal(d.c, dtype=np.float32) * 0.2).astype(np.float32)      # mostly positive: padding would show
    xb, wb, dyb = orc.bf16_round(x), orc.bf16_round(w), orc.bf16_round(dy)
    z = _virtual_map(xb, mean, inv_std, gamma, beta)
    want_y = orc.conv_forward(z, wb, d, orc.host_threads())
    want_dw = orc.conv_weight_grad(z, dyb, d, orc.host_threads())
    norm = tuple(to_dev(v) for v in (mean, inv_std, gamma, beta))
    tx, tw, tdy = to_dev(xb, True), to_dev(wb, True), to_dev(dyb, True)
    y = torch.empty((d.n, d.out_h, d.out_w, d.c_out), dtype=torch.bfloat16, device="cuda")
    sums = torch.zeros(2 * d.c_out, device="cuda")
    shift = to_dev(np.zeros(d.c_out, np.float32))
    gpu.convForwardAffine(tx, tw, y, geo, *norm, epilogue=Epilogue(stats_shift=shift, stats_sums=sums))
    # 64-channel blocks of a stride-1 layer arrive by TMA (NaN outside the image) and are rewritten in place before the MMAs read
    # them; anything TMA cannot fetch is transformed by the gather warps while they build the tile
    assert gpu.last_plan()["a_kind"] == (2 if case[6] == 1 else 5), gpu.last_plan()
    y_written = torch.empty_like(y)
    gpu.convForward(to_dev(z, True), tw, y_written, geo)           # the same layer on the written-out map
    gw = torch.zeros((d.taps, d.c_out), device="cuda")
    gpu.convWeightGradAffine(tdy, tx, gw, geo, *norm)
    torch.cuda.synchronize()
    assert rel_fro(to_host(y), want_y) <= 5e-3, rel_fro(to_host(y), want_y)
    assert rel_fro(to_host(y), to_host(y_written)) <= 5e-3
    assert rel_fro(to_host(gw), want_dw) <= 1e-3, rel_fro(to_host(gw), want_dw)
    stored = y.double().cpu().numpy().reshape(-1, d.c_out)
    got = sums.cpu().numpy()
    assert np.all(np.abs(got[:d.c_out] - stored.sum(0)) <= 0.05 + 1e-5 * np.abs(stored.sum(0)))
    assert np.all(np.abs(got[d.c_out:] - (stored * stored).sum(0)) <= 0.05 + 1e-4 * (stored * stored).sum(0))


def test_grouped_convolution_known_answer(gpu):
    """tests/runtime.zig:62-84: 2 groups of one channel, 2x2 filters on a 3x3 image -> [6, 8, 12, 14, 2, 2, 2, 2] (NCHW)."""
    import torch
    from grad_b200 import conv_geometry

    x = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 1, 0, 1, 0, 1, 0, 1, 0, 1], np.float32).reshape(1, 2, 3, 3).transpose(0, 2, 3, 1)
    w_oihw = np.array([1, 0, 0, 1, 1, 1, 1, 1], np.float32).reshape(2, 1, 2, 2)
    w = np.ascontiguousarray(w_oihw.transpose(2, 3, 1, 0).reshape(4, 2))        # (k*k*c/groups, c_out), row (ky*k+kx)*cg+ic
    geo = conv_geometry(1, 3, 3, 2, 2, 2, groups=2)
    y = torch.empty((1, 2, 2, 2), device="cuda")
    gpu.convForward(to_dev(x), to_dev(w), y, geo, math=0)
    torch.cuda.synchronize()
    assert to_host(y).transpose(0, 3, 1, 2).ravel().tolist() == [6, 8, 12, 14, 2, 2, 2, 2]


@pytest.mark.parametrize("case,groups", [((2, 8, 8, 128, 3, 128, 1, 1, 1), 2), ((2, 8, 8, 64, 3, 96, 1, 1, 1), 4), ((2, 9, 9, 64, 3, 64, 2, 1, 1), 2),
                                         ((3, 6, 6, 12, 3, 8, 1, 1, 1), 4), ((2, 8, 8, 64, 1, 64, 1, 0, 1), 64)])
@pytest.mark.parametrize("math,tol,half", [(0, TOL_F32, False), (1, TOL_TF32, False), (2, TOL_BF16, True)])
def test_grouped_convolution_all_passes(gpu, case, groups, math, tol, half):
    """`groups > 1` through the ABI (src/autograd/autograd.zig:150-155, per element: src/gpu/math/conv.zig:259-340): one product
    per group over channel slices of x, w and y, against the oracle's grouped convolution; the last case is depthwise."""
    import torch
    from grad_b200 import conv_geometry
    from oracle.binding import ConvDims
    from oracle import binding as orc

    n, h, w_, c, k, c_out, s, p, dil = case
    d = ConvDims(n=n, h=h, w=w_, c=c, k=k, stride=s, pad=p, dilation=dil, groups=groups, c_out=c_out)
    geo = conv_geometry(n, h, w_, c, k, c_out, s, p, dil, groups=groups)
    cg = c // groups
    x = seeded(1400, n, h, w_, c)
    w = (seeded(1401, k * k * cg, c_out) * np.float32(np.sqrt(2.0 / (k * k * cg)))).astype(np.float32)
    dy = seeded(1402, n, d.out_h, d.out_w, c_out)
    want_y, want_dx, want_dw = orc.conv_forward(x, w, d), orc.conv_input_grad(dy, w, d), orc.conv_weight_grad(x, dy, d)
    act = torch.bfloat16 if half else torch.float32
    y = torch.full((n, d.out_h, d.out_w, c_out), 5.0, dtype=act, device="cuda")
    gx = torch.zeros((n, h, w_, c), dtype=act, device="cuda")
    gw = torch.zeros((k * k * cg, c_out), device="cuda")
    gpu.convForward(to_dev(x, half), to_dev(w), y, geo, math=math)
    assert gpu.last_plan()["kernel_launches"] >= groups
    gpu.convInputGrad(to_dev(dy, half), to_dev(w), gx, geo, accumulate=True, math=math)
    gpu.convWeightGrad(to_dev(dy, half), to_dev(x, half), gw, geo, math=math)
    torch.cuda.synchronize()
    errs = (rel_fro(to_host(y), want_y), rel_fro(to_host(gx), want_dx), rel_fro(to_host(gw), want_dw))
    assert max(errs) <= tol, (case, groups, math, errs)
