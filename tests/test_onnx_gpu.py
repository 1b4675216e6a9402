"""`Executor.run` against the CPU walk of the same in-memory graph, as tests/onnx_gpu.zig:15-278 compares
`Executor.run` with `Model.run`: logits within tolerance, argmax identical, every node on the device."""
import numpy as np
import pytest

from tests.util import TOL_BF16, TOL_F32, TOL_TF32, rel_fro, seeded

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import grad_b200

    g = grad_b200.Gpu(0)
    yield g
    g.check_status()
    g.close()


@pytest.fixture(scope="module")
def small_case():
    from grad_b200.onnx_gpu import resnet14_model
    from oracle import onnx_cpu

    model = resnet14_model(64, 128, 256, seed=1238)   # the narrower net keeps the CPU walk to a few seconds
    x = seeded(1238, 24, 3072)
    want = onnx_cpu.run(model, {"input": x})["logits"]
    return model, x, want


@pytest.mark.parametrize("mode,tol", [("f32", 1e-4), ("tf32", TOL_TF32), ("bf16", TOL_BF16)])
@pytest.mark.parametrize("fuse", [True, False])
def test_resnet14_logits_match_cpu_walk(gpu, small_case, mode, tol, fuse):
    from grad_b200.onnx_gpu import Executor

    model, x, want = small_case
    ex = Executor(model, gpu, mode=mode, fuse=fuse)
    got = ex.run({"input": x})["logits"]
    assert got.shape == want.shape == (24, 10)
    assert rel_fro(got, want) <= tol, rel_fro(got, want)
    # argmax-identical wherever the CPU's own top-2 margin exceeds the error bound of the mode
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4 * tol * np.abs(want).max()
    assert np.array_equal(got.argmax(1)[clear], want.argmax(1)[clear])
    assert ex.stats.host_nodes == 0 and ex.stats.uploads >= 1 and ex.stats.downloads == 1
    if fuse:
        # 15 convs and 1 product (one launch each, two when K is split), 5 pools, 15 first-run weight reorders
        assert ex.stats.launches <= 2 * (15 + 1) + 5 + 15


def test_fusion_changes_launch_count_not_results(gpu, small_case):
    from grad_b200.onnx_gpu import Executor

    model, x, _ = small_case
    fused, plain = Executor(model, gpu, "tf32", fuse=True), Executor(model, gpu, "tf32", fuse=False)
    a, b = fused.run({"input": x})["logits"], plain.run({"input": x})["logits"]
    assert rel_fro(a, b) <= TOL_TF32   # the unfused walk rounds to TF32 before Add / Relu, the fused one after
    fused.run({"input": x}); plain.run({"input": x})      # second run: weight caches are warm
    assert 21 <= fused.stats.launches <= 37 and plain.stats.launches >= fused.stats.launches + 15


def test_graph_replay_equals_eager_run(gpu, small_case):
    import torch
    from grad_b200.onnx_gpu import Executor

    model, x, _ = small_case
    ex = Executor(model, gpu, "bf16")
    xd = torch.from_numpy(x).cuda()
    eager = ex.run_device({"input": xd})["logits"].clone()
    ex.capture({"input": xd})
    again = ex.replay({"input": xd})["logits"]
    torch.cuda.synchronize()
    assert torch.equal(eager, again)
    other = torch.from_numpy(seeded(99, 24, 3072)).cuda()
    want = ex.run_device({"input": other})["logits"].clone()
    got = ex.replay({"input": other})["logits"]
    torch.cuda.synchronize()
    assert torch.equal(want, got)


@pytest.mark.parametrize("mode,tol", [("tf32", TOL_TF32), ("bf16", TOL_BF16)])
def test_full_width_model_matches_cpu_walk(gpu, mode, tol):
    """The benchmark's own graph (ResNet-14 64-192-384, batch norm folded) against the CPU walk (`Model.run`,
    src/onnx/runtime.zig:560-620) on the same seeded images: logits within the mode's tolerance, argmax identical
    wherever the CPU's own top-2 margin exceeds the error bound."""
    from grad_b200.onnx_gpu import Executor, resnet14_model
    from oracle import onnx_cpu

    model = resnet14_model(64, 192, 384)
    x = seeded(1241, 16, 3072)
    want = onnx_cpu.run(model, {"input": x})["logits"]
    got = Executor(model, gpu, mode=mode).run({"input": x})["logits"]
    assert got.shape == want.shape == (16, 10)
    assert rel_fro(got, want) <= tol, rel_fro(got, want)
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4 * tol * np.abs(want).max()
    assert clear.sum() >= 8 and np.array_equal(got.argmax(1)[clear], want.argmax(1)[clear])


def test_full_width_model_runs_at_batch_100(gpu):
    """The benchmark's graph (64-192-384) at batch 100: shape, finiteness, and bf16 vs tf32 agreement."""
    from grad_b200.onnx_gpu import Executor, resnet14_model

    model = resnet14_model(64, 192, 384)
    x = seeded(5, 100, 3072)
    a = Executor(model, gpu, "tf32").run({"input": x})["logits"]
    b = Executor(model, gpu, "bf16").run({"input": x})["logits"]
    assert a.shape == (100, 10) and np.isfinite(a).all()
    assert rel_fro(b, a) <= TOL_BF16


@pytest.mark.parametrize("mode,tol", [("f32", 1e-5), ("tf32", TOL_TF32), ("bf16", TOL_BF16)])
def test_gemm_nodes_match_cpu_walk(gpu, mode, tol):
    """ONNX `Gemm` (src/onnx/gpu.zig:500-521, CPU: src/onnx/runtime.zig:648-664): transB with a bias vector and a
    following Relu (one launch), transA with a C of the result's shape, and a plain product; against the CPU walk."""
    from grad_b200.onnx_gpu import Executor, Model, Node
    from oracle import onnx_cpu

    rng = np.random.default_rng(77)
    init = {"w1": rng.standard_normal((160, 96)).astype(np.float32) * 0.1, "b1": rng.standard_normal(160).astype(np.float32),
            "w2": rng.standard_normal((160, 64)).astype(np.float32) * 0.1, "c2": rng.standard_normal((48, 64)).astype(np.float32),
            "w3": rng.standard_normal((48, 40)).astype(np.float32) * 0.1}
    nodes = [Node("Gemm", ["input", "w1", "b1"], ["h1"], {"transB": 1}), Node("Relu", ["h1"], ["a1"]),
             Node("Gemm", ["a1", "w2", "c2"], ["h2"], {}),                       # (48,160) x (160,64) + C (48,64)
             Node("Gemm", ["h2", "w3"], ["out"], {"transA": 1})]                 # h2 stored (k=48, m=64): (64,48) x (48,40)
    model = Model(nodes, init, ["input"], ["out"])
    x = seeded(78, 48, 96)
    want = onnx_cpu.run(model, {"input": x})["out"]
    ex = Executor(model, gpu, mode=mode)
    got = ex.run({"input": x})["out"]
    assert got.shape == want.shape == (64, 40)
    assert rel_fro(got, want) <= tol, rel_fro(got, want)
    assert ex.stats.host_nodes == 0 and ex.stats.device_nodes == 4
    with pytest.raises(NotImplementedError):
        Executor(Model([Node("Gemm", ["input", "w1"], ["out"], {"transB": 1, "alpha": 0.5})], init, ["input"], ["out"]), gpu, mode).run({"input": x})


def test_activations_are_released_after_their_last_use(gpu, small_case):
    """The walk drops a value once its last consumer has run: far fewer values are alive at once than the graph
    produces, and the logits do not change."""
    from grad_b200.onnx_gpu import Executor

    model, x, want = small_case
    ex = Executor(model, gpu, "tf32")
    got = ex.run({"input": x})["logits"]
    assert rel_fro(got, want) <= TOL_TF32
    produced = sum(len(n.outputs) for n in model.nodes)
    assert 0 < ex.peak_live <= 4 and produced > 40, (ex.peak_live, produced)


@pytest.mark.parametrize("is_max", [0, 1])
@pytest.mark.parametrize("shape", [(3, 8, 8, 64, 2, 2, 0), (2, 9, 7, 24, 3, 2, 1), (2, 8, 8, 12, 2, 2, 0), (1, 4, 4, 256, 4, 4, 0)])
def test_pool2d_vector_and_scalar_kernels_agree_with_the_window_definition(gpu, is_max, shape):
    """`gb_pool2d` on NHWC: clipped windows, the average over in-bounds taps only (src/gpu/math/conv.zig:152-186).
    bf16 tensors with a multiple of 8 channels take the 16-byte kernel, everything else the scalar one; both
    must reproduce a plain numpy evaluation of the definition on the same bf16 values, bit for bit."""
    import ctypes as C
    import torch

    n, h, w, c, k, stride, pad = shape
    x = torch.from_numpy(seeded(77, n, h, w, c)).cuda().bfloat16()
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    xf = x.float().cpu().numpy()
    want = np.empty((n, oh, ow, c), dtype=np.float32)
    for oy in range(oh):
        for ox in range(ow):
            y0, y1 = max(oy * stride - pad, 0), min(oy * stride + k - pad, h)
            x0, x1 = max(ox * stride - pad, 0), min(ox * stride + k - pad, w)
            win = xf[:, y0:y1, x0:x1, :].reshape(n, -1, c)
            if is_max:
                want[:, oy, ox, :] = win.max(axis=1)
            else:
                acc = np.zeros((n, c), dtype=np.float32)
                for t in range(win.shape[1]):      # the kernels add the taps in row-major window order
                    acc += win[:, t, :]
                want[:, oy, ox, :] = acc / np.float32(win.shape[1])
    want_bf16 = torch.from_numpy(want).bfloat16().float().numpy()
    for dtype, code in ((torch.bfloat16, 1), (torch.float32, 0)):
        xin = x.to(dtype).contiguous()
        y = torch.empty((n, oh, ow, c), dtype=dtype, device="cuda")
        rc = gpu.lib.gb_pool2d(C.c_void_p(torch.cuda.current_stream().cuda_stream), is_max, code, C.c_void_p(xin.data_ptr()),
                               C.c_void_p(y.data_ptr()), n, h, w, c, k, stride, pad)
        assert rc == 0
        torch.cuda.synchronize()
        got = y.float().cpu().numpy()
        assert np.array_equal(got, want_bf16 if dtype == torch.bfloat16 else want), (shape, is_max, dtype)
