"""Oracle parity of the matmul family at the benchmark's own sizes (the GEMM sweep: M = N = K in {4096, 8192} and
the skinny 128 x 4096 x 4096, layouts NN / NT / TN, bf16 and TF32, fused bias + ReLU), through the C ABI.

The CPU oracle cannot finish an 8192^3 product in test time, but a row of the result needs only its row of A:
the GPU computes the whole product and the oracle (`matmulTiled`, src/cpu/kernels.zig:234-448) recomputes a
sample of rows against the full B.  The sample takes rows from every 256-row tile band, from both CTAs of a
pair tile and from all four 32-lane quarters of each, and whole rows, so every 512-column tile, both column
halves of it and every 32-column chunk are covered.  Each case asserts the tile the planner chose, so the test
cannot silently stop covering the 256 x 512 CTA-pair path that the headline number runs on.
"""
import numpy as np
import pytest

from tests.util import TOL_BF16, TOL_F32, TOL_TF32, rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu

LAYOUTS = {"NN": (False, False), "NT": (False, True), "TN": (True, False)}


@pytest.fixture(scope="module")
def gpu():
    import grad_b200

    g = grad_b200.Gpu(0)
    yield g
    g.check_status()
    g.close()


_cache = {}


def _operands(size):
    """Two seeded N(0,1) square matrices and a bias, f32 and bf16-rounded, generated once per size."""
    from oracle import binding as orc

    if size not in _cache:
        _cache.clear()   # one size at a time: 8192^2 f32 is 268 MB per matrix
        rng = np.random.default_rng(1234 + 1)
        a = rng.standard_normal((size, size), dtype=np.float32)
        b = rng.standard_normal((size, size), dtype=np.float32)
        bias = rng.standard_normal(size, dtype=np.float32)
        _cache[size] = (a, b, bias, orc.bf16_round(a), orc.bf16_round(b))
    return _cache[size]


def sample_rows(m, per_band=4, band=256):
    """Rows spread over every `band`-row tile band: both 128-row halves, all four 32-lane quarters, varying lanes."""
    rows = []
    for t in range((m + band - 1) // band):
        for j in range(per_band):
            slot = (t * per_band + j) % 8                     # which (half, quarter) of the band
            lane = (t * 7 + j * 13) % 32
            r = t * band + slot * 32 + lane
            if r < m:
                rows.append(r)
    if m - 1 not in rows:
        rows.append(m - 1)
    return np.array(sorted(set(rows)), dtype=np.int64)


def oracle_rows(a, b, bias, rows, m, n, k, ta, tb, relu=True):
    """Rows `rows` of relu(op(a) * op(b) + bias) by the CPU oracle; a and b are the STORED operands."""
    from oracle import binding as orc

    sub = np.ascontiguousarray(a[:, rows] if ta else a[rows, :])
    out = orc.matmul_tiled(sub, b, len(rows), k, n, ta, tb, threads=orc.host_threads())
    return orc.bias_act(out, bias, relu) if bias is not None else out


def _run(gpu, m, n, k, layout, math, a, b, bias, out_bf16):
    import torch
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape

    ta, tb = LAYOUTS[layout]
    half = math == 2
    out = torch.full((m, n), -3.0, dtype=torch.bfloat16 if out_bf16 else torch.float32, device="cuda")
    gpu.matmul(to_dev(a, half), to_dev(b, half), out, MatmulShape(m, n, k), MatmulOpts(ta, tb),
               epilogue=Epilogue(bias=to_dev(bias), relu=True), math=math)
    torch.cuda.synchronize()
    return out, gpu.last_plan()


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("math,tol", [(2, TOL_BF16), (1, TOL_TF32)])
@pytest.mark.parametrize("size", [4096, 8192])
def test_square_sweep_sizes_on_sampled_rows(gpu, size, math, tol, layout):
    a32, b32, bias, a16, b16 = _operands(size)
    a, b = (a16, b16) if math == 2 else (a32, b32)
    ta, tb = LAYOUTS[layout]
    out, plan = _run(gpu, size, size, size, layout, math, a, b, bias, out_bf16=math == 2)
    assert plan["tensor_path"] == 1 and plan["tile_m"] == 256 and plan["tile_n"] == 512, plan
    rows = sample_rows(size, per_band=8 if size == 4096 else 4)
    want = oracle_rows(a, b, bias, rows, size, size, size, ta, tb)
    got = to_host(out[torch_index(rows)])
    err = rel_fro(got, want)
    assert err <= tol, (size, layout, math, err)
    # every sampled row on its own, so a single bad row (one lane, one band) cannot hide in the norm of the rest
    per_row = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-30)
    assert per_row.max() <= tol, (size, layout, math, int(rows[per_row.argmax()]), float(per_row.max()))
    assert (got >= 0).all()


def torch_index(rows):
    import torch

    return torch.from_numpy(rows).cuda()


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("math,tol", [(2, TOL_BF16), (1, TOL_TF32), (0, TOL_F32)])
def test_skinny_sweep_shape_in_full(gpu, math, tol, layout):
    """128 x 4096 x 4096 (one row tile, weight streaming): every element against the oracle."""
    a32, b32, bias, a16, b16 = _operands(4096)
    m, n, k = 128, 4096, 4096
    ta, tb = LAYOUTS[layout]
    a_full, b = (a16, b16) if math == 2 else (a32, b32)
    a = np.ascontiguousarray(a_full[:, :m] if ta else a_full[:m, :])
    out, plan = _run(gpu, m, n, k, layout, math, a, b, bias, out_bf16=math == 2)
    want = oracle_rows(a, b, bias, np.arange(m), m, n, k, ta, tb)
    err = rel_fro(to_host(out), want)
    assert err <= tol, (layout, math, err, plan)


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("math,tol", [(2, TOL_BF16), (1, TOL_TF32)])
def test_ragged_shape_on_the_512_wide_pair_tile_in_full(gpu, math, tol, layout):
    """2088 x 2584 x 2048: nine 256-row bands with a 40-row tail and six 512-column tiles with a 24-column tail --
    clipped TMA stores, a ragged last chunk and rows past m in the last band -- every element against the oracle."""
    from oracle import binding as orc

    m, n, k = 2088, 2584, 2048
    ta, tb = LAYOUTS[layout]
    rng = np.random.default_rng(4321)
    a = rng.standard_normal((k, m) if ta else (m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    if math == 2:
        a, b = orc.bf16_round(a), orc.bf16_round(b)
    out, plan = _run(gpu, m, n, k, layout, math, a, b, bias, out_bf16=math == 2)
    assert plan["tile_m"] == 256 and plan["tile_n"] == 512, plan
    want = orc.bias_act(orc.matmul_tiled(a, b, m, k, n, ta, tb, threads=orc.host_threads()), bias, True)
    got = to_host(out)
    assert rel_fro(got, want) <= tol, (layout, math, rel_fro(got, want))
    per_row = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-30)
    assert per_row.max() <= tol, (layout, math, int(per_row.argmax()), float(per_row.max()))


def test_accumulate_into_bf16_on_the_512_wide_tile(gpu):
    """C += A*B with a bf16 C at 4096^3 (the `accumulate` read-modify-write of the staged-store epilogue)."""
    import torch
    from grad_b200 import MatmulOpts, MatmulShape
    from oracle import binding as orc

    size = 4096
    _, _, _, a16, b16 = _operands(size)
    start = orc.bf16_round(np.random.default_rng(9).standard_normal((size, size), dtype=np.float32))
    out = to_dev(start, True)
    gpu.matmul(to_dev(a16, True), to_dev(b16, True), out, MatmulShape(size, size, size), MatmulOpts(False, False, True))
    torch.cuda.synchronize()
    assert gpu.last_plan()["tile_n"] == 512
    rows = sample_rows(size, per_band=4)
    sub = np.ascontiguousarray(a16[rows, :])
    want = orc.matmul_tiled(sub, b16, len(rows), size, size, out=np.ascontiguousarray(start[rows, :]), threads=orc.host_threads())
    assert rel_fro(to_host(out[torch_index(rows)]), want) <= TOL_BF16
