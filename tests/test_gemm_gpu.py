"""GPU parity of the matmul family against the CPU oracle, through the C ABI.

Mirrors tests/parity.zig:20-114 of the reference (same shapes, same transpose / accumulate matrix, same
element-wise tolerance) and adds the tolerances the task states: relative Frobenius error <= 1e-5 (f32),
5e-3 (TF32), 2e-2 (bf16) against the f32 CPU result on the same seeded inputs.
"""
import numpy as np
import pytest

from tests.util import TOL_BF16, TOL_F32, TOL_TF32, close_like_parity_zig, rel_fro, seeded, to_dev, to_host

pytestmark = pytest.mark.gpu

PARITY_SHAPES = [(1, 1, 1), (5, 7, 3), (64, 64, 16), (65, 70, 17), (130, 33, 200), (784, 128, 64), (64, 10, 128), (200, 300, 784),
                 (25, 16, 4000), (400, 32, 4099), (512, 64, 576), (300, 130, 96), (32, 768, 128), (32, 512, 256), (32, 256, 768),
                 (256, 768, 32), (100, 600, 40)]
BATCHED_SHAPES = [(3, 5, 7, 3), (8, 64, 64, 16), (5, 65, 70, 17), (4, 16, 16, 64), (6, 40, 20, 33), (2, 20, 12, 700),
                  (12, 33, 129, 40), (1, 7, 9, 11), (16, 300, 48, 40), (1, 4096, 64, 300), (1, 640, 64, 4096)]
LAYOUTS = [(False, False), (True, False), (False, True)]


@pytest.fixture(scope="module")
def gpu():
    import grad_b200

    g = grad_b200.Gpu(0)
    yield g
    g.check_status()
    g.close()


def _oracle(a, b, m, k, n, ta, tb, start=None):
    from oracle import binding as orc

    out = None if start is None else start.copy()
    return orc.matmul_tiled(a, b, m, k, n, ta, tb, out=out, threads=orc.host_threads())


def _check(gpu, batch, m, n, k, ta, tb, accumulate, math, in_bf16=False, out_bf16=False, tol_elem=2e-4, tol_fro=None):
    import torch
    from grad_b200 import MatmulOpts, MatmulShape
    from oracle import binding as orc

    seed = batch * 7919 + m * 1000003 + n * 1009 + k
    a = seeded(seed, batch, *((k, m) if ta else (m, k)), kind="uniform_half")
    b = seeded(seed + 1, batch, *((n, k) if tb else (k, n)), kind="uniform_half")
    if in_bf16 or math == 2:
        # tests/parity.zig:70-73: the tensor-core run is compared on operands already rounded to bf16
        a, b = orc.bf16_round(a), orc.bf16_round(b)
    start = np.ones((batch, m, n), np.float32)
    want = np.stack([_oracle(a[i], b[i], m, k, n, ta, tb, start[i] if accumulate else None) for i in range(batch)])
    da, db = to_dev(a, in_bf16), to_dev(b, in_bf16)
    dc = to_dev(start, out_bf16)
    gpu.matmul(da, db, dc, MatmulShape(m, n, k, batch), MatmulOpts(ta, tb, accumulate), math=math)
    torch.cuda.synchronize()
    got = to_host(dc)
    if tol_fro is not None:
        assert rel_fro(got, want) <= tol_fro, (batch, m, n, k, ta, tb, accumulate, rel_fro(got, want))
    if tol_elem is not None:
        assert close_like_parity_zig(want, got, tol_elem), (batch, m, n, k, ta, tb, accumulate, float(np.abs(want - got).max()))


@pytest.mark.parametrize("shape", PARITY_SHAPES)
def test_f32_matmul_matches_cpu_for_every_transpose_and_accumulate(gpu, shape):
    m, n, k = shape
    for ta, tb in LAYOUTS:
        for acc in (False, True):
            _check(gpu, 1, m, n, k, ta, tb, acc, math=0, tol_elem=2e-4, tol_fro=TOL_F32)


@pytest.mark.parametrize("shape", PARITY_SHAPES)
def test_bf16_tensor_matmul_on_f32_storage(gpu, shape):
    """f32 tensors routed to the bf16 tensor cores (`--tensor-cores`): operands converted on the fly."""
    m, n, k = shape
    for ta, tb in LAYOUTS:
        for acc in (False, True):
            _check(gpu, 1, m, n, k, ta, tb, acc, math=2, tol_elem=2e-4, tol_fro=TOL_BF16)


@pytest.mark.parametrize("shape", PARITY_SHAPES)
def test_bf16_storage_matmul(gpu, shape):
    """bf16 operands consumed in place by TMA where pitches allow, f32 result."""
    m, n, k = shape
    for ta, tb in LAYOUTS:
        for acc in (False, True):
            _check(gpu, 1, m, n, k, ta, tb, acc, math=2, in_bf16=True, tol_elem=2e-4, tol_fro=TOL_BF16)


@pytest.mark.parametrize("shape", PARITY_SHAPES)
def test_tf32_matmul(gpu, shape):
    m, n, k = shape
    for ta, tb in LAYOUTS:
        for acc in (False, True):
            _check(gpu, 1, m, n, k, ta, tb, acc, math=1, tol_elem=None, tol_fro=TOL_TF32)


@pytest.mark.parametrize("shape", BATCHED_SHAPES)
@pytest.mark.parametrize("math", [0, 2])
def test_batched_matmul_matches_one_product_per_matrix(gpu, shape, math):
    batch, m, n, k = shape
    for ta, tb in LAYOUTS:
        for acc in (False, True):
            _check(gpu, batch, m, n, k, ta, tb, acc, math=math, tol_elem=2e-4)


def test_bf16_output_is_rounded_once(gpu):
    """A bf16 result is the f32 accumulator rounded to nearest even exactly once (gpu.zig:1040)."""
    import torch
    from grad_b200 import MatmulOpts, MatmulShape
    from oracle import binding as orc

    m, n, k = 256, 192, 320
    a, b = orc.bf16_round(seeded(1, m, k)), orc.bf16_round(seeded(2, k, n))
    want32 = _oracle(a, b, m, k, n, False, False)
    da, db = to_dev(a, True), to_dev(b, True)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    out32 = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    gpu.matmul(da, db, out, MatmulShape(m, n, k), MatmulOpts())
    gpu.matmul(da, db, out32, MatmulShape(m, n, k), MatmulOpts())
    torch.cuda.synchronize()
    got_bits = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_bits, orc.bf16_encode(to_host(out32)))   # same accumulator, one RNE rounding
    assert rel_fro(to_host(out), want32) <= TOL_BF16


@pytest.mark.parametrize("math,tol", [(0, TOL_F32), (1, TOL_TF32), (2, TOL_BF16)])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_fused_bias_relu_epilogue_equals_unfused_sequence(gpu, math, tol, layout):
    """relu(A*B + bias) in one launch == GEMM, then + bias, then max(.,0), each in f32 (autograd.zig:449-468)."""
    import torch
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape
    from oracle import binding as orc

    ta, tb = layout
    m, n, k = 384, 320, 448
    a = seeded(3, *((k, m) if ta else (m, k)))
    b = seeded(4, *((n, k) if tb else (k, n)))
    bias = seeded(5, n)
    want = orc.bias_act(_oracle(a, b, m, k, n, ta, tb), bias, True)
    in_bf16 = math == 2
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    gpu.matmul(to_dev(a, in_bf16), to_dev(b, in_bf16), out, MatmulShape(m, n, k), MatmulOpts(ta, tb),
               epilogue=Epilogue(bias=to_dev(bias), relu=True), math=math)
    torch.cuda.synchronize()
    got = to_host(out)
    assert rel_fro(got, want) <= tol, rel_fro(got, want)
    assert (got >= 0).all()


@pytest.mark.parametrize("size", [1024, 2048])
@pytest.mark.parametrize("math,tol", [(1, TOL_TF32), (2, TOL_BF16)])
def test_sweep_sizes_against_oracle(gpu, size, math, tol):
    """The benchmark's sweep shapes at sizes the CPU oracle finishes in seconds, N(0,1) inputs, bias + ReLU."""
    import torch
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape
    from oracle import binding as orc

    m = n = k = size
    a, b, bias = seeded(11, m, k), seeded(12, k, n), seeded(13, n)
    want = orc.bias_act(_oracle(a, b, m, k, n, False, False), bias, True)
    in_bf16 = math == 2
    out = torch.empty(m, n, dtype=torch.bfloat16 if in_bf16 else torch.float32, device="cuda")
    gpu.matmul(to_dev(a, in_bf16), to_dev(b, in_bf16), out, MatmulShape(m, n, k), MatmulOpts(),
               epilogue=Epilogue(bias=to_dev(bias), relu=True), math=math)
    torch.cuda.synchronize()
    assert rel_fro(to_host(out), want) <= tol


def test_transpose_out_and_pitched_output(gpu):
    """`transpose_out` and `c_pitch` of TensorShape (args.zig:72): C written as (n, m) into a wider buffer."""
    import torch
    from grad_b200 import MatmulOpts, MatmulShape

    m, n, k = 200, 96, 160
    a, b = seeded(21, m, k), seeded(22, k, n)
    want = _oracle(a, b, m, k, n, False, False)
    for math, tol in ((0, TOL_F32), (2, TOL_BF16)):
        out = torch.full((n, m + 8), 7.0, dtype=torch.float32, device="cuda")
        gpu.matmul(to_dev(a), to_dev(b), out, MatmulShape(m, n, k), MatmulOpts(), math=math, transpose_out=True, ldc=m + 8)
        torch.cuda.synchronize()
        got = to_host(out)
        assert rel_fro(got[:, :m].T, want) <= tol
        assert (got[:, m:] == 7.0).all()   # nothing outside the logical matrix is touched


def test_linearity_and_empty_products(gpu):
    """Size-independent properties: A*(B1+B2) == A*B1 + A*B2 within tolerance; m, n or k of zero is a no-op / zero."""
    import torch
    from grad_b200 import MatmulOpts, MatmulShape

    m, n, k = 512, 384, 1024
    a, b1, b2 = seeded(31, m, k), seeded(32, k, n), seeded(33, k, n)
    outs = []
    for b in (b1, b2, b1 + b2):
        o = torch.empty(m, n, device="cuda")
        gpu.matmul(to_dev(a), to_dev(b), o, MatmulShape(m, n, k), MatmulOpts(), math=0)
        outs.append(to_host(o))
    assert rel_fro(outs[0] + outs[1], outs[2]) <= 1e-5
    o = torch.full((4, 4), 3.0, device="cuda")
    gpu.matmul(to_dev(np.zeros((4, 0), np.float32)), to_dev(np.zeros((0, 4), np.float32)), o, MatmulShape(4, 4, 0), MatmulOpts(), math=0)
    torch.cuda.synchronize()
    assert (to_host(o) == 0).all()
    gpu.matmul(to_dev(a), to_dev(b1), o, MatmulShape(0, n, k), MatmulOpts(), math=2)   # empty grid: nothing happens
    torch.cuda.synchronize()


def test_rejects_both_transposes(gpu):
    import torch
    from grad_b200 import GbError, MatmulOpts, MatmulShape
    from grad_b200 import abi

    d = abi.GemmDesc()
    d.m = d.n = d.k = 8
    d.trans_a = d.trans_b = 1
    need = __import__("ctypes").c_size_t(0)
    assert gpu.lib.gb_gemm_workspace(gpu.handle, d, need) == 1   # GB_ERR_INVALID (src/gpu/gpu.zig:643)
    with pytest.raises(AssertionError):
        t = torch.zeros(8, 8, device="cuda")
        gpu.matmul(t, t, t, MatmulShape(8, 8, 8), MatmulOpts(True, True))
    assert issubclass(GbError, RuntimeError)


@pytest.mark.parametrize("heads,seqs,seq,hd", [(4, 6, 128, 64), (2, 3, 64, 32), (3, 5, 96, 64)])
def test_two_batch_levels_match_one_launch_per_head(gpu, heads, seqs, seq, hd):
    """The attention products of a fused-QKV layout -- activations (rows, 3 * heads * hd), one product per (sequence, head)
    -- as ONE launch with two batch levels (sequence inside, head outside) against one launch per head with a single batch
    level (src/gpu/args.zig:1-12 strides) and against the oracle: scores = Q K^T (NT), mix = P V (NN), dV = P^T dO (TN)."""
    import torch
    from grad_b200 import MatmulOpts
    from oracle import binding as orc

    d = heads * hd
    rows = seqs * seq
    rng = np.random.default_rng(77 + heads)
    qkv = orc.bf16_round(rng.standard_normal((rows, 3 * d), dtype=np.float32))
    do_ = orc.bf16_round(rng.standard_normal((rows, d), dtype=np.float32))
    tq, tdo = to_dev(qkv, True), to_dev(do_, True)
    st = seq * 3 * d

    def run(two_levels, a, b, out, m, n, k, opts, strides, ld, outer_strides):
        if two_levels:
            gpu.matmulStrided(a(0), b(0), out(0), m, n, k, opts, batch=seqs, strides=strides, ld=ld, outer=heads, outer_strides=outer_strides)
        else:
            for h in range(heads):
                gpu.matmulStrided(a(h), b(h), out(h), m, n, k, opts, batch=seqs, strides=strides, ld=ld)

    results = []
    for two_levels in (True, False):
        p = torch.full((heads * seqs, seq, seq), -7.0, dtype=torch.bfloat16, device="cuda")
        o = torch.full((rows, d), -7.0, dtype=torch.bfloat16, device="cuda")
        dv = torch.full((rows, 3 * d), -7.0, dtype=torch.bfloat16, device="cuda")
        q = lambda h: tq[:, h * hd:]
        k_ = lambda h: tq[:, d + h * hd:]
        v = lambda h: tq[:, 2 * d + h * hd:]
        run(two_levels, q, k_, lambda h: p[h * seqs:], seq, seq, hd, MatmulOpts(False, True), (st, st, seq * seq), (3 * d, 3 * d, 0),
            (hd, hd, seqs * seq * seq))
        run(two_levels, lambda h: p[h * seqs:], v, lambda h: o[:, h * hd:], seq, hd, seq, MatmulOpts(), (seq * seq, st, seq * d), (0, 3 * d, d),
            (seqs * seq * seq, hd, hd))
        run(two_levels, lambda h: p[h * seqs:], lambda h: tdo[:, h * hd:], lambda h: dv[:, 2 * d + h * hd:], seq, hd, seq, MatmulOpts(True, False),
            (seq * seq, seq * d, st), (0, d, 3 * d), (seqs * seq * seq, hd, hd))
        torch.cuda.synchronize()
        results.append((p.clone(), o.clone(), dv.clone()))
    for one, per_head in zip(results[0], results[1]):
        assert torch.equal(one, per_head)
    # and against the oracle: head 1 of the second sequence
    h, s_ = 1 % heads, 1 % seqs
    r0 = s_ * seq
    qh, kh, vh = (qkv[r0:r0 + seq, part * d + h * hd:part * d + (h + 1) * hd] for part in range(3))
    want_p = orc.matmul_tiled(np.ascontiguousarray(qh), np.ascontiguousarray(kh), seq, hd, seq, False, True)
    got_p = to_host(results[0][0][h * seqs + s_])
    assert rel_fro(got_p, want_p) <= TOL_BF16
    want_o = orc.matmul_tiled(orc.bf16_round(got_p), np.ascontiguousarray(vh), seq, seq, hd, False, False)
    assert rel_fro(to_host(results[0][1][r0:r0 + seq, h * hd:(h + 1) * hd]), want_o) <= TOL_BF16
    # untouched columns of dv stay as they were (the launch writes the V third only)
    assert (to_host(results[0][2][:, :2 * d]) == -7.0).all()


def test_two_batch_levels_reject_what_they_cannot_do(gpu):
    """Strict f32 and operands that TMA cannot reach have no second batch level: GB_ERR_UNSUPPORTED, nothing launched."""
    import torch
    from grad_b200 import MatmulOpts
    from grad_b200.abi import GbError

    a = torch.zeros((4, 64, 64), device="cuda")
    out = torch.zeros((4, 64, 64), device="cuda")
    with pytest.raises(GbError):
        gpu.matmulStrided(a, a, out, 64, 64, 64, MatmulOpts(), batch=2, strides=(4096, 4096, 4096), outer=2, outer_strides=(8192, 8192, 8192), math=0)


@pytest.mark.parametrize("math,tol", [(1, TOL_TF32), (2, TOL_BF16)])
@pytest.mark.parametrize("m,n,k", [(96, 40, 72), (200, 136, 64)])
def test_two_batch_levels_with_ragged_tiles_against_the_oracle(gpu, math, tol, m, n, k):
    """Two batch levels on shapes whose tiles overhang (rows past m, a last chunk narrower than 32 columns: the per-lane
    store path) and with padded pitches, every product against the oracle; accumulate adds to the old C."""
    import torch
    from grad_b200 import MatmulOpts
    from oracle import binding as orc

    inner, outer = 3, 2
    lda, ldb, ldc = k + 8, n + 8, n + 8
    rng = np.random.default_rng(5 + m + math)
    a = rng.standard_normal((outer, inner, m, lda), dtype=np.float32)
    b = rng.standard_normal((outer, inner, k, ldb), dtype=np.float32)
    c0 = rng.standard_normal((outer, inner, m, ldc), dtype=np.float32)
    half = math == 2
    if half:
        a, b, c0 = orc.bf16_round(a), orc.bf16_round(b), orc.bf16_round(c0)
    ta, tb, tc = to_dev(a, half), to_dev(b, half), to_dev(c0, half)
    gpu.matmulStrided(ta, tb, tc, m, n, k, MatmulOpts(False, False, True), batch=inner, strides=(m * lda, k * ldb, m * ldc), ld=(lda, ldb, ldc),
                      outer=outer, outer_strides=(inner * m * lda, inner * k * ldb, inner * m * ldc), math=math)
    torch.cuda.synchronize()
    got = to_host(tc)
    for o in range(outer):
        for i in range(inner):
            want = orc.matmul_tiled(np.ascontiguousarray(a[o, i, :, :k]), np.ascontiguousarray(b[o, i, :, :n]), m, k, n, False, False,
                                    out=np.ascontiguousarray(c0[o, i, :, :n]))
            assert rel_fro(got[o, i, :, :n], want) <= tol, (o, i, rel_fro(got[o, i, :, :n], want))
            assert np.array_equal(got[o, i, :, n:], c0[o, i, :, n:])   # the padding columns are not written
