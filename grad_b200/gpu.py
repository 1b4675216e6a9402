"""Host-side mirror of grad's ``Gpu`` contraction wrappers (src/gpu/gpu.zig) on top of the C ABI.

Method names and argument meaning follow the reference (`matmul`, `convImplicitForward`,
`convF32Forward`, `convImplicitWeightGrad`, `convF32WeightGrad`) so the parity tests read like
tests/parity.zig and tests/autograd.zig.  Tensors are torch CUDA tensors used purely as device
buffers: the kernels receive their raw addresses, bf16 is 16-bit storage.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import abi
from .abi import ACT_NONE, ACT_RELU, BF16, F32, MATH_BF16, MATH_F32, MATH_TF32


@dataclass
class MatmulOpts:
    """src/gpu/gpu.zig:22 `MatmulOpts`."""

    trans_a: bool = False
    trans_b: bool = False
    accumulate: bool = False


@dataclass
class MatmulShape:
    """src/gpu/gpu.zig:29 `MatmulShape`."""

    m: int
    n: int
    k: int
    batch: int = 1


@dataclass
class Epilogue:
    bias: Optional[torch.Tensor] = None        # f32[n]
    residual: Optional[torch.Tensor] = None    # same shape / dtype as the output
    relu: bool = False
    round_tf32: bool = False                   # store the f32 result rounded to TF32 (nearest, ties away)
    stats_shift: Optional[torch.Tensor] = None # f32[n]: with stats_sums, batch-norm statistics of the stored result
    stats_sums: Optional[torch.Tensor] = None  # f32[2n], += sum(v - shift) and sum((v - shift)^2) per column
    stats_ordered: bool = False                # reproducible sums (ordered partials) instead of atomics


@dataclass
class ConvGeometry:
    """src/gpu/args.zig:78 `ConvGeometry` (forward geometry of the layer)."""

    n: int
    h: int
    w: int
    c: int
    k: int
    stride: int
    pad: int
    out_h: int
    out_w: int
    positions: int
    c_out: int
    dilation: int = 1
    c_step: int = 0
    subsample: int = 1
    groups: int = 1          # grouped convolution: carried in gb_conv_desc.groups, not in the C geometry struct

    def c_struct(self) -> abi.ConvGeometryC:
        return abi.ConvGeometryC(self.n, self.h, self.w, self.c, self.k, self.stride, self.pad, self.out_h, self.out_w,
                                 self.positions, self.c_out, self.dilation, self.c_step, self.subsample)


def conv_geometry(n, h, w, c, k, c_out, stride=1, pad=0, dilation=1, groups=1) -> ConvGeometry:
    """src/autograd/autograd.zig:99-141 `convGeometry` (forward case) with conv.zig's output-size formula."""
    oh = (h + 2 * pad - dilation * (k - 1) - 1) // stride + 1
    ow = (w + 2 * pad - dilation * (k - 1) - 1) // stride + 1
    return ConvGeometry(n, h, w, c, k, stride, pad, oh, ow, n * oh * ow, c_out, dilation, groups=groups)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype in (torch.bfloat16, torch.uint16, torch.int16):
        return BF16
    raise TypeError(f"unsupported dtype {t.dtype}: the path stores f32 or bf16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


class PreparedWeights:
    """A bf16 (or f32) copy of one f32 master weight matrix, made once and refreshed after the optimizer step
    (`gb_prepare_weights` / `gb_refresh_weights`): the reference converts the master on every use (`packMatrix`,
    src/autograd/autograd.zig:955, 1226, 1345).  `tensor` is the copy -- `(rows, cols)` for the plain kind,
    `(cols, rows)` for the rows kind -- to pass as `w` / `b` to the contraction calls."""

    def __init__(self, lib, stream, master: torch.Tensor, kind: int, dtype: torch.dtype):
        assert master.dtype == torch.float32 and master.dim() == 2 and master.is_contiguous()
        rows, cols = master.shape
        self.lib, self.master, self.kind = lib, master, kind
        self.tensor = torch.empty((cols, rows) if kind == abi.WEIGHTS_ROWS else (rows, cols), dtype=dtype, device=master.device)
        handle = C.c_void_p()
        abi.check(lib.gb_prepare_weights(stream, C.c_void_p(master.data_ptr()), rows, cols, kind, _dtype_code(self.tensor),
                                         C.c_void_p(self.tensor.data_ptr()), self.tensor.numel() * self.tensor.element_size(), C.byref(handle)),
                  "gb_prepare_weights")
        self.handle = handle
        assert lib.gb_weights_data(handle) == self.tensor.data_ptr()

    def refresh(self, stream):
        abi.check(self.lib.gb_refresh_weights(self.handle, stream), "gb_refresh_weights")

    def close(self):
        if self.handle:
            self.lib.gb_weights_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gpu:
    """One per device and host thread, like the reference's `Gpu` (src/gpu/gpu.zig:247-477).

    `tensor_cores`, `tf32` and `deterministic` are the reference's `Gpu.Config` (gpu.zig:291-298);
    `tensor_core_min_work` is its threshold for routing an f32 product to the bf16 kernels (:251, 703-705).
    """

    tensor_core_min_work = 1 << 22

    def __init__(self, device: int = 0, tensor_cores: bool = False, tf32: bool = False, deterministic: bool = False):
        if not torch.cuda.is_available():
            raise RuntimeError("grad_b200 needs a CUDA device: there is no CPU fallback")
        self.lib = abi.library()
        self.device = torch.device("cuda", device)
        self.tensor_cores = tensor_cores
        self.tf32 = tf32
        self.deterministic = deterministic
        torch.cuda.set_device(self.device)
        handle = C.c_void_p()
        abi.check(self.lib.gb_create(device, C.byref(handle)), "gb_create")
        self.handle = handle
        self.multiprocessors = int(self.lib.gb_sm_count(handle))
        self._scratch: Optional[torch.Tensor] = None
        self._needs = {}    # descriptor bytes -> workspace bytes (the query is a pure function of the descriptor)
        self.launches = 0   # calls into compute entry points (each is one or two kernel launches)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.gb_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- arena ------------------------------------------------------------------------------------
    def scratch(self, nbytes: int) -> Optional[torch.Tensor]:
        """Grow-only workspace, the role of `Gpu.scratch` (gpu.zig:403-410); allocated outside the timed step."""
        if nbytes == 0:
            return None
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self._scratch

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def prepareWeights(self, master: torch.Tensor, rows_layout: bool = False, dtype: torch.dtype = torch.bfloat16) -> PreparedWeights:
        """The prepared copy of an f32 master weight matrix; call `.refresh(gpu._stream())` after the optimizer step."""
        return PreparedWeights(self.lib, self._stream(), master, abi.WEIGHTS_ROWS if rows_layout else abi.WEIGHTS_PLAIN, dtype)

    def plan_cache_hits(self) -> int:
        return int(self.lib.gb_plan_cache_hits(self.handle))

    def check_status(self) -> int:
        """Synchronises and raises GB_ERR_TIMEOUT if a bounded device wait gave up."""
        word = C.c_uint32(0)
        rc = self.lib.gb_last_status(self.handle, self._stream(), C.byref(word))
        abi.check(rc, f"gb_last_status (device status {word.value})")
        return word.value

    def _count(self) -> int:
        info = abi.PlanInfo()
        self.lib.gb_last_plan(self.handle, C.byref(info))
        return int(info.kernel_launches)

    def last_plan(self) -> dict:
        """Tile width, stages, K split and operand paths of the last compute call (gb_last_plan)."""
        info = abi.PlanInfo()
        abi.check(self.lib.gb_last_plan(self.handle, C.byref(info)), "gb_last_plan")
        return {name: int(getattr(info, name)) for name, _ in abi.PlanInfo._fields_}

    # ---- host <-> device, `Gpu.upload` / `Gpu.download` (src/gpu/gpu.zig:412-431) ---------------------
    def upload(self, dst: torch.Tensor, src: torch.Tensor):
        dst.copy_(src, non_blocking=True)

    def download(self, dst: torch.Tensor, src: torch.Tensor):
        dst.copy_(src, non_blocking=True)

    def _epilogue(self, ep: Optional[Epilogue]):
        if ep is None:
            return None
        stats = None
        if ep.stats_sums is not None:
            self._stats = abi.BnStats(_ptr(ep.stats_shift), _ptr(ep.stats_sums), int(ep.stats_ordered), 0)   # kept alive for the call
            stats = C.pointer(self._stats)
        e = abi.Epilogue(_ptr(ep.bias), _ptr(ep.residual), ACT_RELU if ep.relu else ACT_NONE, abi.EPILOGUE_ROUND_TF32 if ep.round_tf32 else 0, stats)
        return C.byref(e)

    # ---- matmul family ----------------------------------------------------------------------------
    def tensorWorthwhile(self, m: int, n: int, k: int) -> bool:
        return self.tensor_cores and m * n * k >= self.tensor_core_min_work

    def _gemm_math(self, a, b, out, shape: MatmulShape, math: Optional[int]) -> int:
        if math is not None:
            return math
        wide = all(_dtype_code(t) == F32 for t in (a, b, out))
        if not wide or self.tensorWorthwhile(shape.m, shape.n, shape.k):
            return MATH_BF16
        return MATH_F32

    def matmul(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, shape: MatmulShape, opts: MatmulOpts = MatmulOpts(),
               epilogue: Optional[Epilogue] = None, math: Optional[int] = None, transpose_out: bool = False,
               lda: int = 0, ldb: int = 0, ldc: int = 0):
        """`Gpu.matmul` (src/gpu/gpu.zig:642-679): out (+)= op(a) * op(b), row-major; any operand may be bf16."""
        assert not (opts.trans_a and opts.trans_b)
        d = abi.GemmDesc()
        d.m, d.n, d.k, d.batch = shape.m, shape.n, shape.k, shape.batch
        d.stride_a, d.stride_b, d.stride_c = shape.m * shape.k, shape.k * shape.n, shape.m * shape.n
        d.lda, d.ldb, d.ldc = lda, ldb, ldc
        d.trans_a, d.trans_b, d.accumulate, d.transpose_out = opts.trans_a, opts.trans_b, opts.accumulate, transpose_out
        d.dtype_a, d.dtype_b, d.dtype_c = _dtype_code(a), _dtype_code(b), _dtype_code(out)
        d.math = self._gemm_math(a, b, out, shape, math)
        d.deterministic = self.deterministic
        key = bytes(d)
        need = self._needs.get(key)
        if need is None:
            size = C.c_size_t(0)
            abi.check(self.lib.gb_gemm_workspace(self.handle, C.byref(d), C.byref(size)), "gb_gemm_workspace")
            need = self._needs[key] = size.value
        ws = self.scratch(need)
        rc = self.lib.gb_gemm(self.handle, self._stream(), C.byref(d), _ptr(a), _ptr(b), _ptr(out), self._epilogue(epilogue),
                              _ptr(ws), need)
        abi.check(rc, "gb_gemm")
        self.launches += self._count()

    def matmulStrided(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, m: int, n: int, k: int, opts: MatmulOpts = MatmulOpts(),
                      batch: int = 1, strides=(0, 0, 0), ld=(0, 0, 0), outer: int = 1, outer_strides=(0, 0, 0),
                      epilogue: Optional[Epilogue] = None, math: Optional[int] = None):
        """The batched entry with explicit element strides (`GemmShape`, src/gpu/args.zig:1-12) and, with `outer` > 1, a second
        batch level: product (o, i) starts at i * strides[x] + o * outer_strides[x] in a, b and out.  The pointers may be
        views into larger tensors (a head's columns of a (rows, heads * width) activation)."""
        assert not (opts.trans_a and opts.trans_b)
        d = abi.GemmDesc()
        d.m, d.n, d.k, d.batch = m, n, k, batch
        d.stride_a, d.stride_b, d.stride_c = strides
        d.lda, d.ldb, d.ldc = ld
        d.batch_outer = outer
        d.stride_a_outer, d.stride_b_outer, d.stride_c_outer = outer_strides
        d.trans_a, d.trans_b, d.accumulate = opts.trans_a, opts.trans_b, opts.accumulate
        d.dtype_a, d.dtype_b, d.dtype_c = _dtype_code(a), _dtype_code(b), _dtype_code(out)
        d.math = self._gemm_math(a, b, out, MatmulShape(m, n, k, batch * outer), math)
        d.deterministic = self.deterministic
        key = bytes(d)
        need = self._needs.get(key)
        if need is None:
            size = C.c_size_t(0)
            abi.check(self.lib.gb_gemm_workspace(self.handle, C.byref(d), C.byref(size)), "gb_gemm_workspace")
            need = self._needs[key] = size.value
        ws = self.scratch(need)
        rc = self.lib.gb_gemm(self.handle, self._stream(), C.byref(d), _ptr(a), _ptr(b), _ptr(out), self._epilogue(epilogue),
                              _ptr(ws), need)
        abi.check(rc, "gb_gemm")
        self.launches += self._count()

    # ---- convolution ------------------------------------------------------------------------------
    def _conv_desc(self, geo: ConvGeometry, x_like, w_like, y_like, math: Optional[int], accumulate: bool, w_layout: int = 0) -> abi.ConvDesc:
        d = abi.ConvDesc()
        d.groups = getattr(geo, "groups", 1)
        d.geo = geo.c_struct()
        d.dtype_x, d.dtype_w, d.dtype_y = _dtype_code(x_like), _dtype_code(w_like), _dtype_code(y_like)
        if math is None:
            half = d.dtype_x == BF16 or d.dtype_y == BF16
            math = MATH_BF16 if (half or self.tensor_cores) else (MATH_TF32 if self.tf32 else MATH_F32)
        d.math = math
        d.accumulate = accumulate
        d.deterministic = self.deterministic
        d.w_layout = w_layout
        return d

    def _conv_ws(self, which: int, d: abi.ConvDesc):
        key = (which, bytes(d))
        need = self._needs.get(key)
        if need is None:
            size = C.c_size_t(0)
            abi.check(self.lib.gb_conv_workspace(self.handle, which, C.byref(d), C.byref(size)), "gb_conv_workspace")
            need = self._needs[key] = size.value
        return self.scratch(need), need

    def convForward(self, x, w, out, geo: ConvGeometry, accumulate: bool = False, epilogue: Optional[Epilogue] = None,
                    math: Optional[int] = None, w_rows: bool = False):
        """Forward implicit GEMM: `convImplicitForward` (gpu.zig:926-929) for bf16 data, `convF32Forward` (:789-826)
        for f32 data; x is NHWC, w is (k*k*c, c_out), or the prepared (c_out, k*k*c) copy when `w_rows`."""
        d = self._conv_desc(geo, x, w, out, math, accumulate, 1 if w_rows else 0)
        ws, n = self._conv_ws(abi.PASS_FPROP, d)
        rc = self.lib.gb_conv_fprop(self.handle, self._stream(), C.byref(d), _ptr(x), _ptr(w), _ptr(out), self._epilogue(epilogue),
                                    _ptr(ws), n)
        abi.check(rc, "gb_conv_fprop")
        self.launches += self._count()

    convImplicitForward = convForward
    convF32Forward = convForward

    def convInputGrad(self, dy, w, dx, geo: ConvGeometry, accumulate: bool = True, math: Optional[int] = None):
        """dx (+)= adjoint of the forward gather applied to dy * w^T.  The reference runs its forward kernel on the
        reversed geometry with rotated weights (autograd.zig:1052-1100, gpu.zig:856-866); here `geo` stays the
        forward geometry and `w` the unrotated weights."""
        d = self._conv_desc(geo, dx, w, dy, math, accumulate)
        ws, n = self._conv_ws(abi.PASS_DGRAD, d)
        rc = self.lib.gb_conv_dgrad(self.handle, self._stream(), C.byref(d), _ptr(dy), _ptr(w), _ptr(dx), _ptr(ws), n)
        abi.check(rc, "gb_conv_dgrad")
        self.launches += self._count()

    def convForwardAffine(self, x, w, out, geo: ConvGeometry, mean, inv_std, gamma, beta, epilogue: Optional[Epilogue] = None,
                          math: Optional[int] = None):
        """`convImplicitForwardAffineStats` (gpu.zig:951-959): the forward pass over relu(batch_norm(x)) that was never
        written out; the statistics of the result ride in `epilogue.stats_*`."""
        d = self._conv_desc(geo, x, w, out, math, False)
        ws, n = self._conv_ws(abi.PASS_FPROP, d)
        aff = abi.AffineInput(_ptr(mean), _ptr(inv_std), _ptr(gamma), _ptr(beta))
        rc = self.lib.gb_conv_fprop_affine(self.handle, self._stream(), C.byref(d), _ptr(x), _ptr(w), _ptr(out), self._epilogue(epilogue),
                                           C.byref(aff), _ptr(ws), n)
        abi.check(rc, "gb_conv_fprop_affine")
        self.launches += self._count()

    def convWeightGradAffine(self, dy, x, out, geo: ConvGeometry, mean, inv_std, gamma, beta, math: Optional[int] = None, accumulate: bool = True):
        """`convImplicitWeightGrad(..., aff)` (gpu.zig:983-1022): the weight gradient over the same virtual input."""
        d = self._conv_desc(geo, x, out, dy, math, accumulate)
        ws, n = self._conv_ws(abi.PASS_WGRAD, d)
        aff = abi.AffineInput(_ptr(mean), _ptr(inv_std), _ptr(gamma), _ptr(beta))
        rc = self.lib.gb_conv_wgrad_affine(self.handle, self._stream(), C.byref(d), _ptr(dy), _ptr(x), _ptr(out), C.byref(aff), _ptr(ws), n)
        abi.check(rc, "gb_conv_wgrad_affine")
        self.launches += self._count()

    def convInputGradDxStats(self, dy, w, dx, geo: ConvGeometry, x_bn, mean, inv_std, gamma, beta, sums, ordered: bool = False,
                             math: Optional[int] = None):
        """`convImplicitForwardDxStats` (gpu.zig:964-972): the input gradient (stored) whose epilogue also sums the masked
        batch-norm gradient g and g * x_hat per channel into `sums` (2 * c)."""
        d = self._conv_desc(geo, dx, w, dy, math, False)
        ws, n = self._conv_ws(abi.PASS_DGRAD, d)
        st = abi.DxStats(_ptr(x_bn), _ptr(mean), _ptr(inv_std), _ptr(gamma), _ptr(beta), _ptr(sums), int(ordered), 0)
        rc = self.lib.gb_conv_dgrad_stats(self.handle, self._stream(), C.byref(d), _ptr(dy), _ptr(w), _ptr(dx), C.byref(st), _ptr(ws), n)
        abi.check(rc, "gb_conv_dgrad_stats")
        self.launches += self._count()

    def convWeightGrad(self, dy, x, out, geo: ConvGeometry, math: Optional[int] = None, accumulate: bool = True):
        """`convImplicitWeightGrad` (gpu.zig:983-1022) / `convF32WeightGrad` (:828-866): out (taps, c_out) f32 += ...;
        dy is read as stored (positions, c_out), no transposed copy."""
        d = self._conv_desc(geo, x, out, dy, math, accumulate)
        ws, n = self._conv_ws(abi.PASS_WGRAD, d)
        rc = self.lib.gb_conv_wgrad(self.handle, self._stream(), C.byref(d), _ptr(dy), _ptr(x), _ptr(out), _ptr(ws), n)
        abi.check(rc, "gb_conv_wgrad")
        self.launches += self._count()

    convImplicitWeightGrad = convWeightGrad
    convF32WeightGrad = convWeightGrad
