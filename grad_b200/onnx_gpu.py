"""Host-side mirror of `grad.onnx_gpu.Executor` (src/onnx/gpu.zig) for the graphs grad's exporter writes.

The graph is held in memory (`Model`: nodes, initializers, inputs, outputs — the fields of the reference's
`runtime.Model`); the ONNX protobuf reader is not part of this path.  `Executor.run` walks the nodes like
`Executor.run` / `step` (gpu.zig:175-250): a Transpose-Conv-Transpose or Transpose-Pool-Transpose window runs
as one NHWC op (`fusedWindow`, :279-302), OIHW filters are reordered once per weight (`reorderedWeights`,
:566-574), and — new here — the bias, a following `Add` of a residual and a following `Relu` are folded
into the convolution's epilogue, and `MatMul` + `Add(bias)` into one product, so Conv+bias+Add+Relu is one
launch instead of four.  Values may be bf16 (`mode="bf16"`) or f32 (`"tf32"`, `"f32"`).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import abi
from .abi import BF16, F32, MATH_BF16, MATH_F32, MATH_TF32
from .gpu import Epilogue, Gpu, MatmulOpts, MatmulShape, conv_geometry


@dataclass
class Node:
    op: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, object] = field(default_factory=dict)


@dataclass
class Model:
    nodes: List[Node]
    initializers: Dict[str, np.ndarray]
    inputs: List[str]
    outputs: List[str]


@dataclass
class Stats:
    """src/onnx/gpu.zig:155 `Stats`, plus the launches the run issued."""

    device_nodes: int = 0
    host_nodes: int = 0
    uploads: int = 0
    downloads: int = 0
    launches: int = 0


_TO_NCHW = (0, 3, 1, 2)
_TO_NHWC = (0, 2, 3, 1)


def _pair(attrs, name, default):
    v = attrs.get(name)
    if v is None:
        return default
    a, b = int(v[0]), int(v[1] if len(v) > 1 else v[0])
    if a != b:
        raise NotImplementedError(f"{name} must be square on this path (src/onnx/runtime.zig:887)")
    return a


class Executor:
    def __init__(self, model: Model, gpu: Gpu, mode: str = "bf16", fuse: bool = True):
        assert mode in ("bf16", "tf32", "f32")
        self.model, self.gpu, self.mode, self.fuse = model, gpu, mode, fuse
        self.act_dtype = torch.bfloat16 if mode == "bf16" else torch.float32
        self.math = {"bf16": MATH_BF16, "tf32": MATH_TF32, "f32": MATH_F32}[mode]
        self.stats = Stats()
        self.constants: Dict[str, torch.Tensor] = {}   # initializers on the device, as stored
        self.derived: Dict[str, torch.Tensor] = {}     # reordered / cast weights, built once (gpu.zig:566-574)
        self.uses: Dict[str, int] = {}
        for node in model.nodes:
            for name in node.inputs:
                self.uses[name] = self.uses.get(name, 0) + 1
        for name in model.outputs:
            self.uses[name] = self.uses.get(name, 0) + 1
        self.peak_live = 0    # most values alive at once during the last walk
        self._graph = None
        self._static_in: Dict[str, torch.Tensor] = {}
        self._static_out: Dict[str, torch.Tensor] = {}

    # ---- helpers ------------------------------------------------------------------------------------
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.gpu.device).cuda_stream)

    def _code(self, t: torch.Tensor) -> int:
        return BF16 if t.dtype == torch.bfloat16 else F32

    def _constant(self, name: str) -> torch.Tensor:
        if name not in self.constants:
            self.constants[name] = torch.from_numpy(np.ascontiguousarray(self.model.initializers[name], dtype=np.float32)).to(self.gpu.device)
            self.stats.uploads += 1
        return self.constants[name]

    def _conv_weights(self, name: str):
        key = name + "/taps"
        if key not in self.derived:
            w = self._constant(name)
            m, c, kh, kw = w.shape
            if self.mode == "tf32":   # filters are rounded to TF32 once (nearest), not truncated at every use
                w = (w.view(torch.int32) + 0x1000).bitwise_and(-8192).view(torch.float32)
            # filters are kept as (c_out, kh*kw*c): K contiguous per output channel (gb_conv_desc.w_layout = 1) -- unless such a
            # row is not a whole number of 16-byte units (the 3-channel stem: 27 values), which TMA cannot fetch: those stay
            # (kh*kw*c, c_out), whose rows of c_out values it can
            rows = (kh * kw * c * torch.empty((), dtype=self.act_dtype).element_size()) % 16 == 0
            out = torch.empty((m, kh * kw * c) if rows else (kh * kw * c, m), dtype=self.act_dtype, device=self.gpu.device)
            fn = self.gpu.lib.gb_reorder_oihw_rows if rows else self.gpu.lib.gb_reorder_oihw
            abi.check(fn(self._stream(), self._code(out), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()), m, c, kh, kw),
                      "gb_reorder_oihw_rows" if rows else "gb_reorder_oihw")
            self.derived[key] = (out, rows)
            self.stats.launches += 1
        return self.derived[key]

    def _matrix(self, name: str) -> torch.Tensor:
        key = name + "/" + self.mode
        if key not in self.derived:
            self.derived[key] = self._constant(name).to(self.act_dtype).contiguous()
        return self.derived[key]

    def _padded(self, name: str, cols: int, vector: bool) -> torch.Tensor:
        """A constant matrix (or bias vector) with zero columns appended up to `cols`, made once.  A product whose
        column count is not a multiple of 8 (the 10 logits) can use neither TMA boxes nor 16-byte stores (the
        classifier took 50 us through the gather warps and the scalar epilogue, a ninth of a batch-100 pass), and a
        last chunk of fewer than 32 columns still takes the guarded per-element path (13.7 us against 6.3 us for
        the same product padded to 32 columns), so the padding goes to whole 32-column chunks."""
        key = f"{name}/pad{cols}/{self.mode}"
        if key not in self.derived:
            src = self._constant(name) if vector else self._matrix(name)
            out = torch.zeros(src.shape[:-1] + (cols,), dtype=src.dtype, device=src.device)
            out[..., : src.shape[-1]] = src
            # the matrix is kept as (cols, K) rows: a K-major B operand that TMA fetches whatever `cols` is
            self.derived[key] = out if vector else out.t().contiguous()
        return self.derived[key]

    def _value(self, values, name: str) -> torch.Tensor:
        if name in values:
            return values[name]
        if name in self.model.initializers:
            t = self._constant(name)
            return t if t.dtype == self.act_dtype or t.dim() <= 1 else self._matrix(name)
        raise KeyError(f"missing input {name} (error.MissingInput)")

    def _single_use(self, name: str) -> bool:
        return self.uses.get(name, 0) == 1 and name not in self.model.outputs

    def _elementwise(self, op: int, a: torch.Tensor, b: Optional[torch.Tensor], cols: int = 1) -> torch.Tensor:
        out = torch.empty_like(a)
        abi.check(self.gpu.lib.gb_elementwise(self._stream(), op, self._code(a), C.c_void_p(a.data_ptr()),
                                              None if b is None else C.c_void_p(b.data_ptr()), C.c_void_p(out.data_ptr()), a.numel(), cols),
                  "gb_elementwise")
        self.stats.launches += 1
        return out

    # ---- node windows ---------------------------------------------------------------------------------
    def _is_transpose(self, node: Node, perm) -> bool:
        return node.op == "Transpose" and tuple(node.attrs.get("perm", ())) == perm

    def _window(self, at: int, middle: Sequence[str]) -> Optional[Node]:
        """`fusedWindow` (gpu.zig:279-302): Transpose(0,3,1,2) -> op -> Transpose(0,2,3,1), each used once."""
        nodes = self.model.nodes
        if at + 2 >= len(nodes):
            return None
        a, b, c = nodes[at], nodes[at + 1], nodes[at + 2]
        if not (self._is_transpose(a, _TO_NCHW) and b.op in middle and self._is_transpose(c, _TO_NHWC)):
            return None
        if b.inputs[0] != a.outputs[0] or c.inputs[0] != b.outputs[0]:
            return None
        if not (self._single_use(a.outputs[0]) and self._single_use(b.outputs[0])):
            return None
        return b

    def _conv_nhwc(self, values, x: torch.Tensor, node: Node, out_name: str, at_next: int) -> int:
        """`convNhwc` (gpu.zig:576-610) with the bias / Add / Relu that follow folded into the epilogue.
        Returns how many nodes after the window were consumed."""
        if int(node.attrs.get("group", 1)) != 1:
            raise NotImplementedError("grouped convolution takes the NCHW host path in the reference (runtime.zig:871)")
        w, w_rows = self._conv_weights(node.inputs[1])
        m, taps_c = (w.shape[0], w.shape[1]) if w_rows else (w.shape[1], w.shape[0])
        n, h, width, c = x.shape
        k = int(round((taps_c // c) ** 0.5))
        stride, pad, dil = _pair(node.attrs, "strides", 1), _pair(node.attrs, "pads", 0), _pair(node.attrs, "dilations", 1)
        geo = conv_geometry(n, h, width, c, k, m, stride, pad, dil)
        bias = self._constant(node.inputs[2]) if len(node.inputs) > 2 else None
        residual, relu, consumed, result = None, False, 0, out_name
        nodes = self.model.nodes
        if self.fuse:
            nxt = nodes[at_next] if at_next < len(nodes) else None
            if nxt is not None and nxt.op == "Add" and result in nxt.inputs and self._single_use(result):
                other = nxt.inputs[1] if nxt.inputs[0] == result else nxt.inputs[0]
                if other in values and values[other].shape == (n, geo.out_h, geo.out_w, m) and values[other].dtype == self.act_dtype:
                    residual, result, consumed = values[other].contiguous(), nxt.outputs[0], consumed + 1
                    nxt = nodes[at_next + consumed] if at_next + consumed < len(nodes) else None
            if nxt is not None and nxt.op == "Relu" and nxt.inputs[0] == result and self._single_use(result):
                relu, result, consumed = True, nxt.outputs[0], consumed + 1
        y = torch.empty((n, geo.out_h, geo.out_w, m), dtype=self.act_dtype, device=self.gpu.device)
        before = self.gpu.launches
        self.gpu.convForward(x.contiguous(), w, y, geo, epilogue=Epilogue(bias, residual, relu, self.mode == "tf32"), math=self.math, w_rows=w_rows)
        self.stats.launches += self.gpu.launches - before
        values[result] = y
        self.stats.device_nodes += 3 + consumed
        return consumed

    def _pool_nhwc(self, values, x: torch.Tensor, node: Node, out_name: str):
        k = _pair(node.attrs, "kernel_shape", 1)
        stride, pad = _pair(node.attrs, "strides", 1), _pair(node.attrs, "pads", 0)
        n, h, w, c = x.shape
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        y = torch.empty((n, oh, ow, c), dtype=x.dtype, device=x.device)
        abi.check(self.gpu.lib.gb_pool2d(self._stream(), int(node.op == "MaxPool"), self._code(x), C.c_void_p(x.contiguous().data_ptr()),
                                         C.c_void_p(y.data_ptr()), n, h, w, c, k, stride, pad), "gb_pool2d")
        self.stats.launches += 1
        values[out_name] = y
        self.stats.device_nodes += 3

    def _matmul(self, values, at: int) -> int:
        """`Executor.matmul` (gpu.zig:477-499) with a following Add(bias vector) folded in."""
        node = self.model.nodes[at]
        x = self._value(values, node.inputs[0])
        w = self._matrix(node.inputs[1]) if node.inputs[1] in self.model.initializers else self._value(values, node.inputs[1])
        rows = int(np.prod(x.shape[:-1]))
        k, n = x.shape[-1], w.shape[-1]
        result, bias, consumed = node.outputs[0], None, 1
        nxt = self.model.nodes[at + 1] if at + 1 < len(self.model.nodes) else None
        if self.fuse and nxt is not None and nxt.op == "Add" and result in nxt.inputs and self._single_use(result):
            other = nxt.inputs[1] if nxt.inputs[0] == result else nxt.inputs[0]
            if other in self.model.initializers and self.model.initializers[other].shape == (n,):
                bias, result, consumed = self._constant(other), nxt.outputs[0], 2
        out_dtype = torch.float32 if result in self.model.outputs else self.act_dtype
        cols = n
        if n % 32 != 0 and n % 8 != 0 and node.inputs[1] in self.model.initializers:
            cols = (n + 31) // 32 * 32   # whole 32-column chunks: the epilogue's staged TMA stores, no ragged tail
            w = self._padded(node.inputs[1], cols, False)
            if bias is not None:
                bias = self._padded(other, cols, True)
        y = torch.empty(tuple(x.shape[:-1]) + (cols,), dtype=out_dtype, device=self.gpu.device)
        before = self.gpu.launches
        self.gpu.matmul(x.contiguous(), w, y, MatmulShape(rows, cols, k), MatmulOpts(False, cols != n), epilogue=Epilogue(bias, None, False), math=self.math)
        self.stats.launches += self.gpu.launches - before
        values[result] = y if cols == n else y[..., :n]
        self.stats.device_nodes += consumed
        return consumed

    def _gemm(self, values, at: int) -> int:
        """`Executor.gemm` (gpu.zig:500-521): Y = op(A) * op(B) + C for alpha = beta = 1 and at most one transposed
        operand (anything else is a host node in the reference and outside this path).  C broadcasts over the rows
        (a bias vector: folded into the epilogue) or has the result's shape (added as the epilogue's residual); a
        following Relu is folded in as well."""
        node = self.model.nodes[at]
        ta, tb = int(node.attrs.get("transA", 0)) != 0, int(node.attrs.get("transB", 0)) != 0
        if (ta and tb) or float(node.attrs.get("alpha", 1.0)) != 1.0 or float(node.attrs.get("beta", 1.0)) != 1.0:
            raise NotImplementedError("Gemm with alpha/beta != 1 or both operands transposed runs on the host in the reference (gpu.zig:503)")
        x = self._value(values, node.inputs[0]).contiguous()
        w = self._matrix(node.inputs[1]) if node.inputs[1] in self.model.initializers else self._value(values, node.inputs[1]).contiguous()
        if x.dim() != 2 or w.dim() != 2:
            raise NotImplementedError("Gemm operands must be matrices (gpu.zig:506)")
        m, k = (x.shape[1], x.shape[0]) if ta else (x.shape[0], x.shape[1])
        n = w.shape[0] if tb else w.shape[1]
        if (w.shape[1] if tb else w.shape[0]) != k:
            raise ValueError("Gemm: inner dimensions differ (error.ShapeMismatch)")
        bias, residual = None, None
        if len(node.inputs) > 2 and node.inputs[2]:
            c = self._constant(node.inputs[2]) if node.inputs[2] in self.model.initializers else self._value(values, node.inputs[2])
            if tuple(c.shape) in ((n,), (1, n)):
                bias = c.reshape(n).float().contiguous()
            elif tuple(c.shape) == (m, n):
                residual = c.to(torch.float32 if node.outputs[0] in self.model.outputs else self.act_dtype).contiguous()
            else:
                raise NotImplementedError("Gemm: C must broadcast over the rows or have the result's shape (gpu.zig:512-516)")
        result, relu, consumed = node.outputs[0], False, 1
        nxt = self.model.nodes[at + 1] if at + 1 < len(self.model.nodes) else None
        if self.fuse and nxt is not None and nxt.op == "Relu" and nxt.inputs[0] == result and self._single_use(result):
            relu, result, consumed = True, nxt.outputs[0], 2
        out_dtype = torch.float32 if result in self.model.outputs else self.act_dtype
        if residual is not None and residual.dtype != out_dtype:
            residual = residual.to(out_dtype)
        y = torch.empty((m, n), dtype=out_dtype, device=self.gpu.device)
        before = self.gpu.launches
        self.gpu.matmul(x, w, y, MatmulShape(m, n, k), MatmulOpts(ta, tb), epilogue=Epilogue(bias, residual, relu), math=self.math)
        self.stats.launches += self.gpu.launches - before
        values[result] = y
        self.stats.device_nodes += consumed
        return consumed

    # ---- the walk -------------------------------------------------------------------------------------
    def _step(self, values, at: int) -> int:
        nodes = self.model.nodes
        node = nodes[at]
        conv = self._window(at, ("Conv",))
        if conv is not None:
            x = self._value(values, nodes[at].inputs[0])
            return 3 + self._conv_nhwc(values, x, conv, nodes[at + 2].outputs[0], at + 3)
        pool = self._window(at, ("MaxPool", "AveragePool"))
        if pool is not None:
            self._pool_nhwc(values, self._value(values, nodes[at].inputs[0]), pool, nodes[at + 2].outputs[0])
            return 3
        if node.op == "MatMul":
            return self._matmul(values, at)
        if node.op == "Gemm":
            return self._gemm(values, at)
        if node.op == "Relu":
            values[node.outputs[0]] = self._elementwise(1, self._value(values, node.inputs[0]).contiguous(), None)
        elif node.op == "Add":
            a, b = self._value(values, node.inputs[0]), self._value(values, node.inputs[1])
            if b.dim() == 1 and a.dim() > 1:
                values[node.outputs[0]] = self._elementwise(3, a.contiguous(), b.float().contiguous(), b.numel())
            else:
                values[node.outputs[0]] = self._elementwise(0, a.contiguous(), b.contiguous())
        elif node.op in ("Reshape", "Flatten"):
            x = self._value(values, node.inputs[0])
            if node.op == "Flatten":
                shape = (x.shape[0], -1)
            else:
                shape = tuple(int(v) for v in (node.attrs.get("shape") if "shape" in node.attrs else self.model.initializers[node.inputs[1]]))
                shape = tuple(x.shape[i] if v == 0 else v for i, v in enumerate(shape))
            values[node.outputs[0]] = x.reshape(shape)
        elif node.op == "Transpose" and tuple(node.attrs.get("perm", ())) in (_TO_NCHW, _TO_NHWC):
            x = self._value(values, node.inputs[0]).contiguous()
            to_nhwc = tuple(node.attrs["perm"]) == _TO_NHWC
            n, d1, d2, d3 = x.shape
            (c, h, w) = (d1, d2, d3) if to_nhwc else (d3, d1, d2)
            y = torch.empty((n, h, w, c) if to_nhwc else (n, c, h, w), dtype=x.dtype, device=x.device)
            abi.check(self.gpu.lib.gb_permute_layout(self._stream(), self._code(x), int(to_nhwc), C.c_void_p(x.data_ptr()),
                                                     C.c_void_p(y.data_ptr()), n, c, h, w), "gb_permute_layout")
            self.stats.launches += 1
            values[node.outputs[0]] = y
        else:
            raise NotImplementedError(f"node kind {node.op} is outside the contraction path (error.UnsupportedOp)")
        self.stats.device_nodes += 1
        return 1

    def _walk(self, values) -> Dict[str, torch.Tensor]:
        """Runs the nodes in order.  A value is dropped as soon as its last consumer has run (the reference keeps every
        activation until the next `run`, its TODO.md:15), so peak memory follows the live set of the graph, not its
        length: at batch 4096 the ResNet holds three or four activation maps instead of forty."""
        remaining = dict(self.uses)
        self.peak_live = 0
        at = 0
        while at < len(self.model.nodes):
            done = self._step(values, at)
            for node in self.model.nodes[at:at + done]:
                for name in node.inputs:
                    if name in remaining:
                        remaining[name] -= 1
                        if remaining[name] == 0 and name in values and name not in self.model.outputs:
                            del values[name]
            self.peak_live = max(self.peak_live, len(values))
            at += done
        return {name: values[name] for name in self.model.outputs}

    def run_device(self, feeds: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Runs the graph on device-resident feeds (f32 or the activation dtype) and returns device outputs."""
        values = {}
        for name, t in feeds.items():
            if t.dtype != self.act_dtype:
                src = t.contiguous()
                t = torch.empty(src.shape, dtype=self.act_dtype, device=src.device)
                abi.check(self.gpu.lib.gb_cast(self._stream(), self._code(src), self._code(t), C.c_void_p(src.data_ptr()), C.c_void_p(t.data_ptr()),
                                               src.numel()), "gb_cast")
                self.stats.launches += 1
            values[name] = t
        for name in self.model.inputs:
            if name not in values:
                raise KeyError(f"missing input {name} (error.MissingInput)")
        return self._walk(values)

    def run(self, feeds: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        """`Executor.run` (gpu.zig:175-204): host feeds in, host outputs out; one upload per feed, one download per output."""
        self.stats = Stats(uploads=0)
        dev = {}
        for name, arr in feeds.items():
            dev[name] = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(self.gpu.device, non_blocking=True)
            self.stats.uploads += 1
        outs = self.run_device(dev)
        host = {}
        for name, t in outs.items():
            host[name] = t.float().cpu().numpy()
            self.stats.downloads += 1
        return host

    # ---- replay ---------------------------------------------------------------------------------------
    def capture(self, example: Dict[str, torch.Tensor]):
        """Records one run into a CUDA graph, the executor-side use of grad's capture / replay
        (src/gpu/gpu.zig:446-477): `replay` then re-issues every launch of the run with one call."""
        self.run_device(example)   # builds the weight caches outside the capture
        torch.cuda.synchronize()
        self._static_in = {k: v.clone() for k, v in example.items()}
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._static_out = self.run_device(self._static_in)
        self._graph = graph

    def replay(self, feeds: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        for k, v in feeds.items():
            self._static_in[k].copy_(v, non_blocking=True)
        self._graph.replay()
        return self._static_out


def resnet14_model(w1: int = 64, w2: int = 192, w3: int = 384, classes: int = 10, seed: int = 1238) -> Model:
    """The inference graph grad's exporter writes for examples/cifar (main.zig:15-68) with batch norm folded into
    the filters and a bias (src/onnx/onnx.zig:322-363): Reshape, then Transpose-Conv-Transpose windows with
    Relu / Add-Relu, MaxPool and AveragePool windows, Reshape, MatMul + Add.  He-normal filters (nn.zig:100-105),
    folded bias ~ N(0, 0.1), all from `seed`."""
    rng = np.random.default_rng(seed)
    nodes: List[Node] = []
    init: Dict[str, np.ndarray] = {}
    counter = [0]

    def fresh(prefix):
        counter[0] += 1
        return f"{prefix}_{counter[0]}"

    def conv(x, c_in, c_out, k, pad):
        wname, bname = fresh("filters"), fresh("bias")
        init[wname] = (rng.standard_normal((c_out, c_in, k, k)) * np.sqrt(2.0 / (k * k * c_in))).astype(np.float32)
        init[bname] = (rng.standard_normal(c_out) * 0.1).astype(np.float32)
        planar, convolved, out = fresh("planar"), fresh("convolved"), fresh("value")
        nodes.append(Node("Transpose", [x], [planar], {"perm": _TO_NCHW}))
        nodes.append(Node("Conv", [planar, wname, bname], [convolved],
                          {"kernel_shape": (k, k), "strides": (1, 1), "pads": (pad,) * 4, "dilations": (1, 1), "group": 1}))
        nodes.append(Node("Transpose", [convolved], [out], {"perm": _TO_NHWC}))
        return out

    def relu(x):
        out = fresh("value")
        nodes.append(Node("Relu", [x], [out]))
        return out

    def add_relu(a, b):
        s = fresh("sum")
        nodes.append(Node("Add", [a, b], [s]))
        return relu(s)

    def pool(x, kind):
        planar, pooled, out = fresh("planar"), fresh("pooled"), fresh("value")
        nodes.append(Node("Transpose", [x], [planar], {"perm": _TO_NCHW}))
        nodes.append(Node(kind, [planar], [pooled], {"kernel_shape": (2, 2), "strides": (2, 2), "pads": (0, 0, 0, 0)}))
        nodes.append(Node("Transpose", [pooled], [out], {"perm": _TO_NHWC}))
        return out

    def residual(x, c):          # second.forwardChain(first, x, x): relu(conv_b(relu(conv_a(x))) + x)
        return add_relu(conv(relu(conv(x, c, c, 3, 1)), c, c, 3, 1), x)

    def down(x, c_in, c_out):    # b.forwardChain(a, x, skip(x))
        return add_relu(conv(relu(conv(x, c_in, c_out, 3, 1)), c_out, c_out, 3, 1), conv(x, c_in, c_out, 1, 0))

    image = fresh("image")
    nodes.append(Node("Reshape", ["input"], [image], {"shape": (0, 32, 32, 3)}))
    x = relu(conv(image, 3, w1, 3, 1))
    x = pool(residual(residual(x, w1), w1), "MaxPool")
    x = pool(residual(down(x, w1, w2), w2), "MaxPool")
    x = pool(residual(down(x, w2, w3), w3), "MaxPool")
    x = pool(pool(x, "AveragePool"), "AveragePool")
    flat = fresh("flat")
    nodes.append(Node("Reshape", [x], [flat], {"shape": (0, w3)}))
    init["fc_weight"] = (rng.standard_normal((w3, classes)) * np.sqrt(2.0 / w3)).astype(np.float32)
    init["fc_bias"] = np.zeros(classes, np.float32)
    product = fresh("product")
    nodes.append(Node("MatMul", [flat, "fc_weight"], [product]))
    nodes.append(Node("Add", [product, "fc_bias"], ["logits"]))
    return Model(nodes, init, ["input"], ["logits"])
