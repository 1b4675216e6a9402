"""CPU walk of an in-memory ONNX graph with the oracle's kernels: the stand-in for grad's `Model.run`
(src/onnx/runtime.zig:560-620) on the node kinds its exporter writes for a ResNet.  TEST INFRASTRUCTURE ONLY.

Transpose-Conv-Transpose windows use `convolveNhwc` (runtime.zig:868-899, the path `Model.run` fuses to,
:256-279); pooling follows src/gpu/math/conv.zig:152-205 (window clipped to the image, average over the
in-bounds count); MatMul is `matmul` (:621-646); Add / Relu / Reshape are element-wise in f32.
"""
from __future__ import annotations

import numpy as np

from . import binding as orc


def _pool(x, k, stride, pad, is_max):
    n, h, w, c = x.shape
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    out = np.empty((n, oh, ow, c), np.float32)
    for oy in range(oh):
        y0, y1 = max(oy * stride - pad, 0), min(oy * stride + k - pad, h)
        for ox in range(ow):
            x0, x1 = max(ox * stride - pad, 0), min(ox * stride + k - pad, w)
            win = x[:, y0:y1, x0:x1, :]
            out[:, oy, ox, :] = win.max(axis=(1, 2)) if is_max else win.sum(axis=(1, 2), dtype=np.float32) / np.float32((y1 - y0) * (x1 - x0))
    return out


def run(model, feeds, threads=None):
    threads = threads or orc.host_threads()
    values = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in feeds.items()}

    def get(name):
        return values[name] if name in values else model.initializers[name]

    nodes = model.nodes
    at = 0
    while at < len(nodes):
        node = nodes[at]
        window = None
        if node.op == "Transpose" and tuple(node.attrs["perm"]) == (0, 3, 1, 2) and at + 2 < len(nodes):
            mid, last = nodes[at + 1], nodes[at + 2]
            if mid.op in ("Conv", "MaxPool", "AveragePool") and last.op == "Transpose" and tuple(last.attrs["perm"]) == (0, 2, 3, 1):
                window = (mid, last)
        if window is not None:
            mid, last = window
            x = get(node.inputs[0])
            if mid.op == "Conv":
                w = model.initializers[mid.inputs[1]]
                bias = model.initializers[mid.inputs[2]] if len(mid.inputs) > 2 else None
                n, h, width, c = x.shape
                d = orc.ConvDims(n=n, h=h, w=width, c=c, k=w.shape[2], stride=int(mid.attrs["strides"][0]), pad=int(mid.attrs["pads"][0]),
                                 dilation=int(mid.attrs["dilations"][0]), c_out=w.shape[0])
                values[last.outputs[0]] = orc.convolve_nhwc(x, w, bias, d, threads)
            else:
                values[last.outputs[0]] = _pool(x, int(mid.attrs["kernel_shape"][0]), int(mid.attrs["strides"][0]), int(mid.attrs["pads"][0]),
                                                mid.op == "MaxPool")
            at += 3
            continue
        if node.op == "Relu":
            values[node.outputs[0]] = orc.relu(get(node.inputs[0]))
        elif node.op == "Add":
            values[node.outputs[0]] = (get(node.inputs[0]) + get(node.inputs[1])).astype(np.float32)
        elif node.op == "Reshape":
            x = get(node.inputs[0])
            shape = tuple(x.shape[i] if v == 0 else v for i, v in enumerate(node.attrs["shape"]))
            values[node.outputs[0]] = x.reshape(shape)
        elif node.op == "MatMul":
            values[node.outputs[0]] = orc.onnx_matmul(get(node.inputs[0]), get(node.inputs[1]), threads)
        elif node.op == "Gemm":    # runtime.zig:648-664
            c = get(node.inputs[2]) if len(node.inputs) > 2 and node.inputs[2] else None
            row_bias = c is not None and c.size == np.asarray(c).shape[-1]       # broadcast over the rows
            beta = float(node.attrs.get("beta", 1.0))
            out = orc.onnx_gemm(get(node.inputs[0]), get(node.inputs[1]), np.asarray(c).reshape(-1) if row_bias else None,
                                bool(node.attrs.get("transA", 0)), bool(node.attrs.get("transB", 0)), float(node.attrs.get("alpha", 1.0)), beta, threads)
            if c is not None and not row_bias:                                    # C of the result's shape
                out = (out + np.float32(beta) * np.asarray(c, np.float32)).astype(np.float32)
            values[node.outputs[0]] = out
        else:
            raise NotImplementedError(node.op)
        at += 1
    return {name: values[name] for name in model.outputs}
