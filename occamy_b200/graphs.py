"""The benchmark graphs as the Occamy compiler sees them after ONNX import: batch-norm
folded into the convolution bias, dropout removed, global average pooling as a mean
reduction.  Weights are seeded synthetic tensors (He-normal filters, N(0, 0.01) biases,
drawn in layer order, weight then bias) -- no pretrained checkpoint is involved.

A ``Graph`` is a plain list of nodes so that the same description can be (a) handed to
the native program builder (``to_program``) and (b) interpreted by any other
implementation of the operators.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Node:
    op: str
    out: int
    ins: tuple
    attrs: dict = field(default_factory=dict)


class Graph:
    def __init__(self, input_shape, seed=0):
        self.input_shape = tuple(int(v) for v in input_shape)
        self.nodes = []
        self.consts = {}      # value id -> ndarray
        self.shapes = {0: self.input_shape}
        self.nvals = 1        # value 0 is the input
        self.outputs = []
        self.rng = np.random.Generator(np.random.PCG64(seed))
        self.name = "graph"

    # ---- values ----
    def const(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        v = self._new(a.shape)
        self.consts[v] = a
        return v

    def _new(self, shape):
        v = self.nvals
        self.nvals += 1
        self.shapes[v] = tuple(int(s) for s in shape)
        return v

    def he_conv(self, K, C, R, S, bias=True):
        fan_in = C * R * S
        w = self.rng.normal(0.0, np.sqrt(2.0 / fan_in), (K, C, R, S)).astype(np.float32)
        b = self.rng.normal(0.0, 0.01, (K,)).astype(np.float32) if bias else None
        return w, b

    # ---- operators ----
    def conv(self, x, w, b=None, groups=1, pads=(0, 0), strides=(1, 1)):
        wv = self.const(w)
        bv = self.const(b) if b is not None else -1
        N, C, H, W = self.shapes[x]
        K, _, R, S = w.shape
        P = (H + 2 * pads[0] - R) // strides[0] + 1
        Q = (W + 2 * pads[1] - S) // strides[1] + 1
        out = self._new((N, K, P, Q))
        self.nodes.append(Node("conv", out, (x, wv, bv),
                               dict(groups=groups, pads=tuple(pads), strides=tuple(strides))))
        return out

    def _unary(self, op, x, **attrs):
        out = self._new(self.shapes[x])
        self.nodes.append(Node(op, out, (x,), attrs))
        return out

    def relu(self, x):
        return self._unary("relu", x)

    def clip(self, x, lo, hi):
        return self._unary("clip", x, lo=float(lo), hi=float(hi))

    def softmax(self, x, axis=1):
        return self._unary("softmax", x, axis=axis)

    def add(self, a, b):
        out = self._new(self.shapes[a])
        self.nodes.append(Node("add", out, (a, b)))
        return out

    def _pool(self, op, x, kernel, pads, strides):
        N, C, H, W = self.shapes[x]
        P = (H + 2 * pads[0] - kernel[0]) // strides[0] + 1
        Q = (W + 2 * pads[1] - kernel[1]) // strides[1] + 1
        out = self._new((N, C, P, Q))
        self.nodes.append(Node(op, out, (x,), dict(kernel=tuple(kernel), pads=tuple(pads),
                                                    strides=tuple(strides))))
        return out

    def maxpool(self, x, kernel, pads=(0, 0), strides=(1, 1)):
        return self._pool("maxpool", x, kernel, pads, strides)

    def avgpool(self, x, kernel, pads=(0, 0), strides=(1, 1)):
        return self._pool("avgpool", x, kernel, pads, strides)

    def gap(self, x):
        N, C, _, _ = self.shapes[x]
        out = self._new((N, C, 1, 1))
        self.nodes.append(Node("gap", out, (x,)))
        return out

    def flatten(self, x):
        s = self.shapes[x]
        out = self._new((s[0], int(np.prod(s[1:]))))
        self.nodes.append(Node("flatten", out, (x,)))
        return out

    def gemm(self, a, w, b=None, transB=1):
        """Y = A * W^T + b with W stored [out, in] (torch.nn.Linear as exported to ONNX)."""
        wv = self.const(w)
        bv = self.const(b) if b is not None else -1
        M = self.shapes[a][0]
        Nn = w.shape[0] if transB else w.shape[1]
        out = self._new((M, Nn))
        self.nodes.append(Node("gemm", out, (a, wv, bv), dict(transB=transB)))
        return out

    def linear(self, a, n_in, n_out):
        w = self.rng.normal(0.0, np.sqrt(2.0 / n_in), (n_out, n_in)).astype(np.float32)
        b = self.rng.normal(0.0, 0.01, (n_out,)).astype(np.float32)
        return self.gemm(a, w, b)

    def mark_output(self, v):
        self.outputs.append(v)

    # ---- algorithmic work (for roofline figures) ----
    def conv_flops(self):
        total = 0
        for n in self.nodes:
            if n.op == "conv":
                N, K, P, Q = self.shapes[n.out]
                _, Cg, R, S = self.shapes[n.ins[1]]
                total += 2 * N * K * P * Q * Cg * R * S
            elif n.op == "gemm":
                M, Nn = self.shapes[n.out]
                total += 2 * M * Nn * self.shapes[n.ins[0]][1]
        return total

    # ---- hand-off to the native builder ----
    def to_program(self):
        from .replay import Program
        p = Program()
        ids = {0: p.input(self.input_shape)}

        def get(v):
            if v == -1:
                return -1
            if v not in ids:
                ids[v] = p.const(self.consts[v])
            return ids[v]

        for n in self.nodes:
            a = n.attrs
            if n.op == "conv":
                r = p.conv(get(n.ins[0]), get(n.ins[1]), get(n.ins[2]), a["groups"], a["pads"],
                           a["strides"])
            elif n.op == "relu":
                r = p.relu(get(n.ins[0]))
            elif n.op == "clip":
                r = p.clip(get(n.ins[0]), a["lo"], a["hi"])
            elif n.op == "add":
                r = p.add(get(n.ins[0]), get(n.ins[1]))
            elif n.op == "maxpool":
                r = p.maxpool(get(n.ins[0]), a["kernel"], a["pads"], a["strides"])
            elif n.op == "avgpool":
                r = p.avgpool(get(n.ins[0]), a["kernel"], a["pads"], a["strides"])
            elif n.op == "gap":
                r = p.gap(get(n.ins[0]))
            elif n.op == "flatten":
                r = p.flatten(get(n.ins[0]))
            elif n.op == "gemm":
                r = p.gemm(get(n.ins[0]), get(n.ins[1]), get(n.ins[2]), 1.0, 1.0, 0, a["transB"])
            elif n.op == "softmax":
                r = p.softmax(get(n.ins[0]), a["axis"])
            else:
                raise ValueError(n.op)
            ids[n.out] = r
            assert p.shape(r) == self.shapes[n.out], (n.op, p.shape(r), self.shapes[n.out])
        for v in self.outputs:
            p.mark_output(ids[v])
        p.graph = self
        return p


# ---------------------------------------------------------------------------------
def single_conv(seed=0, N=1, C=64, H=56, W=56, K=64, R=3, pad=1, stride=1, relu=True):
    """One Conv + bias (+ ReLU): x ~ U(-1, 1), He-normal filter, N(0, 0.01) bias."""
    g = Graph((N, C, H, W), seed)
    g.name = "single_conv"
    w, b = g.he_conv(K, C, R, R)
    y = g.conv(0, w, b, pads=(pad, pad), strides=(stride, stride))
    if relu:
        y = g.relu(y)
    g.mark_output(y)
    return g


def make_input(g: Graph, seed=0, dist="normal"):
    rng = np.random.Generator(np.random.PCG64(seed + 1000003))
    if dist == "uniform":
        return rng.uniform(-1.0, 1.0, g.input_shape).astype(np.float32)
    return rng.standard_normal(g.input_shape, dtype=np.float32)


def resnet50(batch=1, seed=0, variant="v1", softmax=True, num_classes=1000, image=224):
    """ResNet-50: 7x7/2 stem, 3x3/2 max pool, bottlenecks 3-4-6-3, global average pool,
    2048 x num_classes Gemm, softmax.  variant "v1": the stride sits on the first 1x1 of a
    down-sampling block; "v1.5": on its 3x3 (torchvision's)."""
    g = Graph((batch, 3, image, image), seed)
    g.name = f"resnet50_{variant}"
    w, b = g.he_conv(64, 3, 7, 7)
    x = g.relu(g.conv(0, w, b, pads=(3, 3), strides=(2, 2)))
    x = g.maxpool(x, (3, 3), (1, 1), (2, 2))
    cin = 64
    for mid, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for i in range(blocks):
            s = stride if i == 0 else 1
            s1, s3 = (s, 1) if variant == "v1" else (1, s)
            w1, b1 = g.he_conv(mid, cin, 1, 1)
            y = g.relu(g.conv(x, w1, b1, strides=(s1, s1)))
            w2, b2 = g.he_conv(mid, mid, 3, 3)
            y = g.relu(g.conv(y, w2, b2, pads=(1, 1), strides=(s3, s3)))
            w3, b3 = g.he_conv(mid * 4, mid, 1, 1)
            y = g.conv(y, w3, b3)
            if i == 0:
                wd, bd = g.he_conv(mid * 4, cin, 1, 1)
                sc = g.conv(x, wd, bd, strides=(s, s))
            else:
                sc = x
            x = g.relu(g.add(y, sc))
            cin = mid * 4
    x = g.flatten(g.gap(x))
    x = g.linear(x, 2048, num_classes)
    g.logits = x
    if softmax:
        x = g.softmax(x, 1)
    g.mark_output(x)
    return g


def mobilenet_v2(batch=1, seed=0, num_classes=1000, image=224):
    """MobileNetV2, width 1.0: inverted residuals (1x1 expand t=6, 3x3 depthwise, 1x1
    project), ReLU6 as Clip(0, 6)."""
    g = Graph((batch, 3, image, image), seed)
    g.name = "mobilenet_v2"
    w, b = g.he_conv(32, 3, 3, 3)
    x = g.clip(g.conv(0, w, b, pads=(1, 1), strides=(2, 2)), 0.0, 6.0)
    cin = 32
    for t, c, n, s in ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1),
                       (6, 160, 3, 2), (6, 320, 1, 1)):
        for i in range(n):
            stride = s if i == 0 else 1
            hidden = cin * t
            y = x
            if t != 1:
                we, be = g.he_conv(hidden, cin, 1, 1)
                y = g.clip(g.conv(y, we, be), 0.0, 6.0)
            wd, bd = g.he_conv(hidden, 1, 3, 3)
            y = g.clip(g.conv(y, wd, bd, groups=hidden, pads=(1, 1), strides=(stride, stride)),
                       0.0, 6.0)
            wp, bp = g.he_conv(c, hidden, 1, 1)
            y = g.conv(y, wp, bp)
            x = g.add(x, y) if (stride == 1 and cin == c) else y
            cin = c
    wl, bl = g.he_conv(1280, cin, 1, 1)
    x = g.clip(g.conv(x, wl, bl), 0.0, 6.0)
    x = g.flatten(g.gap(x))
    x = g.linear(x, 1280, num_classes)
    g.logits = x
    g.mark_output(x)
    return g


def vgg16(batch=1, seed=0, num_classes=1000, image=224):
    """VGG-16: 13 3x3 convolutions, five 2x2/2 max pools, 1x1 average pool (the adaptive
    pool of a 224 input), FC 25088-4096-4096-num_classes."""
    g = Graph((batch, 3, image, image), seed)
    g.name = "vgg16"
    x, cin = 0, 3
    for v in (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512,
              "M"):
        if v == "M":
            x = g.maxpool(x, (2, 2), (0, 0), (2, 2))
        else:
            w, b = g.he_conv(v, cin, 3, 3)
            x = g.relu(g.conv(x, w, b, pads=(1, 1)))
            cin = v
    x = g.avgpool(x, (1, 1), (0, 0), (1, 1))
    x = g.flatten(x)
    feat = g.shapes[x][1]
    x = g.relu(g.linear(x, feat, 4096))
    x = g.relu(g.linear(x, 4096, 4096))
    x = g.linear(x, 4096, num_classes)
    g.logits = x
    g.mark_output(x)
    return g
