"""Generates tests/golden/ops_golden.npz: seeded inputs' expected outputs computed by an
implementation that is independent of the oracle -- torch.nn.functional on CPU in float64.

Run from the repository root:  python tests/golden/make_golden.py
The cases mirror the benchmark configurations at sizes that keep the file small; for the
two larger ones (the single-conv configuration and ResNet-50 logits) only the logits /
a strided sample of the output are stored.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from occamy_b200 import graphs  # noqa: E402


def t64(a):
    return torch.from_numpy(np.asarray(a)).double()


def run_graph_torch(g, x):
    vals = {0: t64(x)}
    for k, v in g.consts.items():
        vals[k] = t64(v)
    for n in g.nodes:
        a = n.attrs
        i = [vals[v] if v != -1 else None for v in n.ins]
        if n.op == "conv":
            r = F.conv2d(i[0], i[1], i[2], a["strides"], a["pads"], 1, a["groups"])
        elif n.op == "relu":
            r = F.relu(i[0])
        elif n.op == "clip":
            r = torch.clamp(i[0], a["lo"], a["hi"])
        elif n.op == "add":
            r = i[0] + i[1]
        elif n.op == "maxpool":
            r = F.max_pool2d(i[0], a["kernel"], a["strides"], a["pads"])
        elif n.op == "avgpool":
            r = F.avg_pool2d(i[0], a["kernel"], a["strides"], a["pads"], count_include_pad=True)
        elif n.op == "gap":
            r = i[0].mean((2, 3), keepdim=True)
        elif n.op == "flatten":
            r = i[0].flatten(1)
        elif n.op == "gemm":
            r = i[0] @ (i[1].T if a["transB"] else i[1])
            if i[2] is not None:
                r = r + i[2]
        elif n.op == "softmax":
            r = F.softmax(i[0], a["axis"])
        vals[n.out] = r
    return [vals[v].numpy() for v in g.outputs]


def main():
    out = {}
    # the single-conv benchmark configuration: strided sample of the 64x56x56 output
    g = graphs.single_conv(seed=0)
    x = graphs.make_input(g, 0, "uniform")
    (y,) = run_graph_torch(g, x)
    out["c1_sample"] = y[:, ::4, ::7, ::7].astype(np.float64)
    out["c1_sum"] = np.array([y.sum(), np.abs(y).sum()])
    # ResNet-50 v1 / v1.5, batch 2: logits
    for variant in ("v1", "v1.5"):
        g = graphs.resnet50(batch=2, seed=0, variant=variant, softmax=False)
        x = graphs.make_input(g, 0)
        (y,) = run_graph_torch(g, x)
        out[f"resnet50_{variant}_b2_logits"] = y
    g = graphs.mobilenet_v2(batch=2, seed=0, image=96)
    (y,) = run_graph_torch(g, graphs.make_input(g, 0))
    out["mobilenet_v2_b2_i96_logits"] = y
    g = graphs.vgg16(batch=2, seed=0, image=64, num_classes=100)
    (y,) = run_graph_torch(g, graphs.make_input(g, 0))
    out["vgg16_b2_i64_logits"] = y
    # small single-operator cases, full outputs
    r = np.random.Generator(np.random.PCG64(42))
    x = r.uniform(-1, 1, (2, 6, 9, 8)).astype(np.float32)
    w = r.normal(0, 0.3, (4, 3, 3, 3)).astype(np.float32)
    b = r.normal(0, 0.1, 4).astype(np.float32)
    out["op_conv_g2_s2_p1"] = F.conv2d(t64(x), t64(w), t64(b), 2, 1, 1, 2).numpy()
    out["op_maxpool_3s2p1"] = F.max_pool2d(t64(x), 3, 2, 1).numpy()
    out["op_avgpool_3s2p1_incl"] = F.avg_pool2d(t64(x), 3, 2, 1, count_include_pad=True).numpy()
    out["op_softmax_axis1"] = F.softmax(t64(x), 1).numpy()
    out["op_x"], out["op_w"], out["op_b"] = x, w, b
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ops_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
