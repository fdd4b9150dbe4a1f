"""Test-side helpers: the oracle interpreter of a Graph and the parity metrics.

Only tests import this module (it pulls in the CPU oracle)."""
import numpy as np

from oracle import ref


def run_graph_oracle(g, x, f64_conv=False, keep=False):
    """Evaluate a occamy_b200.graphs.Graph with the CPU oracle; returns the outputs (and
    every intermediate value when keep=True)."""
    vals = {0: np.ascontiguousarray(x, np.float32)}
    vals.update(g.consts)
    last_use = {}
    for i, n in enumerate(g.nodes):
        for v in n.ins:
            last_use[v] = i
    for i, n in enumerate(g.nodes):
        a = n.attrs
        ins = [vals[v] if v != -1 else None for v in n.ins]
        if n.op == "conv":
            r = ref.conv2d(ins[0], ins[1], ins[2], a["pads"], a["strides"], a["groups"], act=5,
                           f64=f64_conv)
        elif n.op == "relu":
            r = ref.activation(ins[0], 1)
        elif n.op == "clip":
            r = ref.clip(ins[0], a["lo"], a["hi"])
        elif n.op == "add":
            r = ref.tensor_op(0, ins[0], ins[1])
        elif n.op == "maxpool":
            r = ref.pool2d(ins[0], a["kernel"], a["pads"], a["strides"], avg=False)
        elif n.op == "avgpool":
            r = ref.pool2d(ins[0], a["kernel"], a["pads"], a["strides"], avg=True)
        elif n.op == "gap":
            s = ins[0].shape
            r = ref.reduce_mean(ins[0], (s[0], s[1], 1, 1))
        elif n.op == "flatten":
            r = ins[0].reshape(ins[0].shape[0], -1).copy()
        elif n.op == "gemm":
            r = ref.matmul2d(ins[0], ins[1], transB=a["transB"])
            if ins[2] is not None:
                r = ref.tensor_op(0, r, ins[2].reshape(1, -1))
        elif n.op == "softmax":
            r = ref.softmax(ins[0], a["axis"])
        else:
            raise ValueError(n.op)
        vals[n.out] = r
        if not keep:
            for v in n.ins:
                if v > 0 and last_use.get(v) == i and v not in g.outputs and v not in g.consts:
                    vals.pop(v, None)
    outs = [vals[v] for v in g.outputs]
    return (outs, vals) if keep else outs


def max_rel_err(y, ref_y):
    """max |y - ref| / max |ref| over the tensor (the per-tensor relative error)."""
    y = np.asarray(y, np.float64)
    ref_y = np.asarray(ref_y, np.float64)
    denom = max(np.abs(ref_y).max(), 1e-30)
    return float(np.abs(y - ref_y).max() / denom)


def top1_agrees(y, ref_y):
    """Identical top-1 indices, row by row.  A row whose two largest reference logits lie
    closer together than one bf16 step of their own magnitude (2^-8 relative) is undecidable
    for any 16-bit arithmetic -- both round to the same or to neighbouring stored values -- and
    is left out; the second value returned is how many rows that were."""
    y, ref_y = np.asarray(y), np.asarray(ref_y)
    srt = np.sort(ref_y, axis=1)
    tie = (srt[:, -1] - srt[:, -2]) < np.abs(srt[:, -1]) * 2.0 ** -8
    same = y.argmax(1) == ref_y.argmax(1)
    return bool(np.all(same | tie)), int(tie.sum())
