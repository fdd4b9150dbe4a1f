"""Timing of the memory-bound operator kernels through the C ABI.

    python -m occamy_b200.opbench [--batch 256] [--reps 20] [--only pool] [--out table.txt]

Every row calls one ABI symbol (pooling, element-wise add / ReLU / Clip, depthwise convolution,
global average pool, softmax) on device-resident tensors of the sizes ResNet-50 and MobileNetV2
produce at the given batch, in bf16 mode with the input already in the runtime's bf16 NHWC
format (it is the output of a convolution call, as in a model).  Times are CUDA-event medians on
the runtime's stream; between repetitions the tensors (hundreds of MB) do not fit the L2.
"achieved" is algorithmic bytes / time, "frac" its share of the measured copy bandwidth in
MEASURED_PEAKS.json (fallback 6650 GB/s).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics

import numpy as np

from . import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _hbm_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class _T:
    def __init__(self, shape, data=None):
        self.shape = tuple(int(s) for s in shape)
        n = int(np.prod(self.shape))
        if data is not None:
            self.buf = rt.DeviceBuffer.from_numpy(np.ascontiguousarray(data, np.float32))
        else:
            self.buf = rt.DeviceBuffer(max(n, 1) * 4)
        self.ptr = self.buf.ptr


def _bf16_tensor(h, rng, N, Cc, H, W):
    """A [N,Cc,H,W] tensor in the runtime's bf16 NHWC format: the output of a 1x1 convolution."""
    cin = 16
    x = _T((N, cin, H, W), rng.standard_normal((N, cin, H, W), dtype=np.float32))
    w = _T((Cc, cin, 1, 1), rng.standard_normal((Cc, cin, 1, 1), dtype=np.float32) * 0.25)
    y = _T((N, Cc, H, W))
    rt.lib().DNNConvFunc(h, x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), None, 0, 1, 1,
                         rt.dims((0, 0)), rt.dims((1, 1)), y.ptr)
    rt.lib().occamy_synchronize()
    x.buf.free()
    return y


def run(batch=256, reps=20, only="", math=rt.MATH_BF16, role_timers=False):
    """Times the rows whose name contains one of the comma-separated pieces of `only` (all rows
    when empty); returns [(name, algorithmic MB, ms, GB/s, fraction of the copy bandwidth)] and
    the peak used."""
    import torch

    class _Args:
        pass
    args = _Args()
    args.batch, args.reps, args.only = batch, reps, only
    wanted = [t for t in only.split(",") if t]
    torch.cuda.init()
    rt.set_math_mode(math)
    L = rt.lib()
    h = C.c_void_p()
    L.cudnnCreate(C.byref(h))
    stream = torch.cuda.ExternalStream(L.occamy_stream())
    rng = np.random.Generator(np.random.PCG64(0))
    peak, peak_src = _hbm_peak()
    B = args.batch
    rows = []
    # Analysis builds of the library (-DOCCAMY_TC_TIMERS) count, for CTA 0 of every tensor-core
    # convolution launch, the cycles each role spends in its barrier waits and in total.
    timers = None
    if role_timers:
        raw = C.CDLL(rt.LIB_PATH)
        if not hasattr(raw, "occamy_tc_timers"):
            raise SystemExit("--role-timers needs a library built with OCCAMY_NVCC_EXTRA=-DOCCAMY_TC_TIMERS")
        raw.occamy_tc_timers.argtypes = [C.POINTER(C.c_longlong), C.c_int]
        tbuf = (C.c_longlong * 20)()
        timers = lambda: (raw.occamy_tc_timers(tbuf, 1), list(tbuf))[1]
    ROLES = (("loads", ("ring slot free",)), ("MMA issue", ("accumulator free", "operands landed")),
             ("epilogue 0", ("accumulator full", "slab buffer ready")),
             ("epilogue 1", ("accumulator full", "slab buffer ready")),
             ("slab store 0", ("slab written", "earlier store read out")))

    def timed(name, nbytes, fn):
        if wanted and not any(t in name for t in wanted):
            return
        if timers:
            timers()
        for _ in range(3):
            fn()
        ms = []
        inner = 4   # calls per event pair: the launch latency of an idle stream is paid once, not per call
        for _ in range(args.reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(inner):
                fn()
            e1.record(stream)
            e1.synchronize()
            ms.append(e0.elapsed_time(e1) / inner)
        t = statistics.median(ms)
        gbs = nbytes / t / 1e6
        rows.append((name, nbytes / 1e6, t, gbs, gbs / peak))
        if timers:
            v = timers()
            for i, (role, kinds) in enumerate(ROLES):
                total = v[4 * i + 3]
                if total:
                    waits = ", ".join(f"{k} {v[4 * i + j] / total:.2f}" for j, k in enumerate(kinds))
                    print(f"#   {name}: {role:12s} share of its time waiting for: {waits}")
        err = rt.last_error()
        if err:
            raise SystemExit(f"{name}: runtime error {err}")

    def pool(x, k, pad, st, avg):
        N, Cc, H, W = x.shape
        P = (H + 2 * pad - k) // st + 1
        y = _T((N, Cc, P, P))
        fn = L.DNNAveragePoolFunc if avg else L.DNNMaxPoolFunc
        call = lambda: fn(h, x.ptr, rt.dims(x.shape), y.ptr, rt.dims(y.shape), rt.dims((k, k)),
                          rt.dims((pad, pad, pad, pad)), rt.dims((st, st)))
        return call, 2 * (int(np.prod(x.shape)) + int(np.prod(y.shape))), y

    def depthwise(x, st):
        N, Cc, H, W = x.shape
        P = (H + 2 - 3) // st + 1
        w = _T((Cc, 1, 3, 3), rng.standard_normal((Cc, 1, 3, 3), dtype=np.float32) * 0.3)
        y = _T((N, Cc, P, P))
        call = lambda: L.DNNConvFunc(h, x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), None, 0, 1, Cc,
                                     rt.dims((1, 1)), rt.dims((st, st)), y.ptr)
        return call, 2 * (int(np.prod(x.shape)) + int(np.prod(y.shape))) + 36 * Cc, (w, y)

    def sel(*pieces):   # does the selection keep any row whose name holds one of these?
        return not wanted or any(any(t in pc or pc in t for pc in pieces) for t in wanted)

    # ---- ResNet-50 sized tensors ----
    if sel("max pool"):
        x = _bf16_tensor(h, rng, B, 64, 112, 112)
        call, nb, keep = pool(x, 3, 1, 2, False)
        timed(f"max pool 3x3/2 [{B},64,112,112]", nb, call)
        del keep
        x.buf.free()

    if not sel("add", "ReLU", "Clip", "average pool 2x2"):
        a = None
    else:
        a = _bf16_tensor(h, rng, B, 256, 56, 56)
    if a is not None:
        a, b, out, n = _elementwise_rows(a, h, rng, B, L, timed, pool)
        for t in (a, b, out):
            t.buf.free()
    if sel("global average pool"):
        g = _bf16_tensor(h, rng, B, 2048, 7, 7)
        gy = _T((B, 2048, 1, 1))
        timed(f"global average pool [{B},2048,7,7]", 2 * int(np.prod(g.shape)) + 4 * B * 2048,
              lambda: L.DNNReduceFunc(h, 4, g.ptr, rt.dims(g.shape), gy.ptr, rt.dims(gy.shape), 5))
        g.buf.free()
    _rest(h, rng, B, L, timed, depthwise, sel)
    if any("conv" in t for t in wanted):
        _conv_rows(h, rng, B, L, timed, wanted)
    L.cudnnDestroy(h)
    return rows, peak, peak_src


def _elementwise_rows(a, h, rng, B, L, timed, pool):
    b = _bf16_tensor(h, rng, B, 256, 56, 56)
    out = _T(a.shape)
    n = int(np.prod(a.shape))
    timed(f"add [{B},256,56,56]", 6 * n,
          lambda: L.DNNTensorOpFunc(h, 0, a.ptr, rt.dims(a.shape), 4, b.ptr, rt.dims(b.shape), 4, out.ptr,
                                    rt.dims(a.shape), 4, 1.0))
    timed(f"ReLU [{B},256,56,56]", 4 * n,
          lambda: L.DNNActiveFunc(h, a.ptr, rt.dims(a.shape), 1, out.ptr))
    timed(f"Clip(0,6) [{B},256,56,56]", 4 * n,
          lambda: L.CUDAClipFunc(a.ptr, out.ptr, rt.dims(a.shape), 0.0, 6.0, 4))
    call, nb, keep = pool(a, 2, 0, 2, True)
    timed(f"average pool 2x2/2 [{B},256,56,56]", nb, call)
    del keep
    return a, b, out, n


# (name, C, K, R, H, stride, residual): tensor-core convolution layers of ResNet-50; timed only when
# named in `only` (they are the per-layer rows of bench.py's --per-layer table, one at a time)
CONV_ROWS = [("conv3x3 256->256 @14", 256, 256, 3, 14, 1, False),
             ("conv3x3 512->512 @7", 512, 512, 3, 7, 1, False),
             ("conv3x3 128->128 @28", 128, 128, 3, 28, 1, False),
             ("conv3x3 64->64 @56", 64, 64, 3, 56, 1, False),
             ("conv1x1 1024->256 @14", 1024, 256, 1, 14, 1, False),
             ("conv1x1 2048->512 @7", 2048, 512, 1, 7, 1, False),
             ("conv1x1 256->1024 @14 +res", 256, 1024, 1, 14, 1, True),
             ("conv1x1 512->2048 @7 +res", 512, 2048, 1, 7, 1, True),
             ("conv1x1 64->256 @56 +res", 64, 256, 1, 56, 1, True),
             ("conv1x1 512->128 @28", 512, 128, 1, 28, 1, False),
             # MobileNetV2's few-channel layers on large images
             ("conv1x1 32->16 @112", 32, 16, 1, 112, 1, False),
             ("conv1x1 16->96 @112", 16, 96, 1, 112, 1, False),
             ("conv1x1 144->24 @56", 144, 24, 1, 56, 1, False),
             # short reductions into few channels: two CTAs share an SM
             ("conv1x1 64->64 @56", 64, 64, 1, 56, 1, False),
             ("conv1x1 256->64 @56", 256, 64, 1, 56, 1, False),
             ("conv1x1 256->128 /2 @56", 256, 128, 1, 56, 2, False),
             ("conv1x1 96->24 @56", 96, 24, 1, 56, 1, False),
             ("conv1x1 192->32 @28", 192, 32, 1, 28, 1, False),
             ("conv1x1 384->64 @14", 384, 64, 1, 14, 1, False),
             ("conv1x1 576->96 @14", 576, 96, 1, 14, 1, False),
             ("conv1x1 24->144 @56", 24, 144, 1, 56, 1, False)]


def _conv_rows(h, rng, B, L, timed, wanted):
    """Fused convolution (+ bias + ReLU, + residual add through the call sequence a model
    issues) on device-resident 16-bit tensors; algorithmic bytes as in the per-layer table."""
    for name, Cc, K, R, H, st, res in CONV_ROWS:
        if not any(t in name for t in wanted):
            continue
        x = _bf16_tensor(h, rng, B, Cc, H, H)
        w = _T((K, Cc, R, R), rng.standard_normal((K, Cc, R, R), dtype=np.float32) * (2.0 / (Cc * R * R)) ** 0.5)
        b = _T((K,), rng.standard_normal((K,), dtype=np.float32) * 0.01)
        P = (H + 2 * (R // 2) - R) // st + 1
        y = _T((B, K, P, P))
        pads, strides = rt.dims((R // 2, R // 2)), rt.dims((st, st))
        nbytes = 2 * (B * Cc * H * H + K * Cc * R * R + B * K * P * P) + 4 * K
        if res:
            r_ = _bf16_tensor(h, rng, B, K, P, P)
            out = _T((B, K, P, P))
            nbytes += 2 * B * K * P * P

            def call():   # conv (identity) -> add residual -> ReLU: folds into one launch once seen
                hh = C.c_void_p()
                L.cudnnCreate(C.byref(hh))
                L.DNNConvBiasActivFunc(hh, x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), b.ptr,
                                       rt.dims((1, K, 1, 1)), None, 0, 1, pads, strides, 5, y.ptr)
                L.DNNTensorOpFunc(hh, 0, y.ptr, rt.dims(y.shape), 4, r_.ptr, rt.dims(y.shape), 4,
                                  out.ptr, rt.dims(y.shape), 4, 1.0)
                L.DNNActiveFunc(hh, out.ptr, rt.dims(y.shape), 1, out.ptr)
                L.cudnnDestroy(hh)
        else:
            def call():
                L.DNNConvBiasActivFunc(h, x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), b.ptr,
                                       rt.dims((1, K, 1, 1)), None, 0, 1, pads, strides, 1, y.ptr)
        flops = 2.0 * B * K * P * P * Cc * R * R
        timed(f"{name} [{B}] ({flops / 1e9:.1f} GFLOP)", nbytes, call)
        for t in (x, w, b, y):
            t.buf.free()


def _rest(h, rng, B, L, timed, depthwise, sel):
    # ---- MobileNetV2 sized depthwise convolutions ----
    if sel("depthwise"):
        for (Cc, H, st) in ((32, 112, 1), (96, 112, 2), (144, 56, 1), (192, 28, 2), (384, 14, 1),
                            (960, 7, 1)):
            x = _bf16_tensor(h, rng, B, Cc, H, H)
            call, nb, keep = depthwise(x, st)
            timed(f"depthwise 3x3/{st} [{B},{Cc},{H},{H}]", nb, call)
            del keep
            x.buf.free()
    if sel("softmax"):
        s = _T((B, 1000), rng.standard_normal((B, 1000), dtype=np.float32))
        sy = _T((B, 1000))
        timed(f"softmax [{B},1000] fp32", 8 * B * 1000,
              lambda: L.CUDASoftmaxFunc(s.ptr, rt.dims(s.shape), sy.ptr, rt.dims(s.shape), 1, 2))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--only", default="", help="run only the rows whose name contains one of "
                                               "these comma-separated pieces of text")
    ap.add_argument("--math", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--role-timers", action="store_true",
                    help="print the per-role wait shares of the tensor-core convolution kernel "
                         "(needs a library built with OCCAMY_NVCC_EXTRA=-DOCCAMY_TC_TIMERS)")
    args = ap.parse_args()
    B = args.batch
    rows, peak, peak_src = run(B, args.reps, args.only,
                               rt.MATH_BF16 if args.math == "bf16" else rt.MATH_F16, args.role_timers)
    lines = [f"# memory-bound operator kernels through the C ABI, batch {B}, {args.math} mode; "
             f"peak = {peak:.0f} GB/s ({peak_src} copy bandwidth)",
             "# op | MB (algorithmic) | ms | GB/s | frac of peak"]
    for r in rows:
        lines.append(f"{r[0]:44s} {r[1]:9.1f} {r[2]:8.4f} {r[3]:8.1f} {r[4]:6.3f}")
    text = "\n".join(lines)
    print(text)
    if args.out:
        open(args.out, "w").write(text + "\n")


if __name__ == "__main__":
    main()
