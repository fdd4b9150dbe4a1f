#!/usr/bin/env python
"""Headline benchmark: images/s of ResNet-50 (v1, BN folded) batch-256 inference through the
Occamy runtime C ABI on B200, batch-sharded over N GPUs, logits gathered with NCCL.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the CPU restatement on the host cores

One step = one inference of the whole batch: the replayed call sequence a compiled model
would issue (pool init, mem-offsets, constant uploads, 53 fused conv calls, adds, pools,
Gemm, softmax).  `value` times it with the input batch resident in HBM (device->device
copy into the pool, logits left on the device); `e2e` times the same calls with the batch
in pinned host memory and the logits read back to the host.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

GLOBAL_BATCH = 256


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, power, reasons = [], [], [], set()
        for line in self.tmp.read().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.tmp.name)
        if sm:
            # median over the samples taken under load (upper half of the power readings)
            cut = statistics.median(power)
            loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
            out.update(sm_mhz=statistics.median(loaded), sm_max_mhz=max(mx),
                       reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_baseline_sample(batch: int, repeats: int, graph: str = "resnet50"):
    """Times the CPU restatement (oracle port) of the same graph on the host cores."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import run_graph_oracle
    from occamy_b200 import graphs
    g = getattr(graphs, graph)(batch=batch, seed=0)
    x = graphs.make_input(g, 0)
    run_graph_oracle(g, x)  # warm-up (page in the library, OpenMP pool)
    t0 = time.perf_counter()
    for _ in range(repeats):
        run_graph_oracle(g, x)
    dt = (time.perf_counter() - t0) / repeats
    return batch / dt, dt


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path.  Its own onnx-mlir
    CPU build cannot be produced offline, so this is the C restatement (oracle port), all
    host threads, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_batch = 2
    cores = os.cpu_count() or 1
    metric = GRAPH_DEFAULTS[args.graph][1]
    for _ in range(max(args.warmup, 1)):
        cpu_baseline_sample(sample_batch, 1, args.graph)
    times = []
    for _ in range(args.steps):
        _, dt = cpu_baseline_sample(sample_batch, 1, args.graph)
        times.append(dt)
    ms = 1000.0 * sum(times) / len(times)
    value = sample_batch / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args.graph, args.batch, int(os.environ.get("WORLD_SIZE", "1")),
                                  args.fuse),
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_batch} images per step of the batch-{args.batch} "
                                   "workload, fp32 C restatement with OpenMP"},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_incumbent_arm(args):
    """--impl incumbent (not part of the driver's contract): the reference's own GPU runtime
    -- its cuDNN / cuBLASLt wrappers compiled unchanged into oracle/_ref -- replaying the same
    call program on this GPU, host batch in, host logits out, wall-clock timed (its work runs
    on the legacy default stream and every inference ends in a blocking copy)."""
    import torch
    from occamy_b200 import graphs, replay
    from oracle import build as obuild
    if not os.path.exists(obuild.REF_SO):
        print(json.dumps({"impl": "incumbent", "unavailable": "oracle/_ref not built"}))
        return
    torch.cuda.set_device(0)
    g = getattr(graphs, args.graph)(batch=args.batch, seed=0)
    prog = g.to_program()
    prog.lower(fuse=args.fuse, workspace_bytes=256 << 20)
    binding = replay.Binding(obuild.REF_SO)
    x = torch.from_numpy(graphs.make_input(g, 0)).pin_memory()
    out = torch.empty(g.shapes[g.outputs[0]], dtype=torch.float32).pin_memory()
    for _ in range(max(args.warmup, 1)):
        prog.run_raw(binding, x.data_ptr(), 1, [out.data_ptr()], 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        prog.run_raw(binding, x.data_ptr(), 1, [out.data_ptr()], 1)
    torch.cuda.synchronize()
    ms = 1000.0 * (time.perf_counter() - t0) / args.steps
    print(json.dumps({"impl": "incumbent", "metric": GRAPH_DEFAULTS[args.graph][1],
                      "value": args.batch / (ms / 1000.0),
                      "unit": "images/s", "n_gpus": 1, "steps": args.steps, "ms_per_step": ms,
                      "dtype": "f32 (cuDNN default math)", "data": "synthetic",
                      "config": {"workload": f"{g.name} batch {args.batch}, reference wrappers "
                                             f"(cuDNN {torch.backends.cudnn.version()}), "
                                             f"fuse={args.fuse}, weights re-uploaded every "
                                             "inference as the compiled model does"}}), flush=True)


# graph -> (global batch of the configuration, metric name, arithmetic mode of the headline run)
GRAPH_DEFAULTS = {
    "resnet50": (256, "images/sec ResNet-50 b=256", "bf16"),
    "mobilenet_v2": (128, "images/sec MobileNetV2 b=128", "fp16"),
    "vgg16": (64, "images/sec VGG-16 b=64", "bf16"),
}
PARITY_TOL = {"fp32": 1e-4, "bf16": 2e-2, "fp16": 2e-2}
GRAPH_NAMES = {"resnet50": "resnet50_v1", "mobilenet_v2": "mobilenet_v2", "vgg16": "vgg16"}


def workload_config(graph, batch, world, fuse):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": f"{GRAPH_NAMES[graph]} inference, global batch {batch} "
                        f"({batch // world} per GPU), N(0,1) images, He-normal weights, "
                        f"replayed fused call sequence (fuse={fuse})",
            "global_batch": batch, "parallelism": f"dp{world}",
            "l2": "per-step working set (activations > 1 GB) exceeds the 126 MB L2"}


def torch_cpu_baseline(graph_name, batch, threads, seconds=4.0):
    """Independent CPU number: the same graph evaluated by PyTorch's CPU kernels (oneDNN) with
    `threads` threads; images/s over about `seconds` of work."""
    import torch
    import torch.nn.functional as F
    from occamy_b200 import graphs
    g = getattr(graphs, graph_name)(batch=batch, seed=0)
    x = torch.from_numpy(graphs.make_input(g, 0))
    consts = {k: torch.from_numpy(v) for k, v in g.consts.items()}
    old = torch.get_num_threads()
    torch.set_num_threads(threads)

    def run():
        vals = {0: x}
        vals.update(consts)
        for n in g.nodes:
            a, i = n.attrs, [vals[v] if v != -1 else None for v in n.ins]
            if n.op == "conv":
                r = F.conv2d(i[0], i[1], i[2], a["strides"], a["pads"], 1, a["groups"])
            elif n.op == "relu":
                r = F.relu(i[0])
            elif n.op == "clip":
                r = i[0].clamp(a["lo"], a["hi"])
            elif n.op == "add":
                r = i[0] + i[1]
            elif n.op == "maxpool":
                r = F.max_pool2d(i[0], a["kernel"], a["strides"], a["pads"])
            elif n.op == "avgpool":
                r = F.avg_pool2d(i[0], a["kernel"], a["strides"], a["pads"])
            elif n.op == "gap":
                r = i[0].mean((2, 3), keepdim=True)
            elif n.op == "flatten":
                r = i[0].flatten(1)
            elif n.op == "gemm":
                r = F.linear(i[0], i[1], i[2])
            elif n.op == "softmax":
                r = F.softmax(i[0], a["axis"])
            else:
                raise ValueError(n.op)
            vals[n.out] = r
        return vals[g.outputs[0]]

    with torch.no_grad():
        run()
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < seconds:
            run()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
    torch.set_num_threads(old)
    return batch / dt


def incumbent_line(graph, batch, fuse, steps):
    """The reference's own GPU runtime on this box, in a child process (it brings its own cuDNN
    and cuBLASLt); None when oracle/_ref was not built."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "incumbent",
                            "--graph", graph, "--batch", str(batch), "--fuse", str(fuse),
                            "--steps", str(steps), "--warmup", "1"], capture_output=True, text=True,
                           timeout=600)
        for ln in reversed(r.stdout.splitlines()):
            if ln.startswith("{"):
                d = json.loads(ln)
                return None if "unavailable" in d else d
    except Exception:
        pass
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "incumbent"])
    ap.add_argument("--graph", default="resnet50", choices=sorted(GRAPH_DEFAULTS))
    ap.add_argument("--batch", type=int, default=0, help="global batch (default: the graph's configuration)")
    ap.add_argument("--math", default="", choices=["", "bf16", "fp16", "fp32"])
    ap.add_argument("--fuse", type=int, default=1)
    ap.add_argument("--warm-seconds", type=float, default=2.0,
                    help="keep running warm-up steps until this much time has passed, so that the "
                         "timed steps see the clocks and power state of a loaded GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the incumbent, PyTorch-CPU and memory-bound-kernel legs")
    ap.add_argument("--per-layer", default="", help="write a per-launch roofline table here")
    args = ap.parse_args()
    cfg_batch, metric, cfg_math = GRAPH_DEFAULTS[args.graph]
    if not args.batch:
        args.batch = cfg_batch
    if not args.math:
        args.math = cfg_math
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.impl == "incumbent":
        run_incumbent_arm(args)
        return

    import torch
    import torch.distributed as dist
    from occamy_b200 import graphs, replay, sharding
    from occamy_b200 import runtime as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: no CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import datetime
        # a collective that some rank never joins ends in an error after two minutes, not in a
        # kernel that spins until the job is killed
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=120))
    lo_img, hi_img = sharding.shard_range(args.batch, rank, world)
    per_rank = hi_img - lo_img

    math_mode = {"bf16": rt.MATH_BF16, "fp16": rt.MATH_F16, "fp32": rt.MATH_FP32}[args.math]
    rt.set_math_mode(math_mode)
    builder = getattr(graphs, args.graph)
    g = builder(batch=per_rank, seed=0)
    prog = g.to_program()
    prog.lower(fuse=args.fuse, dealloc_opt=True, pool_opt=True)
    binding = replay.Binding()
    stream = torch.cuda.ExternalStream(rt.lib().occamy_stream())

    # rank r owns images [r*B/R, (r+1)*B/R) of the seeded global batch
    full = graphs.make_input(builder(batch=1, seed=0), 0).shape[1:]

    def rank_images(r, count):
        rg = np.random.Generator(np.random.PCG64(1000003 + r))
        return rg.standard_normal((per_rank,) + tuple(full), dtype=np.float32)[:count]

    x_host = torch.from_numpy(rank_images(rank, per_rank)).pin_memory()
    x_dev = x_host.cuda(non_blocking=False)
    n_out = g.shapes[g.outputs[0]][1]
    out_dev = torch.empty((per_rank, n_out), dtype=torch.float32, device="cuda")
    gathered = torch.empty((args.batch, n_out), dtype=torch.float32, device="cuda")
    out_host = torch.empty((args.batch, n_out), dtype=torch.float32).pin_memory()
    import ctypes as C

    def step_resident():
        prog.run_raw(binding, x_dev.data_ptr(), 3, [out_dev.data_ptr()], 3)
        if world > 1:
            with torch.cuda.stream(stream):
                sharding.gather_logits(out_dev, gathered)

    def step_e2e():
        """What a compiled model does per inference: host batch in through wrapDNNMemcpy kind 1,
        result back through the blocking kind 2 copy; the call returns when the result is in host
        memory (ONNXToDNNCommon.cpp:129-183).  With several ranks the gather sits between the
        model's device result and the one copy to rank 0's host buffer, and the host waits for
        it before the next step, just the same."""
        if world == 1:
            prog.run_raw(binding, x_host.data_ptr(), 1, [out_host.data_ptr()], 1)
            return
        prog.run_raw(binding, x_host.data_ptr(), 1, [out_dev.data_ptr()], 3)
        with torch.cuda.stream(stream):
            src = sharding.gather_logits(out_dev, gathered)
            if rank == 0:
                out_host.copy_(src, non_blocking=True)
        stream.synchronize()

    def step_e2e_pipelined():
        """The same copies without the host wait: a server that keeps several inferences in
        flight overlaps step i+1's upload with step i's kernels."""
        prog.run_raw(binding, x_host.data_ptr(), 1, [out_dev.data_ptr()], 3)
        with torch.cuda.stream(stream):
            src = sharding.gather_logits(out_dev, gathered) if world > 1 else out_dev
            if rank == 0:
                out_host[: src.shape[0]].copy_(src, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
        for _ in range(steps):
            fn()
        with torch.cuda.stream(stream):
            e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- warm-up: at least W steps (the first packs and caches the weights), then more until
    # the GPU has been under load for --warm-seconds; the clock sampler covers all of it ----
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step_resident()
    torch.cuda.synchronize()
    if rt.last_error():
        raise SystemExit("runtime reported an error during warm-up")
    # the same K steps on the GPU as the W warm-up steps leave it (cool, boost clocks): reported
    # beside `value`, which is taken after the GPU has been under load for --warm-seconds
    ms_burst = timed(step_resident, args.steps)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_end = time.perf_counter() + args.warm_seconds
    more = 0
    while True:
        go = torch.tensor([1.0 if time.perf_counter() < t_end else 0.0], device="cuda")
        if world > 1:
            dist.all_reduce(go, op=dist.ReduceOp.MIN)     # every rank runs the same number
        if go.item() < 0.5:
            break
        for _ in range(10):
            step_resident()
        torch.cuda.synchronize()
        more += 10
    warm += more

    c0 = rt.counters()
    if rank == 0:   # for profilers: which launch the timed region starts at
        print(f"[bench] kernel launches before the timed region: {c0['launches']}", file=sys.stderr,
              flush=True)
    ms_total = timed(step_resident, args.steps)
    c1 = rt.counters()
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    for _ in range(3):
        step_e2e_pipelined()
    ms_pipe = timed(step_e2e_pipelined, args.steps)

    # ---- dominant kernel: CUDA-event pair around every tensor-core launch ----
    rt.lib().occamy_profile_begin()
    prof_steps = 5
    for _ in range(prof_steps):
        step_resident()
    buf = (C.c_float * 8192)()
    n_prof = rt.lib().occamy_profile_end(buf, 8192)
    clocks = sampler.stop() if sampler else None
    per_step = n_prof // prof_steps if prof_steps else 0
    tc_ms = [[buf[s * per_step + i] for s in range(prof_steps)] for i in range(per_step)]
    tc_ms = [statistics.median(v) for v in tc_ms]
    tc_total_ms = sum(tc_ms)
    err = rt.last_error()
    if err:
        raise SystemExit(f"runtime reported error {err}")

    # ---- parity of what was timed: the logits of a few images against the CPU oracle ----
    # Every rank replays the same program once more with the pre-softmax tensor marked as an
    # output as well (identical kernels up to the softmax) and the ranks' logits are gathered
    # like the result is; rank 0 then compares rows of its own and of the last rank's shard.
    g2 = builder(batch=per_rank, seed=0)
    logits_all = None
    if getattr(g2, "logits", None) is not None:
        if g2.logits not in g2.outputs:
            g2.mark_output(g2.logits)
        p2 = g2.to_program()
        p2.lower(fuse=args.fuse, dealloc_opt=True, pool_opt=True)
        outs2 = [torch.empty(g2.shapes[v], dtype=torch.float32, device="cuda") for v in g2.outputs]
        p2.run_raw(binding, x_host.data_ptr(), 1, [t.data_ptr() for t in outs2], 3)
        logits_dev = outs2[g2.outputs.index(g2.logits)]
        with torch.cuda.stream(stream):
            logits_all = sharding.gather_logits(logits_dev) if world > 1 else logits_dev
        stream.synchronize()
    parity = None
    if rank == 0:
        parity = check_parity(args, builder, out_host, logits_all.cpu().numpy() if logits_all is not None
                              else None, world, per_rank, rank_images, x_host)

    ms_step = ms_total / args.steps
    value = args.batch / (ms_step / 1000.0)
    peaks = measured_peaks()
    flops = g.conv_flops()            # algorithmic conv + Gemm FLOPs of this rank's batch
    achieved = flops / (tc_total_ms / 1000.0) / 1e12 if tc_total_ms > 0 else 0.0
    # The denominator is the burst figure: each launch is timed alone between two events.
    peak = peaks["bf16_tflops"]

    if args.per_layer and rank == 0:
        write_per_layer(args.per_layer, g, tc_ms, peaks, ms_step)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    def per_s(ms):
        return args.batch / (ms / args.steps / 1000.0)

    line = {
        "metric": metric, "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": {"bf16": "bf16", "fp16": "f16", "fp32": "f32"}[args.math], "data": "synthetic",
        "config": workload_config(args.graph, args.batch, world, args.fuse),
        "warm_seconds": args.warm_seconds,
        "burst": {"value": per_s(ms_burst), "unit": "images/s", "ms_per_step": ms_burst / args.steps,
                  "how": "the same K steps right after the W warm-up steps, before the GPU has "
                         "been loaded for warm_seconds"},
        "e2e": {"value": per_s(ms_e2e), "unit": "images/s",
                "h2d_bytes_per_step": int(x_host.numel() * 4 * world),
                "d2h_bytes_per_step": int(args.batch * n_out * 4),
                "how": "host batch in (wrapDNNMemcpy kind 1), blocking copy of the result to the "
                       "host (kind 2) every inference: the reference's own call sequence"},
        "e2e_pipelined": {"value": per_s(ms_pipe), "unit": "images/s",
                          "how": "same copies, no host wait between inferences"},
        "gpu_launches": int(c1["launches"] - c0["launches"]),
        "clocks": clocks,
        "parity_checked": parity,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak else None,
                     "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
                     "traffic": profiled_traffic(per_rank, args.graph) if world == 1 else None,
                     "traffic_note": "DRAM read+write bytes of the tensor-core launches of one "
                                     "step (ncu, profiles/tc_conv_traffic_resnet50_b256.txt)",
                     "kernel": "tc_conv_kernel (+ tc_conv_pn_kernel, stem_pool_kernel)",
                     "launches_per_step": per_step,
                     "kernel_ms_per_step": tc_total_ms,
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16: launches are timed "
                                                      "one by one)"},
    }
    if clocks and clocks.get("sm_mhz"):
        line["ms_per_step_x_sm_mhz"] = ms_step * clocks["sm_mhz"]
    if world == 1 and not args.no_extras:
        from occamy_b200 import opbench
        rows, hbm, hbm_src = opbench.run(batch=args.batch, reps=10, math=rt.MATH_BF16)
        line["roofline"]["membound"] = [
            {"op": r[0], "ms": round(r[2], 4), "gbs": round(r[3], 1), "frac": round(r[4], 3)}
            for r in rows]
        line["roofline"]["membound_peak"] = {"gbs": hbm, "source": hbm_src + " copy bandwidth"}
        rt.set_math_mode(math_mode)
        inc = {}
        for fuse in (1, 0):
            d = incumbent_line(args.graph, args.batch, fuse, 5)
            if d:
                inc["fused" if fuse else "unfused"] = {"value": d["value"], "unit": "images/s",
                                                        "ms_per_step": d["ms_per_step"]}
        if inc:
            inc["what"] = ("the reference's own cuDNN / cuBLASLt wrappers compiled unchanged, same "
                           "call program, same GPU, host batch in and host result out")
            line["incumbent"] = inc
    if not args.no_cpu_baseline and world == 1:
        cores = os.cpu_count() or 1
        sample = 16
        v, dt = cpu_baseline_sample(sample, 3, args.graph)
        line["cpu_baseline"] = {"value": v, "unit": "images/s", "cores": cores, "kind": "port",
                                "sample": f"{sample} images (of the batch-{args.batch} workload), fp32 C "
                                          f"restatement with OpenMP, {dt:.2f} s per pass"}
        if not args.no_extras:
            line["cpu_baseline_torch"] = {
                "unit": "images/s", "what": "PyTorch CPU (oneDNN), same graph and weights",
                "all_threads": {"value": torch_cpu_baseline(args.graph, 16, cores), "threads": cores},
                "four_threads": {"value": torch_cpu_baseline(args.graph, 8, 4), "threads": 4,
                                 "why": "the thread count of the reference's own timing script "
                                        "(test/models/resnet50/run.py:83)"}}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def check_parity(args, builder, out_host, logits_all, world, per_rank, rank_images, x_host):
    """Runs the CPU oracle on four images of the batch that was timed and compares (a) the
    timed program's own output, as the last end-to-end step left it in rank 0's host buffer, and
    (b) the logits of the same images (`logits_all`, gathered over the ranks).  With several
    ranks two of the images belong to the last rank, so the gathered tensors are what is
    checked.  No step is run here: with several ranks a step is a collective, and only rank 0
    comes this way."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import max_rel_err, run_graph_oracle, top1_agrees
    picks = [(0, 0), (0, per_rank // 3), (world - 1, 2 * per_rank // 3), (world - 1, per_rank - 1)]
    imgs = []
    cache = {0: x_host.numpy()}
    for r, i in picks:
        if r not in cache:
            cache[r] = rank_images(r, per_rank)
        imgs.append(cache[r][i])
    rows = [r * per_rank + i for r, i in picks]
    gs = builder(batch=len(picks), seed=0)
    outs, vals = run_graph_oracle(gs, np.stack(imgs), keep=True)
    want_out, want_logits = outs[0], vals[gs.logits]
    got_out = out_host.numpy()[rows]
    res = {"images": len(picks), "rows": rows, "tolerance": PARITY_TOL[args.math],
           "output_max_abs_err": float(np.abs(got_out - want_out).max()),
           # identical top-1, except rows whose two largest reference values are closer than
           # one bf16 step of their magnitude (see tests/helpers.py::top1_agrees)
           "top1_equal": top1_agrees(got_out, want_out)[0]}
    if logits_all is not None:
        got_logits = logits_all[rows]
        res["max_rel"] = max_rel_err(got_logits, want_logits)
        ok, ties = top1_agrees(got_logits, want_logits)
        res["top1_equal"] = res["top1_equal"] and ok
        res["near_ties_left_out"] = ties
    else:
        res["max_rel"] = max_rel_err(got_out, want_out)
    res["ok"] = bool(res["max_rel"] <= PARITY_TOL[args.math] and res["top1_equal"])
    if not res["ok"]:
        print(f"[bench] PARITY FAILED: {res}", file=sys.stderr, flush=True)
    return res


def profiled_traffic(batch, graph):
    """DRAM bytes per step of the dominant kernel, from the committed ncu summary of this
    workload (profiles/); None when the run is a different workload."""
    path = os.path.join(ROOT, "profiles", "tc_conv_traffic_resnet50_b256.txt")
    if graph != "resnet50" or batch != GLOBAL_BATCH or not os.path.exists(path):
        return None
    for line in open(path):
        if line.startswith("dram_bytes_per_step:"):
            return float(line.split(":")[1])
    return None


def write_per_layer(path, g, tc_ms, peaks, ms_step):
    """Per-launch table: algorithmic FLOPs and bytes (bf16 activations, bf16 weights) of each
    convolution / Gemm, its CUDA-event time, and the fraction of max(tensor, HBM) roofline."""
    rows = []
    idx = 0
    for n in g.nodes:
        if n.op not in ("conv", "gemm"):
            continue
        if n.op == "conv":
            N, K, P, Q = g.shapes[n.out]
            _, Cg, R, S = g.shapes[n.ins[1]]
            if n.attrs["groups"] != 1:
                continue
            flops = 2 * N * K * P * Q * Cg * R * S
            _, _, H, W = g.shapes[n.ins[0]]
            st = n.attrs["strides"]
            # input pixels the convolution actually touches (a strided 1x1 skips most)
            hh = min(H, P * R if R < st[0] else (P - 1) * st[0] + R)
            ww = min(W, Q * S if S < st[1] else (Q - 1) * st[1] + S)
            xin = N * Cg * hh * ww
            out_elems = N * K * P * Q
            name = f"conv {Cg}->{K} {R}x{S} s{n.attrs['strides'][0]} out {P}x{Q}"
            extra = 0
            # what the fused call sequence folds into this launch: a residual operand read,
            # or (stem) the max pool, which shrinks the tensor that is written
            cur = n.out
            for m in g.nodes:
                if cur not in m.ins:
                    continue
                if m.op == "relu":
                    cur = m.out
                elif m.op == "add":
                    # the add folds into the convolution right before it; the other branch's
                    # convolution only produces the operand
                    between = g.nodes[g.nodes.index(n) + 1:g.nodes.index(m)]
                    if any(b.op == "conv" for b in between):
                        break
                    extra += 2 * out_elems
                    cur = m.out
                elif m.op == "maxpool" and Cg < 16:
                    out_elems = int(np.prod(g.shapes[m.out]))
                    xin = N * 4 * H * (W + 8)          # padded channels-last rows, 4 channels
                    name += " +pool"
                    break
                else:
                    break
            byts = 2 * xin + 2 * K * Cg * R * S + 4 * K + 2 * out_elems + extra
        else:
            M, Nn = g.shapes[n.out]
            Kd = g.shapes[n.ins[0]][1]
            flops = 2 * M * Nn * Kd
            byts = 4 * M * Kd + 2 * Nn * Kd + 4 * M * Nn
            name = f"gemm {M}x{Kd}x{Nn}"
        if idx >= len(tc_ms):
            break
        ms = tc_ms[idx]
        idx += 1
        t_tensor = flops / (peaks["bf16_tflops"] * 1e12) * 1e3   # burst: launches are timed alone
        t_hbm = byts / (peaks["hbm_gbs"] * 1e9) * 1e3
        bound = max(t_tensor, t_hbm)
        rows.append((name, flops / 1e9, byts / 1e6, ms, flops / ms / 1e9 if ms else 0,
                     byts / ms / 1e6 if ms else 0, "tensor" if t_tensor >= t_hbm else "hbm",
                     bound / ms if ms else 0))
    with open(path, "w") as f:
        f.write(f"# {g.name}: per tensor-core launch, ms_per_step {ms_step:.3f}; peaks: "
                f"{peaks['bf16_tflops']:.1f} TFLOP/s (burst cuBLAS bf16) and {peaks['hbm_gbs']:.1f} GB/s "
                f"({peaks['source']}); frac = max(tensor time, HBM time) / measured time\n")
        f.write("# layer | GFLOP | MB (bf16 activations, incl. residual operand) | ms | TFLOP/s | GB/s | "
                "bound | frac of roofline\n")
        for r in rows:
            f.write(f"{r[0]:40s} {r[1]:9.2f} {r[2]:9.2f} {r[3]:8.4f} {r[4]:8.1f} {r[5]:8.1f} "
                    f"{r[6]:7s} {r[7]:6.3f}\n")
        f.write(f"# total kernel ms {sum(r[3] for r in rows):.3f}\n")


if __name__ == "__main__":
    main()
