"""In-tree build of the native libraries (nvcc, sm_100a only).

Produces, under ``occamy_b200/lib/``:
  liboccamy_dnn.so      the operator runtime behind the reference's C ABI
  libcd_dnn_wrapper.a   the same objects under the archive name the Occamy compiler
                        links (``-lcd_dnn_wrapper``)
  liboccamy_replay.so   host-side program builder / pool planner / replayer
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(LIB, "obj")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

RUNTIME_SRCS = ["runtime.cu", "kernels_f32.cu", "kernels_nhwc.cu", "conv_tc.cu", "conv_tc_inst_256_64.cu",
                "conv_tc_inst_256_32.cu", "conv_tc_inst_128_64.cu", "conv_tc_inst_64_64.cu",
                "conv_tc_inst_32_32.cu", "stem_pool.cu", "trace.cu", "abi.cu", "misc_ops.cu", "no_alloc.cu"]
REPLAY_SRCS = [os.path.join("host", "replay.cpp")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-I", CSRC, "-I", INCLUDE]
NVCC_FLAGS += os.environ.get("OCCAMY_NVCC_EXTRA", "").split()   # e.g. -DOCCAMY_TUNING (sweep hooks)

RUNTIME_SO = os.path.join(LIB, "liboccamy_dnn.so")
RUNTIME_A = os.path.join(LIB, "libcd_dnn_wrapper.a")
REPLAY_SO = os.path.join(LIB, "liboccamy_replay.so")


def _deps_mtime() -> float:
    t = os.path.getmtime(__file__)
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".h", ".hpp", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    for f in os.listdir(INCLUDE):
        t = max(t, os.path.getmtime(os.path.join(INCLUDE, f)))
    return t


def _compile(src: str, hdr_t: float, verbose: bool, ptxas_v: bool) -> str:
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ, src.replace(os.sep, "_") + ".o")
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_t):
        return obj
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", path, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if ptxas_v:
        print(r.stderr)
    return obj


def build(verbose: bool = False, ptxas_v: bool = False) -> dict:
    os.makedirs(OBJ, exist_ok=True)
    hdr_t = _deps_mtime()
    srcs = list(RUNTIME_SRCS)
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr_t, verbose, ptxas_v), srcs))
        robjs = list(ex.map(lambda s: _compile(s, hdr_t, verbose, False), REPLAY_SRCS))

    def stale(target, deps):
        return not os.path.exists(target) or any(os.path.getmtime(d) > os.path.getmtime(target) for d in deps)

    if stale(RUNTIME_SO, objs):
        subprocess.run(["nvcc", "-shared", "-o", RUNTIME_SO] + objs + ["-lcudart"], check=True)
    if stale(RUNTIME_A, objs):
        if os.path.exists(RUNTIME_A):
            os.remove(RUNTIME_A)
        subprocess.run(["ar", "rcs", RUNTIME_A] + objs, check=True)
    if stale(REPLAY_SO, robjs):
        subprocess.run(["g++", "-shared", "-o", REPLAY_SO] + robjs + ["-ldl"], check=True)
    return {"runtime": RUNTIME_SO, "archive": RUNTIME_A, "replay": REPLAY_SO}


if __name__ == "__main__":
    print(build(verbose=True, ptxas_v="--ptxas" in sys.argv))
