"""Build recipe for the CPU oracle (test infrastructure, never shipped).

``build_oracle()`` compiles ``occamy_oracle.c`` into ``oracle/liboccamy_oracle.so``.
``build_reference_wrappers()`` compiles the reference's own GPU runtime wrappers
(src/Tools/dnn-wrapper of corelab-src/occamy) from where they lie in a reference
checkout into ``oracle/_ref/libcd_dnn_wrapper_ref.so``; it needs the checkout and
the cuDNN / cuBLAS development files of the ``nvidia-*`` pip wheels, and is skipped
when either is absent.  No reference source is copied.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboccamy_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libcd_dnn_wrapper_ref.so")


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "occamy_oracle.c")
    if not force and _newer(ORACLE_SO, [src, __file__]):
        return ORACLE_SO
    # x86-64-v3 (AVX2) rather than -march=native: the .so is built on one host
    # and timed on another.  -ffp-contract=off keeps results bit-reproducible.
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp",
           "-shared", "-fPIC", "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def _wheel_dir(name: str):
    try:
        import importlib
        mod = importlib.import_module(f"nvidia.{name}")
        return list(mod.__path__)[0]
    except Exception:
        return None


def reference_checkout():
    """Where a checkout of corelab-src/occamy lies: the directory named by the environment
    variable OCCAMY_REFERENCE_DIR, else a directory called `reference` beside this repository.
    None when neither holds the wrappers' sources."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("OCCAMY_REFERENCE_DIR"), os.path.join(os.path.dirname(here), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "Tools", "dnn-wrapper")):
            return cand
    return None


def build_reference_wrappers(reference_root: str = None, force: bool = False):
    """Compile the reference runtime (cuDNN/cuBLASLt wrappers) unchanged. Returns
    the .so path, or None with a reason string when it cannot be built."""
    reference_root = reference_root or reference_checkout()
    if not reference_root:
        return None, "reference checkout not present"
    wrap = os.path.join(reference_root, "src", "Tools", "dnn-wrapper")
    if not os.path.isdir(wrap):
        return None, "reference checkout not present"
    cudnn, cublas = _wheel_dir("cudnn"), _wheel_dir("cublas")
    if not cudnn or not cublas:
        return None, "cuDNN/cuBLAS wheels not importable"
    srcs = sorted(glob.glob(os.path.join(wrap, "cudnn", "*.cpp")) +
                  glob.glob(os.path.join(wrap, "cudnn", "fusedOp", "*.cpp")) +
                  glob.glob(os.path.join(wrap, "cublas", "*.cu")) +
                  glob.glob(os.path.join(wrap, "cuda", "*.cu")) +
                  glob.glob(os.path.join(wrap, "cuda", "*.cpp")))
    if not force and _newer(REF_SO, srcs):
        return REF_SO, "up to date"
    os.makedirs(REF_DIR, exist_ok=True)
    cudnn_lib = glob.glob(os.path.join(cudnn, "lib", "libcudnn.so.*"))
    cublas_lib = glob.glob(os.path.join(cublas, "lib", "libcublasLt.so.*"))
    if not cudnn_lib or not cublas_lib:
        return None, "libcudnn / libcublasLt not found in the wheels"
    objdir = os.path.join(REF_DIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    for src in srcs:
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-w",
               "-Xcompiler", "-fPIC,-fpermissive", "-x", "cu",
               "-I", os.path.join(cudnn, "include"), "-I", os.path.join(cublas, "include"),
               "-I", wrap, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True)
        if r.returncode != 0:
            return None, "nvcc failed: " + r.stderr.decode("utf-8", "replace")[-600:]
        objs.append(obj)
    # shared cudart so that cudaStreamCreate & co. resolve through the library, as they do
    # for a compiled model that links -lcudart
    cmd = ["nvcc", "-shared", "-cudart", "shared", "-o", REF_SO] + objs + [
        "-L", os.path.join(cudnn, "lib"), "-L", os.path.join(cublas, "lib"),
        "-l:" + os.path.basename(cudnn_lib[0]), "-l:" + os.path.basename(cublas_lib[0]),
        "-Xlinker", "-rpath," + os.path.join(cudnn, "lib"),
        "-Xlinker", "-rpath," + os.path.join(cublas, "lib"),
        "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True)
    if r.returncode != 0:
        return None, "link failed: " + r.stderr.decode("utf-8", "replace")[-600:]
    return REF_SO, "built"


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference_wrappers(force="--force" in sys.argv))
