"""The drop-in boundary without a GPU: the shared library loads, and it and the static
archive export every symbol the public header declares."""
import os
import re
import subprocess

from occamy_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "occamy_dnn_api.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_reference_symbol_set():
    syms = declared_symbols()
    # 44 Occamy symbols + cudnnCreate / cudnnDestroy (cudaStreamCreate/Destroy stay in
    # libcudart) + this library's own controls
    for name in ("DNNConvFunc", "DNNConvBiasActivFunc", "DNNTensorOpFunc", "DNNActiveFunc",
                 "DNNMaxPoolFunc", "DNNAveragePoolFunc", "DNNReduceFunc", "CUBLASMatmul2dFunc",
                 "CUDASoftmaxFunc", "CUDAClipFunc", "CUDAFlattenFunc", "CUDAReshapeFunc",
                 "wrapDNNMalloc", "wrapDNNMemPoolInit", "wrapDNNMemOffset", "wrapDNNMemcpy",
                 "wrapDNNDealloc", "cudnnCreate", "cudnnDestroy", "CUDAMatmulNdFunc",
                 "CUDATranspose6DInt64Func", "CUDACastI64toFloatFunc"):
        assert name in syms
    occamy = [s for s in syms if not s.startswith("occamy_") and not s.startswith("cudnn")]
    assert len(occamy) == 44


def test_shared_library_loads_and_exports_every_declared_symbol(native_libs):
    lib = rt.load_library(native_libs["runtime"])       # dlopen only; no GPU call
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert set(declared_symbols()) <= set(rt.abi_symbols()) | {"cudnnCreate", "cudnnDestroy"}


def test_static_archive_has_the_compilers_link_name(native_libs):
    path = native_libs["archive"]
    assert os.path.basename(path) == "libcd_dnn_wrapper.a"
    out = subprocess.run(["nm", "-g", "--defined-only", path], capture_output=True, text=True,
                         check=True).stdout
    defined = set(line.split()[-1] for line in out.splitlines() if " T " in line)
    for name in declared_symbols():
        assert name in defined, name


def test_missing_library_fails_loudly(tmp_path):
    import pytest
    with pytest.raises(RuntimeError, match="no Python/CPU fallback"):
        rt.load_library(str(tmp_path / "liboccamy_dnn.so"))
