"""Build recipe: nvcc for sm_100a only. Produces, inside this directory,
libtffn.so (the C-ABI library of include/tffn.h) and tensor-ffn-inference (the command line).
The built files stay in-tree (git-ignored) so they travel with the source snapshot.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtffn.so")
CLI = os.path.join(HERE, "tensor-ffn-inference")
LIB_SOURCES = ["host_io.cpp", "c_api.cpp", "tp_comm.cpp", "engine.cu", "gemm_tc.cu", "rows.cu", "attn.cu", "decode_bs1.cu", "noalloc.cu"]
CLI_SOURCES = ["cli_main.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr"]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs += [os.path.join(HERE, "..", "include", f) for f in ("tffn.h", "tffn_diag.h")]
    return hs


def _compile(src: str, verbose: bool, extra: list[str]) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if _newer(obj, [path] + _headers()):
        cmd = ["nvcc"] + NVCC_FLAGS + extra + ["-x", "cu", "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return obj


def build(verbose: bool = False, ptxas_verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_verbose else []
    lib_sources = [s for s in LIB_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with ThreadPoolExecutor(8) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, extra), lib_sources))
        cli_objs = list(ex.map(lambda s: _compile(s, verbose, extra), CLI_SOURCES))
    if _newer(LIB, objs):
        subprocess.check_call(["nvcc", "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"])
    if _newer(CLI, cli_objs + [LIB]):
        subprocess.check_call(["nvcc", "-o", CLI] + cli_objs + ["-L" + HERE, "-ltffn", "-Xlinker", "-rpath,$ORIGIN",
                                                              "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, ptxas_verbose="--ptxas" in sys.argv))
