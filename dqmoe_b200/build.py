"""Build recipe of the native library: nvcc, sm_100a only, in-tree output.

`python -m dqmoe_b200.build` compiles dqmoe_b200/csrc/*.cu into
dqmoe_b200/libdqmoe_b200.so (a plain C-ABI shared library with no torch or
Python dependency; the CUDA runtime is linked statically). nvcc cross-compiles,
so no GPU is needed to build.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libdqmoe_b200.so")

SOURCES = ["common.cu", "route.cu", "permute.cu", "quant.cu", "quant_mx.cu", "gemm_sm100.cu", "gemm_mx_sm100.cu", "layer.cu",
           "ep.cu", "decode.cu", "plugin.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the dqmoe_b200 native library cannot be built")
    return nvcc


def _digest(paths) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(PKG_DIR), "include", "dqmoe.h"))
    return hs


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if its sources changed; return the path of the .so."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    stamp_path = os.path.join(OBJ_DIR, "stamp.txt")
    all_src = [os.path.join(CSRC, s) for s in SOURCES]
    digest = _digest(all_src + headers)
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == digest:
                return LIB_PATH

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose and res.stderr:
            sys.stderr.write(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(all_src))) as pool:
        objs = list(pool.map(compile_one, all_src))

    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs,
            "-Xcompiler", "-fPIC"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp_path, "w") as f:
        f.write(digest)
    return LIB_PATH


EXT_DIR = os.path.join(PKG_DIR, "dropin_ext")
EXT_SRC = os.path.join(CSRC, "moe_test_pybind.cpp")


def build_extension(force: bool = False) -> str:
    """Compile the pybind11 `moe_test` extension module (csrc/moe_test_pybind.cpp) into
    dqmoe_b200/dropin_ext/, linked against libdqmoe_b200.so next door and against torch (host code only: g++,
    no nvcc). Put dqmoe_b200/dropin_ext on sys.path to import it; dqmoe_b200/dropin holds the ctypes
    module of the same name for setups without a C++ compiler."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    build()
    os.makedirs(EXT_DIR, exist_ok=True)
    out = os.path.join(EXT_DIR, "moe_test" + sysconfig.get_config_var("EXT_SUFFIX"))
    stamp_path = os.path.join(OBJ_DIR, "ext_stamp.txt")
    h = hashlib.sha256()
    for p in (EXT_SRC, os.path.join(os.path.dirname(PKG_DIR), "include", "dqmoe.h")):
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(torch.__version__.encode())
    digest = h.hexdigest()
    if not force and os.path.exists(out) and os.path.exists(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == digest:
                return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=moe_test",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(cuda_home, "include")]
    cmd += ["-I" + p for p in ce.include_paths()]
    cmd += [EXT_SRC, "-o", out, "-L" + PKG_DIR, "-l:libdqmoe_b200.so", "-Wl,-rpath,$ORIGIN/.."]
    for lp in ce.library_paths():
        cmd += ["-L" + lp, "-Wl,-rpath," + lp]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the moe_test extension failed:\n{res.stdout[-3000:]}\n{res.stderr[-3000:]}")
    with open(stamp_path, "w") as f:
        f.write(digest)
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    if "--ext" in sys.argv:
        print(build_extension(force="--force" in sys.argv))
