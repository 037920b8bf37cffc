"""In-tree build of the native library (`eth_b200/_C*.so`) for sm_100a.

The reference JIT-compiles its four CUDA extensions and the dataset helper at start-up for
sm_70/sm_80 (eth/runtime/megatron/fused_kernels/__init__.py:30-95,
eth/runtime/megatron/data/Makefile). Here everything is compiled ahead of time by plain
`nvcc` / `g++` commands: kernel sources (`csrc/*.cu`) carry no PyTorch headers and build in
seconds; one `bindings.cpp` exposes them to Python through pybind11 + ATen.

Usage: `python -m eth_b200.build_ext [--force] [--verbose]`.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
LIB_NAME = "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")
HELPERS_NAME = "_data_helpers" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"


def _nvcc() -> str:
    return os.path.join(_cuda_home(), "bin", "nvcc")


def _digest(paths, extra="") -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout, r.stderr)
    return r


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA/C++ source for sm_100a and link `eth_b200/_C*.so`. Returns its path."""
    import torch
    from torch.utils import cpp_extension as ce

    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    cu_sources = sorted(CSRC.glob("*.cu"))
    cpp_sources = [CSRC / "bindings.cpp"]
    stamp_file = BUILD / "stamp.json"
    stamps = {}
    if stamp_file.exists() and not force:
        try:
            stamps = json.loads(stamp_file.read_text())
        except Exception:
            stamps = {}
    hdr_digest = _digest(headers, extra=torch.__version__)
    out_lib = PKG / LIB_NAME

    nvcc_flags = ARCH_FLAGS + [
        "-lineinfo", "-O3", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC",
        "--expt-relaxed-constexpr", "-I", str(CSRC), "-DNDEBUG",
    ]
    py_inc = sysconfig.get_paths()["include"]
    torch_inc = ce.include_paths()
    cxx_flags = [
        "-O2", "-std=c++17", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
        "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", str(CSRC), "-I", py_inc,
        "-I", os.path.join(_cuda_home(), "include"),
    ]
    for inc in torch_inc:
        cxx_flags += ["-isystem", inc]

    jobs = []
    objects = []
    for src in cu_sources:
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        d = _digest([src], extra=hdr_digest)
        if stamps.get(src.name) == d and obj.exists():
            continue
        jobs.append((src.name, d, [_nvcc()] + nvcc_flags + ["-c", src, "-o", obj]))
    for src in cpp_sources:
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        d = _digest([src], extra=hdr_digest)
        if stamps.get(src.name) == d and obj.exists():
            continue
        jobs.append((src.name, d, ["g++"] + cxx_flags + ["-c", src, "-o", obj]))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _run(j[2], verbose), jobs))
        for name, d, _ in jobs:
            stamps[name] = d

    if jobs or not out_lib.exists():
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        link = ["g++", "-shared", "-o", out_lib] + objects + [
            "-L", torch_lib, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda",
            "-ltorch_cuda", "-L", os.path.join(_cuda_home(), "lib64"), "-lcudart_static", "-lrt",
            "-lpthread", "-ldl", f"-Wl,-rpath,{torch_lib}",
        ]
        _run(link, verbose)

    # host-only dataset index helpers (no torch dependency)
    helper_src = CSRC / "data_helpers.cpp"
    helper_lib = PKG / HELPERS_NAME
    if helper_src.exists():
        d = _digest([helper_src])
        if stamps.get(helper_src.name) != d or not helper_lib.exists():
            import pybind11
            import numpy  # noqa: F401  (the helper uses pybind11/numpy.h)
            _run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-I", py_inc, "-I",
                  pybind11.get_include(), helper_src, "-o", helper_lib], verbose)
            stamps[helper_src.name] = d

    stamp_file.write_text(json.dumps(stamps, indent=1))
    return out_lib


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
