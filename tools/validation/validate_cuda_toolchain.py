#!/usr/bin/env python3
"""Check that the CUDA toolchain can build and run the sm_100a kernels: nvcc >= 12.8 (first
release with sm_100a) and the same CUDA major version as the PyTorch build.

The reference pins CUDA 12.4 exactly for both (tools/validation/validate_cuda_toolchain.py:20-41);
that release cannot target Blackwell, so the rule here is a lower bound plus major agreement."""
import argparse
import re
import subprocess
import sys

MIN_NVCC = (12, 8)


def nvcc_version(nvcc: str):
    out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=True).stdout
    m = re.search(r"release (\d+)\.(\d+)", out)
    if not m:
        raise ValueError(f"cannot parse nvcc version from: {out!r}")
    return int(m.group(1)), int(m.group(2))


def validate_versions(torch_cuda, nvcc):
    """torch_cuda: 'major.minor' string or None; nvcc: (major, minor). Returns an error string or None."""
    if torch_cuda is None:
        return "PyTorch was built without CUDA"
    tmaj = int(str(torch_cuda).split(".")[0])
    if nvcc < MIN_NVCC:
        return f"nvcc {nvcc[0]}.{nvcc[1]} cannot target sm_100a; need >= {MIN_NVCC[0]}.{MIN_NVCC[1]}"
    if tmaj != nvcc[0]:
        return f"CUDA major mismatch: PyTorch {torch_cuda} vs nvcc {nvcc[0]}.{nvcc[1]}"
    return None


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--nvcc", required=True)
    a = ap.parse_args(argv)
    try:
        import torch
        err = validate_versions(torch.version.cuda, nvcc_version(a.nvcc))
    except (OSError, ValueError, subprocess.CalledProcessError) as e:
        err = str(e)
    if err:
        print(f"CUDA toolchain validation failed: {err}", file=sys.stderr)
        return 1
    print("CUDA toolchain validated")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
