"""JIT-extension handling for the reference arm, kept outside the reference tree.

The reference compiles four CUDA extensions at start-up through `torch.utils.cpp_extension.load`
with `-gencode` flags for sm_70 and sm_80 only (eth/runtime/megatron/fused_kernels/__init__.py:36-54)
and then imports them by bare module name (model/fused_layer_norm.py:67-69,
model/fused_softmax.py:32). Two things are supplied from here while the reference runs:

* an sm_100 target appended to `extra_cuda_cflags`, and
* a warm build cache: the four extensions take over twenty minutes to compile, so they can be
  compiled ahead of time (`python -m baseline.reference_build`, no GPU needed) into the
  reference's own build directory; at run time an extension whose sources still hash to the
  recorded stamp is imported from there without invoking the compiler. Otherwise the reference's
  normal JIT build runs (with the extra target).

Either way the module is registered in `sys.modules`, because current PyTorch no longer does that
for JIT-loaded extensions and the reference's by-name imports rely on it.
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_RUNTIME = os.path.join(HERE, "_ref", "eth", "runtime")
SM100_GENCODE = ["-gencode", "arch=compute_100,code=sm_100"]
STAMP = "prebuilt_stamp.json"


def _sources_digest(sources, flags) -> str:
    h = hashlib.sha256(json.dumps([str(f) for f in flags]).encode())
    for src in sorted(str(s) for s in sources):
        h.update(os.path.basename(src).encode())
        with open(src, "rb") as f:
            h.update(f.read())
    folder = os.path.dirname(str(sorted(str(s) for s in sources)[0]))
    for name in sorted(os.listdir(folder)):          # headers the sources include
        if name.endswith((".h", ".cuh")):
            with open(os.path.join(folder, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    return h.hexdigest()


def _import_shared_object(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[name] = module
    return module


def wrap_extension_loader(log=None):
    """Replaces `cpp_extension.load` until the returned function is called. `log` collects one
    line per extension saying whether it was reused or compiled."""
    from torch.utils import cpp_extension
    original = cpp_extension.load

    def load(name, sources, *args, **kwargs):
        flags = list(kwargs.get("extra_cuda_cflags") or []) + SM100_GENCODE
        kwargs["extra_cuda_cflags"] = flags
        build_dir = kwargs.get("build_directory")
        if build_dir is not None:
            build_dir = str(build_dir)
            so = os.path.join(build_dir, name + ".so")
            stamp = os.path.join(build_dir, STAMP)
            try:
                recorded = json.load(open(stamp)).get(name)
            except (OSError, ValueError):
                recorded = None
            if recorded and os.path.exists(so) and recorded == _sources_digest(sources, flags):
                if log is not None:
                    log.append(f"{name}: reused prebuilt")
                return _import_shared_object(name, so)
        module = original(name, sources, *args, **kwargs)
        if isinstance(module, types.ModuleType):
            sys.modules[name] = module
        if build_dir is not None:
            stamp = os.path.join(build_dir, STAMP)
            try:
                stamps = json.load(open(stamp))
            except (OSError, ValueError):
                stamps = {}
            stamps[name] = _sources_digest(sources, flags)
            tmp = f"{stamp}.{os.getpid()}.tmp"
            with open(tmp, "w") as f:
                json.dump(stamps, f, indent=1)
            os.replace(tmp, stamp)
        if log is not None:
            log.append(f"{name}: compiled")
        return module

    cpp_extension.load = load
    return lambda: setattr(cpp_extension, "load", original)


def prebuild() -> None:
    """Compile the reference's extensions and its dataset helper into the copied tree."""
    sys.path[:0] = [REF_RUNTIME, os.path.join(HERE, "shims")]
    os.chdir(REF_RUNTIME)
    log = []
    restore = wrap_extension_loader(log)
    try:
        from megatron import fused_kernels
        t0 = time.time()
        fused_kernels.load(types.SimpleNamespace(rank=0, masked_softmax_fusion=True))
        print(f"extensions ready in {time.time() - t0:.0f} s: {log}")
        from megatron.data.dataset_utils import compile_helper
        compile_helper()
    finally:
        restore()


if __name__ == "__main__":
    prebuild()
