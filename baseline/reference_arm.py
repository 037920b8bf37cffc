"""Reference arm of the benchmark.

The reference (YuMJie/ETH) ships no packaging metadata: `pip install --no-index --no-build-isolation
--find-links /opt/wheelhouse --target baseline/_ref <reference>` stops in metadata generation
("Multiple top-level packages discovered in a flat-layout: ['eth', 'LICENSES', 'external']"), with
and without `--no-deps`, from the read-only mount and from a writable copy. Run from its source
tree it still cannot execute on sm_100 unmodified: its LayerNorm / softmax extensions are compiled
with `-gencode arch=compute_70,code=sm_70` and `compute_80,sm_80` only (no PTX, so no forward
compatibility; eth/runtime/megatron/fused_kernels/__init__.py:36-54), the runtime imports `apex`
unconditionally while the pinned submodule is empty (optimizer/__init__.py:18-19), and the launcher
insists on CUDA 12.4 (tools/validation/validate_cuda_toolchain.py:34-40). This arm therefore
reports `unavailable` and exits 0.
"""
import json
import os

REASON = ("reference is not pip-installable (no packaging metadata: setuptools flat-layout discovery fails) and "
          "its CUDA extensions are built for sm_70/sm_80 only, apex submodule empty")


def run(opts, model, layouts, samples_per_gpu, micro_batch, vocab):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": REASON}), flush=True)
