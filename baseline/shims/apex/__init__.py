"""Stand-in for NVIDIA Apex, kept outside the reference tree.

The reference imports `apex.optimizers` and `apex.multi_tensor_apply` unconditionally
(eth/runtime/megatron/optimizer/__init__.py:18-19, optimizer/optimizer.py:23,
optimizer/clip_grads.py:21, utils.py:31) while its pinned `external/apex` submodule is empty.
This package makes those imports succeed and reports the fused extensions as absent, which is the
situation the reference itself handles: its optimizer factory falls back to `torch.optim.AdamW`
when the fused constructor raises "requires cuda extensions" (optimizer/__init__.py:28-34), and
its norm / scale helpers take their PyTorch branch when `multi_tensor_applier.available` is False.
"""
