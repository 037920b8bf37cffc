"""Dataset index helpers: the compiled extension when built, else a NumPy/Python restatement."""
from __future__ import annotations

import numpy as np

try:
    from .. import _data_helpers as _native
except Exception:  # pragma: no cover - extension not built
    _native = None


def build_sample_idx_python(sizes, doc_idx, seq_length: int, num_epochs: int, tokens_per_epoch: int):
    """Reference semantics in plain Python (oracle of the compiled helper)."""
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    pos, offset = 0, 0
    for s in range(1, num_samples + 1):
        need = seq_length + 1
        while need != 0:
            left = int(sizes[doc_idx[pos]]) - offset
            need -= left
            if need <= 0:
                offset += need + left - 1
                need = 0
            else:
                pos += 1
                offset = 0
        out[s] = (pos, offset)
    return out


def build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    if _native is not None:
        return _native.build_sample_idx(np.ascontiguousarray(sizes, dtype=np.int32),
                                        np.ascontiguousarray(doc_idx, dtype=np.int32), seq_length, num_epochs,
                                        tokens_per_epoch)
    return build_sample_idx_python(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)


def build_blending_indices(weights, size: int, verbose: bool = False):
    weights = np.asarray(weights, dtype=np.float64)
    ds = np.zeros(size, dtype=np.uint8)
    sample = np.zeros(size, dtype=np.int64)
    if _native is not None:
        _native.build_blending_indices(ds, sample, weights, len(weights), size, verbose)
        return ds, sample
    taken = np.zeros(len(weights), dtype=np.int64)
    for i in range(size):
        err = weights * max(float(i), 1.0) - taken
        k = int(np.argmax(err))
        ds[i], sample[i] = k, taken[k]
        taken[k] += 1
    return ds, sample


def native_available() -> bool:
    return _native is not None
