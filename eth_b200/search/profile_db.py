"""Profile tables consumed by the search.

Layout of a profile directory (the schema of the reference, eth/profiler/op_profiler.py:424-445,
comm_profiler.py:157-171, p2p_band_profiler.py:91-95, validated by
eth/searching/profile_validation.py:114-136):
    gpt_<size>_mbs<m>_tp<t>_algo<a>.csv   op_name, forward-compute, backward-compute (us),
                                          input_size, output_size, weights, activations,
                                          fwd_reserved, bwd_reserved (MB) -- one row per op of the
                                          one-layer op list
    prim_gpt_<size>_<collective>_<n>gpus.csv   data_size(MB), time(ms)
    p2p_intra_node.csv [/ p2p_inter_node.csv]  row 0 sizes (MB), row 1 send GB/s, row 2 recv GB/s
    profile_metadata.json
A search over several GPU types reads one such directory per type:
    <root>/<gpu type>/gpt_<size>/...  and  <root>/<gpu type>/p2p_intra_node.csv
(the `profile_view` that search_gpt.sh builds, scripts/search_gpt.sh:104-110).
"""
from __future__ import annotations

import bisect
import csv
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

OP_HEADER = ["op_name", "forward-compute", "backward-compute", "input_size", "output_size", "weights",
             "activations", "fwd_reserved", "bwd_reserved"]
COLLECTIVES = ("all_gather", "all_reduce", "reduce_scatter", "all_to_all")
MISSING_TIME_US = 1.0e6   # sentinel of the reference for an unmeasured op (state.py:100-215)
TP_SIZES = (1, 2, 4, 6, 8)


@dataclass
class OpRecord:
    name: str
    fwd_us: float
    bwd_us: float
    input_mb: float
    output_mb: float
    weights_mb: float
    activations_mb: float
    fwd_reserved_mb: float
    bwd_reserved_mb: float


@dataclass
class LayerCost:
    """Aggregated cost of a contiguous group of ops (pre, one layer, post) at one (mbs, tp, algo)."""
    fwd_us: float = 0.0
    bwd_us: float = 0.0
    weights_mb: float = 0.0
    activations_mb: float = 0.0
    reserved_mb: float = 0.0
    boundary_mb: float = 0.0   # size of the tensor leaving the group


class ProfileDB:
    """Profile of one GPU type for one model size."""

    def __init__(self, gpu_type: str, model_size: str):
        self.gpu_type, self.model_size = gpu_type, model_size
        self.ops: Dict[Tuple[int, int, int], List[OpRecord]] = {}      # (mbs, tp, algo) -> rows
        self.collective: Dict[Tuple[str, int], List[Tuple[float, float]]] = {}  # (prim, n) -> sorted (MB, ms)
        self.p2p_sizes: List[float] = []
        self.p2p_intra: List[float] = []
        self.p2p_inter: List[float] = []

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, profile_dir: str, gpu_type: str, model_size: str, mbs_list: Sequence[int] = (1, 2, 4, 8),
             max_tp: int = 8, p2p_dir: Optional[str] = None, inter_node_file: Optional[str] = None) -> "ProfileDB":
        db = cls(gpu_type, model_size)
        for mbs in mbs_list:
            for tp in [t for t in TP_SIZES if t <= max_tp]:
                for algo in (0, 1):
                    path = os.path.join(profile_dir, f"gpt_{model_size}_mbs{mbs}_tp{tp}_algo{algo}.csv")
                    if os.path.exists(path):
                        db.ops[(mbs, tp, algo)] = read_op_csv(path)
        for prim in COLLECTIVES:
            for n in [t for t in TP_SIZES if 1 < t <= max_tp]:
                path = os.path.join(profile_dir, f"prim_gpt_{model_size}_{prim}_{n}gpus.csv")
                if os.path.exists(path):
                    db.collective[(prim, n)] = read_collective_csv(path)
        p2p_dir = p2p_dir or profile_dir
        intra = os.path.join(p2p_dir, "p2p_intra_node.csv")
        if os.path.exists(intra):
            db.p2p_sizes, db.p2p_intra = read_p2p_csv(intra)
        if inter_node_file and os.path.exists(inter_node_file):
            _, db.p2p_inter = read_p2p_csv(inter_node_file)
        else:
            db.p2p_inter = list(db.p2p_intra)
        if not db.ops:
            raise FileNotFoundError(f"no op profile records for gpt_{model_size} in {profile_dir}")
        return db

    # ------------------------------------------------------------------ queries
    def op_names(self) -> List[str]:
        return [r.name for r in next(iter(self.ops.values()))]

    def has(self, mbs: int, tp: int, algo: int = 0) -> bool:
        return (mbs, tp, algo) in self.ops

    def records(self, mbs: int, tp: int, algo: int = 0) -> List[OpRecord]:
        return self.ops[(mbs, tp, algo)]

    def collective_ms(self, prim: str, n: int, size_mb: float) -> float:
        """Measured time of a collective, interpolated between the neighbouring sizes."""
        if n <= 1 or size_mb <= 0:
            return 0.0
        table = self.collective.get((prim, n))
        if not table:
            return 0.0
        sizes = [s for s, _ in table]
        i = bisect.bisect_left(sizes, size_mb)
        if i == 0:
            return table[0][1] * (size_mb / table[0][0]) if table[0][0] > 0 else table[0][1]
        if i >= len(table):
            s, t = table[-1]
            return t * size_mb / s
        (s0, t0), (s1, t1) = table[i - 1], table[i]
        if s1 == s0:
            return t1
        return t0 + (t1 - t0) * (size_mb - s0) / (s1 - s0)

    def p2p_ms(self, size_mb: float, inter_node: bool = False) -> float:
        """size / bandwidth(size) with the bandwidth taken from the log2 size bucket
        (reference: cost_model.py:145-171)."""
        if size_mb <= 0:
            return 0.0
        bw = self.p2p_inter if inter_node else self.p2p_intra
        if not bw:
            return 0.0
        idx = min(len(bw) - 1, max(0, int(math.floor(math.log2(max(size_mb, 1.0))))))
        gbs = max(bw[idx], 1e-6)
        return size_mb / 1024.0 / gbs * 1e3


def read_op_csv(path: str) -> List[OpRecord]:
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if not rows or [c.strip() for c in rows[0]] != OP_HEADER:
        raise ValueError(f"invalid profile record schema: {os.path.basename(path)}")
    out = []
    for r in rows[1:]:
        if not r:
            continue
        vals = [float(x) for x in r[1:9]]
        out.append(OpRecord(r[0], *vals))
    return out


def read_collective_csv(path: str) -> List[Tuple[float, float]]:
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    out = [(float(r[0]), float(r[1])) for r in rows[1:] if r]
    return sorted(out)


def read_p2p_csv(path: str) -> Tuple[List[float], List[float]]:
    with open(path, newline="") as f:
        rows = [r for r in csv.reader(f) if r]
    sizes = [float(x) for x in rows[0]]
    send = [float(x) for x in rows[1]]
    return sizes, send
