"""Tensor-parallel linears fused with their all-reduce over NVLink peer memory.

Row-parallel forward (`Y = sum_r X_r W_r^T`) and column-parallel data-gradient
(`dX = sum_r dY_r W_r`) are each ONE launch of the tcgen05 GEMM. Tiles are owned round-robin; every
rank computes the tiles its peers own first and pushes those partials into the owners' staging areas
while the tensor cores already work on the next tile, and computes its own tiles last: by then the
peers' partials have arrived, so the epilogue adds them to the accumulator in fp32 and writes the
result into every rank's output buffer. Only that last transfer is exposed after the final MMA
(reference: a cuBLAS GEMM followed by an exposed NCCL all-reduce,
eth/runtime/megatron/mpu/layers.py:459-461, mappings.py:84-97).

The outputs live in a small ring of symmetric buffers (peers write into them directly), so a
returned tensor is valid until `ring` further fused calls have been issued; the stage program
consumes every such tensor with the very next kernel.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native
from .peer_memory import SymmetricBuffer

MAX_TILES = 8192
RING = 4


def reduce_scatter_schedule(cta: int, grid: int, it: int, tiles_m: int, tiles_n: int, world: int, group_m: int = 16):
    """Host mirror of the device tile schedule of the fused GEMM + reduce-scatter (`sched_tile` in
    csrc/gemm_sm100.cu): the it-th tile of CTA `cta` as (owner, tile row, tile column), or None past
    the end. Within one `it`, the CTAs W * j + r cover, for every owner, G / W consecutive tiles of
    that owner's row block, so a CTA's tiles alternate between owners and every tile is visited once."""
    rows_per = tiles_m // world
    vp = it * (grid // world) + cta // world
    if vp >= rows_per * tiles_n:
        return None
    per_band = group_m * tiles_n
    band, r = divmod(vp, per_band)
    rows = min(group_m, rows_per - band * group_m)
    tn, rr = divmod(r, rows)
    owner = (cta + it) % world
    return owner, owner * rows_per + band * group_m + rr, tn


def all_reduce_order(okey: int, n_tiles: int, world: int, rank: int):
    """Host mirror of `comm_order` in csrc/gemm_sm100.cu: the order in which a CTA (or CTA pair)
    with ownership key `okey` walks its list of `n_tiles` tiles in the fused all-reduce. List index
    `it` is owned by rank (okey + it) % world; tiles of rank+1 come first, then rank+2, ..., and the
    rank's own tiles last."""
    order = []
    for g in range(1, world + 1):
        owner = (rank + g) % world
        first = (owner - okey) % world
        order.extend(range(first, n_tiles, world))
    return order


class FusedTPBackend:
    def __init__(self, group_ranks, my_rank, group, device, max_tokens: int, hidden: int, dtype):
        self.group, self.device, self.dtype = group, torch.device(device), dtype
        self.world = len(group_ranks)
        self.max_tokens, self.hidden = max_tokens, hidden
        esize = 2
        rows = (max_tokens + 127) // 128 * 128
        cols = (hidden + 255) // 256 * 256
        self.out_slot_bytes = rows * cols * esize
        # staging holds `world` partials of each owned tile (about one full output) plus one spare
        # slot per CTA and source, because slots are assigned per CTA
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.stage_elems = rows * cols + (sms + 1) * self.world * 128 * 256
        self.stage = SymmetricBuffer(self.stage_elems * esize, group_ranks, my_rank, group, device, holds_data=True)
        self.out = SymmetricBuffer(self.out_slot_bytes * RING, group_ranks, my_rank, group, device, holds_data=True)
        self.flags = SymmetricBuffer(MAX_TILES * 9 * 4, group_ranks, my_rank, group, device)
        # all-gather + GEMM: a ring of [max_tokens, hidden-or-wider] operand buffers and their own flags
        self.ag_cols = max(hidden, cols)
        self.ag_slot_bytes = rows * self.ag_cols * esize
        self.ag = SymmetricBuffer(self.ag_slot_bytes * RING, group_ranks, my_rank, group, device, holds_data=True)
        self.ag_flags = SymmetricBuffer((64 + rows // 8) * 4, group_ranks, my_rank, group, device)
        self.ag_slot = 0
        self.rank = self.stage.index
        self.epoch = 0
        self.slot = 0

    @classmethod
    def create(cls, pstate, coll, device, args):
        cfg = pstate.config
        max_tokens = pstate.local_micro_batch * cfg["seq_length"]
        return cls(pstate.tp_group_ranks, pstate.rank, pstate.tp_group, device, max_tokens, cfg["hidden_size"],
                   args.params_dtype)

    def supports(self, m: int, n: int) -> bool:
        return m <= self.max_tokens and n <= self.hidden and n % 8 == 0

    def gemm_all_reduce(self, a, b, *, b_mn=False, bias=None, residual=None, alpha=1.0, dropout=None):
        """sum over the TP group of (a x b^T) (+ bias, dropout, + residual, applied once, by the rank
        that reduces a tile). `dropout` = (p, seed, offset). Returns a view of a ring slot holding
        the [M, N] result."""
        m = a.shape[0]
        n = b.shape[1] if b_mn else b.shape[0]
        if not self.supports(m, n):
            raise ValueError(f"fused all-reduce GEMM: shape {m}x{n} exceeds the symmetric buffers")
        self.epoch += 1
        slot = self.slot
        self.slot = (self.slot + 1) % RING
        off = slot * self.out_slot_bytes
        p_drop, seed, offset = dropout if (dropout is not None and dropout[0] > 0) else (0.0, 0, 0)
        native.lib().gemm_allreduce(a, False, b, b_mn, bias, residual, float(alpha), native.status(a.device),
                                    self.stage.ptrs, self.out.offset_ptrs(off), self.flags.ptrs, self.rank,
                                    self.epoch, MAX_TILES, self.stage_elems, n, 0, float(p_drop), int(seed), int(offset))
        out = self.out.tensor((m, n), self.dtype, off)
        out._ethb_ring = True   # short-lived: valid until RING further fused calls
        return out

    def gemm_reduce_scatter(self, a, b, *, b_mn=False, bias=None, residual=None, alpha=1.0):
        """Rows [rank * M / world, (rank + 1) * M / world) of the sum over the TP group of (a x b^T)
        (+ bias, + residual given as this rank's [M / world, N] slice): the sequence-parallel form of
        a row-parallel linear. One kernel: every rank pushes the partial tiles of a peer's row block
        into that peer's staging area while it computes the next tile; the owner reduces and keeps
        the rows. M must be a multiple of 128 * world. Returns a view of a ring slot."""
        m = a.shape[0]
        n = b.shape[1] if b_mn else b.shape[0]
        if not self.supports(m, n):
            raise ValueError(f"fused reduce-scatter GEMM: shape {m}x{n} exceeds the symmetric buffers")
        if m % (128 * self.world):
            raise ValueError("fused reduce-scatter GEMM: rows must be a multiple of 128 * world")
        self.epoch += 1
        slot = self.slot
        self.slot = (self.slot + 1) % RING
        off = slot * self.out_slot_bytes
        native.lib().gemm_allreduce(a, False, b, b_mn, bias, residual, float(alpha), native.status(a.device),
                                    self.stage.ptrs, self.out.offset_ptrs(off), self.flags.ptrs, self.rank,
                                    self.epoch, MAX_TILES, self.stage_elems, n, 1)
        out = self.out.tensor((m // self.world, n), self.dtype, off)
        out._ethb_ring = True
        return out

    def gather_buffer(self, m: int, k: int):
        """Next [m, k] operand buffer of the all-gather ring and the view of this rank's own row block
        inside it; the caller writes its block (e.g. as the output of the producing kernel) and then
        passes the buffer to `gemm_all_gather`."""
        if m > self.max_tokens or k > self.ag_cols or m % (128 * self.world) or k % 8:
            raise ValueError(f"all-gather GEMM: operand {m}x{k} not supported by the symmetric buffers")
        off = self.ag_slot * self.ag_slot_bytes
        self.ag_slot = (self.ag_slot + 1) % RING
        full = self.ag.tensor((m, k), self.dtype, off)
        rows = m // self.world
        full._ethb_ring, full._ethb_offset = True, off
        return full, full[self.rank * rows:(self.rank + 1) * rows]

    def gemm_all_gather(self, full, weight, *, b_mn=False, bias=None, gelu_out=None, out=None):
        """out = concat_r(A_r) x weight^T where every rank has written its row block A_r into its own
        `full` buffer (from `gather_buffer`). One kernel: a gather warp per CTA pushes this rank's block
        into the peers' buffers over NVLink while the MMAs start on the local rows; tiles of a peer's
        rows wait for those rows only. The column-parallel forward of a sequence-parallel layer."""
        m = full.shape[0]
        n = weight.shape[1] if b_mn else weight.shape[0]
        if out is None:
            out = torch.empty((m, n), dtype=self.dtype, device=self.device)
        self.epoch += 1
        native.lib().gemm_allgather(full, weight, b_mn, out, bias, gelu_out, native.status(full.device),
                                    self.ag.offset_ptrs(full._ethb_offset), self.ag_flags.ptrs, self.rank, self.epoch)
        return out

    def all_reduce_(self, t):
        dist.all_reduce(t, group=self.group)
        return t

    def close(self):
        for b in (self.stage, self.out, self.flags, self.ag, self.ag_flags):
            b.close()
