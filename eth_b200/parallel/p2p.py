"""Pipeline point-to-point transfers with cross-stage resharding (TP_a x DP_a -> TP_b x DP_b).

A boundary tensor is described by `(name, features/hidden, tp_sharded, per_token)`. Per-token
tensors are `[tokens, features]` with batch-major rows, so a data-parallel rank owns a contiguous
block of rows; a TP-sharded tensor additionally owns a block of columns. The transfer plan is the
set of rectangle intersections between what every source rank holds and what every destination
rank needs; replicated sources are read from exactly one TP rank (`dst_tp_rank % src_tp`), so no
element is sent twice. The same planner serves activations (stage i -> i+1) and gradients
(stage i+1 -> i). All ranks derive the same plan from the canonical topology, which fixes the
order of the batched isend/irecv calls on both sides.

Reference behaviour: static fan-out / fan-in maps by ratio (eth/runtime/megatron/mpu/initialize.py:
212-280), chunk on send / concatenate on receive (model/flex_model.py:63-169,
p2p_communication.py:84-198), one batched isend/irecv per tensor followed by a device-wide
synchronize (:234-322). Here one batch covers all tensors of a boundary and nothing synchronizes
the host: completion is a stream dependency.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Piece:
    """A rectangle moved between one source and one destination rank, in local coordinates."""
    name: str
    src_rank: int
    dst_rank: int
    src_rows: Tuple[int, int]     # sample range inside the source's local batch
    dst_rows: Tuple[int, int]     # sample range inside the destination's local batch
    src_cols: Tuple[int, int]     # in units of the tensor's features on the source rank
    dst_cols: Tuple[int, int]
    per_token: bool


def _overlap(a: Tuple[int, int], b: Tuple[int, int]) -> Optional[Tuple[int, int]]:
    lo, hi = max(a[0], b[0]), min(a[1], b[1])
    return (lo, hi) if lo < hi else None


def plan_transfers(src_stage, dst_stage, tensor_spec, micro_batch: int, hidden: int) -> List[Piece]:
    """Every piece that must move from `src_stage` to `dst_stage` for one micro-batch.

    `tensor_spec`: iterable of (name, feature_multiple, tp_sharded, per_token).
    Rows are counted in samples (the caller multiplies by the sequence length)."""
    pieces: List[Piece] = []
    ts, ds, td, dd = src_stage.tp_degree, src_stage.dp_degree, dst_stage.tp_degree, dst_stage.dp_degree
    if micro_batch % ds or micro_batch % dd:
        raise ValueError("micro batch must be divisible by both stages' DP degrees")
    src_b, dst_b = micro_batch // ds, micro_batch // dd
    for name, mult, tp_sharded, per_token in tensor_spec:
        feat = mult * hidden
        if not per_token and ds != dd:
            raise NotImplementedError(
                f"boundary tensor {name!r} is a per-stage vector; a stage cut that carries it needs equal "
                f"data-parallel degrees on both sides (got {ds} and {dd}); cut at a layer boundary instead")
        for dc in dst_stage.rank_coordinates:
            need_rows = (dc.dp_rank * dst_b, (dc.dp_rank + 1) * dst_b) if per_token else (0, 1)
            need_cols = ((dc.tp_rank * feat // td, (dc.tp_rank + 1) * feat // td) if tp_sharded else (0, feat))
            for sc in src_stage.rank_coordinates:
                if per_token:
                    have_rows = (sc.dp_rank * src_b, (sc.dp_rank + 1) * src_b)
                else:
                    # vectors are replicated over the source's DP ranks: take the matching replica
                    if sc.dp_rank != dc.dp_rank % ds:
                        continue
                    have_rows = (0, 1)
                rows = _overlap(need_rows, have_rows)
                if rows is None:
                    continue
                if tp_sharded:
                    have_cols = (sc.tp_rank * feat // ts, (sc.tp_rank + 1) * feat // ts)
                else:
                    if sc.tp_rank != dc.tp_rank % ts:
                        continue
                    have_cols = (0, feat)
                cols = _overlap(need_cols, have_cols)
                if cols is None:
                    continue
                pieces.append(Piece(
                    name=name, src_rank=sc.global_rank, dst_rank=dc.global_rank,
                    src_rows=(rows[0] - have_rows[0], rows[1] - have_rows[0]),
                    dst_rows=(rows[0] - need_rows[0], rows[1] - need_rows[0]),
                    src_cols=(cols[0] - have_cols[0], cols[1] - have_cols[0]),
                    dst_cols=(cols[0] - need_cols[0], cols[1] - need_cols[0]),
                    per_token=per_token))
    pieces.sort(key=lambda p: (p.src_rank, p.dst_rank, p.name, p.dst_rows, p.dst_cols))
    return pieces


class BoundaryChannel:
    """Sends / receives the tensors of one stage boundary in one direction for this rank."""

    def __init__(self, rank: int, pieces: Sequence[Piece], seq_len: int, group=None):
        self.rank, self.seq_len, self.group = rank, seq_len, group
        self.sends = [p for p in pieces if p.src_rank == rank]
        self.recvs = [p for p in pieces if p.dst_rank == rank]

    def _view(self, t: torch.Tensor, rows, cols, per_token: bool) -> torch.Tensor:
        if not per_token:
            return t[cols[0]:cols[1]]
        s = self.seq_len
        return t[rows[0] * s:rows[1] * s, cols[0]:cols[1]]

    def make_ops(self, send_tensors: Optional[Dict[str, torch.Tensor]], recv_buffers: Optional[Dict[str, torch.Tensor]]):
        """P2POps plus the list of (staging, destination view) copies to run after completion."""
        ops, post = [], []
        if send_tensors is not None:
            for p in self.sends:
                v = self._view(send_tensors[p.name], p.src_rows, p.src_cols, p.per_token)
                if not v.is_contiguous():
                    v = v.contiguous()
                ops.append(dist.P2POp(dist.isend, v, p.dst_rank, self.group))
        if recv_buffers is not None:
            for p in self.recvs:
                v = self._view(recv_buffers[p.name], p.dst_rows, p.dst_cols, p.per_token)
                if v.is_contiguous():
                    ops.append(dist.P2POp(dist.irecv, v, p.src_rank, self.group))
                else:
                    tmp = torch.empty(v.shape, dtype=v.dtype, device=v.device)
                    ops.append(dist.P2POp(dist.irecv, tmp, p.src_rank, self.group))
                    post.append((tmp, v))
        return ops, post


def run_batch(op_lists) -> None:
    """Issue all P2POps of several channels as one batch; wait on the stream, copy staged pieces."""
    ops, post = [], []
    for o, p in op_lists:
        ops += o
        post += p
    if not ops:
        return
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    for tmp, dst in post:
        dst.copy_(tmp)


class PipelineComm:
    """The four channels of a rank: activations in/out and gradients in/out."""

    def __init__(self, pstate, hidden: int, seq_len: int, in_spec, out_spec, dtype, device, group=None,
                 neighbours=None):
        """`neighbours`: (previous stage, next stage) topologies when they are not the adjacent
        physical stages (interleaved pipelining wraps from the last stage to the first)."""
        self.pstate, self.dtype, self.device, self.seq_len, self.hidden = pstate, dtype, device, seq_len, hidden
        mbs = pstate.micro_batch_size
        prev, nxt = neighbours if neighbours is not None else (pstate.neighbour(-1), pstate.neighbour(+1))
        me = pstate.stage
        self.in_spec, self.out_spec = tuple(in_spec), tuple(out_spec)
        r = pstate.rank
        self.fwd_in = BoundaryChannel(r, plan_transfers(prev, me, in_spec, mbs, hidden), seq_len, group) if prev else None
        self.fwd_out = BoundaryChannel(r, plan_transfers(me, nxt, out_spec, mbs, hidden), seq_len, group) if nxt else None
        self.bwd_in = BoundaryChannel(r, plan_transfers(nxt, me, out_spec, mbs, hidden), seq_len, group) if nxt else None
        self.bwd_out = BoundaryChannel(r, plan_transfers(me, prev, in_spec, mbs, hidden), seq_len, group) if prev else None

    def _buffers(self, spec, grad: bool = False) -> Dict[str, torch.Tensor]:
        ps = self.pstate
        tokens = ps.local_micro_batch * self.seq_len
        out = {}
        for name, mult, tp_sharded, per_token in spec:
            feat = mult * self.hidden // (ps.tp_size if tp_sharded else 1)
            shape = (tokens, feat) if per_token else (feat,)
            dt = torch.float32 if (grad and not per_token) else self.dtype
            out[name] = torch.empty(shape, dtype=dt, device=self.device)
        return out

    # -- the combinations used by the schedules (reference: p2p_communication.py:344-538)
    def recv_forward(self):
        if self.fwd_in is None:
            return None
        bufs = self._buffers(self.in_spec)
        run_batch([self.fwd_in.make_ops(None, bufs)])
        return bufs

    def send_forward(self, outputs):
        if self.fwd_out is not None:
            run_batch([self.fwd_out.make_ops(outputs, None)])

    def recv_backward(self):
        if self.bwd_in is None:
            return None
        bufs = self._buffers(self.out_spec, grad=True)
        run_batch([self.bwd_in.make_ops(None, bufs)])
        return bufs

    def send_backward(self, grads):
        if self.bwd_out is not None:
            run_batch([self.bwd_out.make_ops(self._complete(grads, self.in_spec), None)])

    def send_forward_recv_backward(self, outputs):
        if self.fwd_out is None:
            return None
        bufs = self._buffers(self.out_spec, grad=True)
        run_batch([self.fwd_out.make_ops(outputs, None), self.bwd_in.make_ops(None, bufs)])
        return bufs

    def send_backward_recv_forward(self, grads):
        if self.bwd_out is None:
            return None
        bufs = self._buffers(self.in_spec)
        run_batch([self.bwd_out.make_ops(self._complete(grads, self.in_spec), None), self.fwd_in.make_ops(None, bufs)])
        return bufs

    def _complete(self, grads, spec):
        """Gradients missing from a backward pass are sent as zeros (reference: schedules.py:196-227)."""
        out = dict(grads)
        need = self._buffers(spec, grad=True) if any(n not in out for n, *_ in spec) else {}
        for name, *_ in spec:
            if name not in out:
                out[name] = need[name].zero_()
        return out


def exchange(send_next=None, send_prev=None, recv_prev=None, recv_next=None):
    """One batched call with up to four transfers of possibly different model chunks:
        send_next = (comm, activations)   output of a chunk to the stage that runs the next virtual stage
        send_prev = (comm, gradients)     input gradients of a chunk to the stage before it
        recv_prev = comm                  inputs of that comm's chunk
        recv_next = comm                  output gradients of that comm's chunk
    always posted in this order. Every rank uses the same order, so two ranks that are each other's
    previous AND next stage (a two-stage interleaved pipeline wraps around) pair their messages
    correctly. Returns (received activations or None, received gradients or None)."""
    batches, got_fwd, got_bwd = [], None, None
    if send_next is not None and send_next[0].fwd_out is not None:
        comm, tensors = send_next
        batches.append(comm.fwd_out.make_ops(tensors, None))
    if send_prev is not None and send_prev[0].bwd_out is not None:
        comm, grads = send_prev
        batches.append(comm.bwd_out.make_ops(comm._complete(grads, comm.in_spec), None))
    if recv_prev is not None and recv_prev.fwd_in is not None:
        got_fwd = recv_prev._buffers(recv_prev.in_spec)
        batches.append(recv_prev.fwd_in.make_ops(None, got_fwd))
    if recv_next is not None and recv_next.bwd_in is not None:
        got_bwd = recv_next._buffers(recv_next.out_spec, grad=True)
        batches.append(recv_next.bwd_in.make_ops(None, got_bwd))
    run_batch(batches)
    return got_fwd, got_bwd
