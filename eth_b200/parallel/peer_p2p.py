"""Pipeline transfers through peer memory: copy engines move the data, flags say when it is there.

The NCCL path (`p2p.PipelineComm`) runs send and receive kernels that spin on an SM until their
partner shows up, and the compute stream waits for both. Inside one NVLink domain none of that is
needed. Every rank owns two inboxes in symmetric (CUDA-IPC) memory, one for activations coming
from the previous stage and one for gradients coming from the next stage, each a ring of slots
laid out for the boundary's tensors. A sender copies its rectangles (the same rectangle plan as
the NCCL path, `p2p.plan_transfers`, so any TP x DP -> TP x DP boundary works) straight into the
receivers' slots with 2-D device-to-device copies on a copy stream that waits for an event of the
compute stream: no SM takes part and the compute stream never waits for a send. Then it posts the
transfer's sequence number to one flag per receiver. A receive is a one-warp wait kernel on the
compute stream for the flags of the ranks that write to this slot; the received tensors are views
of the slot, so nothing is copied out, and receives are "posted" for the whole run by construction.

Slot reuse needs no acknowledgement under 1F1B: a stage sends micro-batch i + R forward only after
it has received the gradient of micro-batch i + R - (stages - stage) from its successor, which
the successor sends after its backward of that micro-batch, i.e. after everything it did with
micro-batch i; with R = stages + 1 slots that covers activations, and gradients live only during
one backward. Forward-only passes have no such feedback and keep using the NCCL channels.

Reference behaviour replaced: eth/runtime/megatron/p2p_communication.py:234-322 (batched
isend/irecv followed by a device synchronize).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .p2p import Piece, plan_transfers

FLAG_BYTES = 256          # room for 64 int32 flags at the start of an inbox
ALIGN = 256
WAIT_LIMITS = 5           # a stage may wait for its neighbour this many wait limits (5 x 2 s)


def _align(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


@dataclass(frozen=True)
class SlotTensor:
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype
    offset: int            # bytes from the start of a slot

    @property
    def nbytes(self) -> int:
        n = torch.empty((), dtype=self.dtype).element_size()
        for d in self.shape:
            n *= d
        return n


def slot_layout(spec, tokens: int, hidden: int, tp: int, dtype: torch.dtype, grads: bool) -> Tuple[List[SlotTensor], int]:
    """Tensors of one ring slot for a rank with `tokens` local rows in a stage of TP degree `tp`,
    and the slot's size. Gradients of per-stage vectors travel in fp32 (they are column sums)."""
    out, cursor = [], 0
    for name, mult, tp_sharded, per_token in spec:
        feat = mult * hidden // (tp if tp_sharded else 1)
        shape = (tokens, feat) if per_token else (feat,)
        dt = torch.float32 if (grads and not per_token) else dtype
        t = SlotTensor(name, shape, dt, cursor)
        out.append(t)
        cursor = _align(cursor + t.nbytes)
    return out, cursor


@dataclass(frozen=True)
class CopyOp:
    """One rectangle of one transfer, in bytes, relative to the source tensor and the receiver's slot."""
    name: str
    dst_rank: int
    src_offset: int        # from the source tensor's first element
    src_pitch: int
    dst_offset: int        # from the start of the receiver's slot
    dst_pitch: int
    width: int
    rows: int


class Direction:
    """One direction of one boundary as seen by one rank: what it sends where, what it waits for."""

    def __init__(self, rank: int, pieces: Sequence[Piece], spec, seq_len: int, hidden: int, dtype, grads: bool,
                 src_stage, dst_stage, micro_batch: int):
        self.rank, self.spec, self.grads = rank, tuple(spec), grads
        esize = {n: torch.empty((), dtype=(torch.float32 if (grads and not pt) else dtype)).element_size()
                 for n, _, _, pt in spec}
        feats = {n: (m, sharded) for n, m, sharded, _ in spec}
        src_tp, dst_tp = src_stage.tp_degree, dst_stage.tp_degree
        dst_tokens = micro_batch // dst_stage.dp_degree * seq_len
        self.dst_layout, self.slot_bytes = slot_layout(spec, dst_tokens, hidden, dst_tp, dtype, grads)
        at = {t.name: t for t in self.dst_layout}
        self.copies: List[CopyOp] = []
        for p in pieces:
            if p.src_rank != rank:
                continue
            mult, sharded = feats[p.name]
            e = esize[p.name]
            src_feat = mult * hidden // (src_tp if sharded else 1)
            dst_feat = mult * hidden // (dst_tp if sharded else 1)
            width = (p.src_cols[1] - p.src_cols[0]) * e
            if p.per_token:
                rows = (p.src_rows[1] - p.src_rows[0]) * seq_len
                src_off = (p.src_rows[0] * seq_len * src_feat + p.src_cols[0]) * e
                dst_off = at[p.name].offset + (p.dst_rows[0] * seq_len * dst_feat + p.dst_cols[0]) * e
            else:
                rows, src_off, dst_off = 1, p.src_cols[0] * e, at[p.name].offset + p.dst_cols[0] * e
            self.copies.append(CopyOp(p.name, p.dst_rank, src_off, src_feat * e, dst_off, dst_feat * e, width, rows))
        # flags: receiver d keeps one flag per rank that writes to it, in sorted rank order
        writers: Dict[int, List[int]] = {}
        for p in pieces:
            writers.setdefault(p.dst_rank, [])
            if p.src_rank not in writers[p.dst_rank]:
                writers[p.dst_rank].append(p.src_rank)
        self.writers = {d: sorted(w) for d, w in writers.items()}
        self.my_writers = self.writers.get(rank, [])                   # ranks I wait for as a receiver
        self.my_receivers = sorted({c.dst_rank for c in self.copies})  # ranks I post to as a sender
        if any(len(w) > 16 for w in self.writers.values()) or len(self.my_receivers) > 16:
            raise ValueError("a rank exchanges pipeline data with more than 16 peers")

    def flag_index_at(self, receiver: int) -> int:
        return self.writers[receiver].index(self.rank)


def inbox_bytes(direction: Optional[Direction], slots: int) -> int:
    return FLAG_BYTES + (slots * direction.slot_bytes if direction is not None else 0)


class PeerPipelineComm:
    """The calls the 1F1B schedule makes (`recv_forward`, `send_forward`, `recv_backward`,
    `send_backward`, and the two combined forms), over peer memory. Collective constructor: every
    rank of the world allocates its two inboxes, also ranks of single-stage pipelines."""

    def __init__(self, pstate, hidden: int, seq_len: int, in_spec, out_spec, dtype, device, world_ranks: Sequence[int],
                 slots: Optional[int] = None):
        import torch.distributed as dist
        from ..ops import native
        from .peer_memory import SymmetricBuffer
        self.pstate, self.device, self.dtype = pstate, torch.device(device), dtype
        self.lib, self.native = native.lib(), native
        self.slots = slots or (pstate.num_stages + 1)
        r, mbs = pstate.rank, pstate.micro_batch_size
        prev, nxt, me = pstate.neighbour(-1), pstate.neighbour(+1), pstate.stage
        mk = lambda pieces, spec, grads, a, b: Direction(r, pieces, spec, seq_len, hidden, dtype, grads, a, b, mbs)
        # as a receiver / as a sender, per direction
        self.fwd_in = mk(plan_transfers(prev, me, in_spec, mbs, hidden), in_spec, False, prev, me) if prev else None
        self.fwd_out = mk(plan_transfers(me, nxt, out_spec, mbs, hidden), out_spec, False, me, nxt) if nxt else None
        self.bwd_in = mk(plan_transfers(nxt, me, out_spec, mbs, hidden), out_spec, True, nxt, me) if nxt else None
        self.bwd_out = mk(plan_transfers(me, prev, in_spec, mbs, hidden), in_spec, True, me, prev) if prev else None
        self.in_spec, self.out_spec = tuple(in_spec), tuple(out_spec)
        # this rank's own view of its input tensors, as gradients (what `send_backward` ships)
        self.my_inputs, _ = slot_layout(in_spec, pstate.local_micro_batch * seq_len, hidden, pstate.tp_size, dtype, True)
        need = [inbox_bytes(self.fwd_in, self.slots), inbox_bytes(self.bwd_in, self.slots), self.slots]
        gathered = [None] * len(world_ranks)
        dist.all_gather_object(gathered, need)
        self.act_inbox = SymmetricBuffer(max(g[0] for g in gathered), tuple(world_ranks), r, None, device, holds_data=False)
        self.grad_inbox = SymmetricBuffer(max(g[1] for g in gathered), tuple(world_ranks), r, None, device, holds_data=False)
        self.index_of = {g: i for i, g in enumerate(world_ranks)}
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.sent = {"fwd": 0, "bwd": 0}
        self.received = {"fwd": 0, "bwd": 0}
        self._zeros: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ sending
    def _send(self, direction: Direction, inbox, tensors: Dict[str, torch.Tensor], key: str) -> None:
        seq = self.sent[key]
        self.sent[key] = seq + 1
        slot_base = FLAG_BYTES + (seq % self.slots) * direction.slot_bytes
        ready = torch.cuda.Event()
        ready.record()
        self.copy_stream.wait_event(ready)
        dev = self.device.index
        layout = {t.name: t for t in direction.dst_layout}
        with torch.cuda.stream(self.copy_stream):
            held = {}
            for c in direction.copies:
                t = held.get(c.name)
                if t is None:
                    t = tensors[c.name]
                    if t.dtype != layout[c.name].dtype:
                        t = t.to(layout[c.name].dtype)
                    if not t.is_contiguous():
                        t = t.contiguous()
                    held[c.name] = t
                dst = inbox.ptrs[self.index_of[c.dst_rank]] + slot_base + c.dst_offset
                self.lib.peer_copy_2d(dst, c.dst_pitch, t.data_ptr() + c.src_offset, c.src_pitch, c.width, c.rows, dev)
            flags = [inbox.ptrs[self.index_of[d]] + 4 * direction.flag_index_at(d) for d in direction.my_receivers]
            if flags:
                self.lib.flags_post(flags, seq + 1, dev)
            for t in held.values():
                t.record_stream(self.copy_stream)
        for t in tensors.values():
            if isinstance(t, torch.Tensor) and t.is_cuda:
                t.record_stream(self.copy_stream)

    # ------------------------------------------------------------------ receiving
    def _receive(self, direction: Direction, inbox, key: str) -> Dict[str, torch.Tensor]:
        seq = self.received[key]
        self.received[key] = seq + 1
        slot_base = FLAG_BYTES + (seq % self.slots) * direction.slot_bytes
        flags = [inbox.local_ptr + 4 * i for i in range(len(direction.my_writers))]
        self.lib.flags_wait(flags, seq + 1, WAIT_LIMITS, self.native.status(self.device))
        return {t.name: inbox.tensor(t.shape, t.dtype, slot_base + t.offset) for t in direction.dst_layout}

    # ------------------------------------------------------------------ the schedule's vocabulary
    def recv_forward(self):
        return self._receive(self.fwd_in, self.act_inbox, "fwd") if self.fwd_in is not None else None

    def send_forward(self, outputs):
        if self.fwd_out is not None:
            self._send(self.fwd_out, self.act_inbox, outputs, "fwd")

    def recv_backward(self):
        return self._receive(self.bwd_in, self.grad_inbox, "bwd") if self.bwd_in is not None else None

    def send_backward(self, grads):
        if self.bwd_out is not None:
            self._send(self.bwd_out, self.grad_inbox, self._complete(grads), "bwd")

    def send_forward_recv_backward(self, outputs):
        if self.fwd_out is None:
            return None
        self.send_forward(outputs)
        return self.recv_backward()

    def send_backward_recv_forward(self, grads):
        if self.bwd_out is None:
            return None
        self.send_backward(grads)
        return self.recv_forward()

    def _complete(self, grads):
        """A gradient the backward pass did not produce travels as zeros."""
        out = dict(grads)
        for t in self.my_inputs:
            if t.name not in out:
                if t.name not in self._zeros:
                    self._zeros[t.name] = torch.zeros(t.shape, dtype=t.dtype, device=self.device)
                out[t.name] = self._zeros[t.name]
        return out

    def close(self):
        self.act_inbox.close()
        self.grad_inbox.close()
