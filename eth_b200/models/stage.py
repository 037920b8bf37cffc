"""One pipeline stage of the GPT op graph: parameters, flat buffers, and the explicit
forward / backward interpreter with op-granular activation recomputation.

Memory layout (B200-first): every parameter of the stage is a view into ONE flat 16-bit buffer,
its persistent gradient (`main_grad`, the LocalDDP contract of
eth/runtime/megatron/model/distributed.py:68-123) a view into ONE flat gradient buffer, and the
fp32 master copy and Adam moments views into flat fp32 buffers with the same element order
(weight-decayed parameters first). The optimizer, the gradient norm and zeroing then are a
handful of launches over contiguous memory instead of one per tensor.

Recomputation follows the reference contract (model/flex_model.py:564-588): `recompute_ops` is a
0/1 list over the stage's ops; every maximal run of 1s (broken at `enc-1st-layernorm`) is executed
in forward without keeping its op contexts -- only the environment at the run's entry is kept --
and is re-executed right before its backward. Dropout masks are functions of (seed, offset), so the
replay is exact without capturing RNG state.
"""
from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .gpt_ops import (LIVE_AFTER, GPTModelConfig, Op, ParamSpec, TPComm, build_op_descriptors, init_full_tensor,
                      make_op, shard_of)


@dataclass
class ParamEntry:
    op: Op
    spec: ParamSpec
    param: torch.Tensor        # view into the flat parameter buffer (carries .main_grad)
    offset: int                # element offset inside the flat buffers
    numel: int
    tied_alias: bool = False   # second use of a tensor that already has an entry (same-stage tying)


class MicroBatch(SimpleNamespace):
    """Per-micro-batch record: index, local batch, seq, global_step, dp_rank, op contexts."""


def _align(n: int, a: int = 128) -> int:
    return (n + a - 1) // a * a


class GPTStage:
    """`chunks`: for interleaved pipelining a rank owns several op ranges (model chunks) that are
    not adjacent in the model; they share the flat buffers and are executed one chunk at a time
    (`forward(..., chunk=c)`). Without it the stage is the single range [op_begin, op_end)."""

    def __init__(self, cfg: GPTModelConfig, op_begin: int, op_end: int, tp: Optional[TPComm] = None,
                 device="cpu", recompute_ops: Optional[Sequence[int]] = None, fuse: bool = True,
                 chunks: Optional[Sequence[Tuple[int, int]]] = None, algo_ops: Optional[Sequence[int]] = None):
        self.cfg = cfg
        self.tp = tp or TPComm()
        self.device = torch.device(device)
        self.descriptors = build_op_descriptors(cfg.num_layers, getattr(cfg, "model_impl", "gpt"))
        self.chunk_ranges: List[Tuple[int, int]] = [tuple(c) for c in chunks] if chunks else [(op_begin, op_end)]
        self.op_begin, self.op_end = self.chunk_ranges[0][0], self.chunk_ranges[-1][1]
        self.ops: List[Op] = []
        self._chunk_slices: List[Tuple[int, int]] = []      # index range of every chunk inside self.ops
        n_ops = sum(e - b for b, e in self.chunk_ranges)
        algos = list(algo_ops) if algo_ops is not None else [0] * n_ops
        if len(algos) != n_ops:
            raise ValueError("algo_ops length must equal the stage's op count")
        for b, e in self.chunk_ranges:
            start = len(self.ops)
            self.ops += [make_op(d, cfg, self.tp, algos[start + k]) for k, d in enumerate(self.descriptors[b:e])]
            self._chunk_slices.append((start, len(self.ops)))
        self.is_first = self.chunk_ranges[0][0] == 0
        self.is_last = self.chunk_ranges[-1][1] == len(self.descriptors)
        self.recompute = list(recompute_ops) if recompute_ops is not None else [0] * len(self.ops)
        if len(self.recompute) != len(self.ops):
            raise ValueError("recompute_ops length must equal the stage's op count")
        self._build_params()
        if fuse:
            self._mark_fusions()
        self._segments_by_chunk = [self._plan_segments(a, z) for a, z in self._chunk_slices]
        self._segments = self._segments_by_chunk[0]
        self._contexts: Dict[object, dict] = {}
        # called with the global op index after every op's backward (the engine sets it for the last
        # micro-batch of an iteration to start gradient reductions while backward is still running)
        self.after_op_backward = None
        self.op_events = None   # set to a list to record (op name, phase, start event, end event)
        self.chunk_specs = []         # per chunk: (tensors entering it, tensors leaving it)
        for b, e in self.chunk_ranges:
            prev = self.descriptors[b - 1]["name"] if b > 0 else None
            spec_in = LIVE_AFTER[prev] if prev else ()
            spec_out = LIVE_AFTER[self.descriptors[e - 1]["name"]]
            if spec_in is None or spec_out is None:
                raise ValueError("a stage boundary may not fall inside the unfused attention block "
                                 "(enc-attention-score .. enc-attention-context)")
            self.chunk_specs.append((spec_in, spec_out))
        self.input_spec, self.output_spec = self.chunk_specs[0][0], self.chunk_specs[-1][1]

    # ------------------------------------------------------------------ parameters
    def _build_params(self):
        cfg, tp = self.cfg, self.tp
        entries: List[Tuple[Op, ParamSpec]] = [(op, s) for op in self.ops for s in op.specs()]
        # a tied parameter that appears twice in one stage gets one storage
        uniq: List[Tuple[Op, ParamSpec]] = []
        seen: Dict[str, int] = {}
        alias: List[Tuple[Op, ParamSpec, int]] = []
        for op, s in entries:
            if s.logical_id in seen:
                alias.append((op, s, seen[s.logical_id]))
            else:
                seen[s.logical_id] = len(uniq)
                uniq.append((op, s))
        order = sorted(range(len(uniq)), key=lambda i: (0 if uniq[i][1].weight_decay else 1, i))
        offsets, cursor = {}, 0
        self.decay_numel = 0
        for i in order:
            n = 1
            for d in uniq[i][1].local_shape(tp.size):
                n *= d
            offsets[i] = (cursor, n)
            cursor += _align(n)
            if uniq[i][1].weight_decay:
                self.decay_numel = cursor   # decayed parameters come first, so this ends their region
        total = max(cursor, 1)
        dev = self.device
        self.param_buf = torch.zeros(total, dtype=cfg.params_dtype, device=dev)
        self.grad_buf = torch.zeros(total, dtype=cfg.grad_dtype, device=dev)
        self.total_numel = total
        self.entries: List[ParamEntry] = []
        by_uniq: Dict[int, ParamEntry] = {}
        for i, (op, spec) in enumerate(uniq):
            off, n = offsets[i]
            shape = spec.local_shape(tp.size)
            p = self.param_buf[off:off + n].view(shape)
            full = init_full_tensor(spec, cfg, dev)
            p.copy_(shard_of(full, spec, tp.size, tp.rank).to(cfg.params_dtype))
            del full
            p.main_grad = self.grad_buf[off:off + n].view(shape)
            p.requires_grad = False
            op.params[spec.local_name] = p
            e = ParamEntry(op, spec, p, off, n)
            self.entries.append(e)
            by_uniq[i] = e
        for op, spec, i in alias:
            op.params[spec.local_name] = by_uniq[i].param
            self.entries.append(ParamEntry(op, spec, by_uniq[i].param, by_uniq[i].offset, by_uniq[i].numel, True))

    def rebind_grad_buffer(self, buf: torch.Tensor) -> None:
        """Move the flat gradient buffer into `buf` (same numel and dtype, e.g. a symmetric
        allocation that peers can address) and re-create every parameter's `main_grad` view."""
        if buf.numel() != self.grad_buf.numel() or buf.dtype != self.grad_buf.dtype:
            raise ValueError("replacement gradient buffer must match the flat buffer's size and dtype")
        buf.copy_(self.grad_buf)
        self.grad_buf = buf
        for e in self.entries:
            e.param.main_grad = buf[e.offset:e.offset + e.numel].view(e.param.shape)

    def unique_entries(self) -> List[ParamEntry]:
        return [e for e in self.entries if not e.tied_alias]

    def named_parameters(self):
        for e in self.unique_entries():
            yield e.spec.logical_id, e.param

    def zero_grad_buffer(self):
        self.grad_buf.zero_()

    def _mark_fusions(self):
        for start, end in self._chunk_slices:       # never across a chunk boundary
            ops = self.ops[start:end]
            for a, b in zip(ops, ops[1:]):
                # the GeLU epilogues belong to the usual sharding: with algo 1 the bias is added after a
                # reduction (GEMM-1) and the data gradient is reduced before it is cut (GEMM-2)
                if a.name == "enc-MLP-GEMM-1" and b.name == "enc-MLP-gelu" and a.algo == 0:
                    a.fuse_next = True
                if a.name == "enc-MLP-gelu" and b.name == "enc-MLP-GEMM-2" and b.algo == 0:
                    b.fuse_prev = True
                # bias-dropout-add in the epilogue of the row-parallel GEMM that feeds it
                if (a.name in ("enc-attention-dense", "enc-MLP-GEMM-2") and a.algo == 0
                        and b.name in ("enc-post-attention-dropout", "enc-post-MLP-dropout")):
                    a.fused_dropout_add = b

    # ------------------------------------------------------------------ recompute segments
    def _plan_segments(self, start: int = 0, end: Optional[int] = None) -> List[Tuple[int, int, bool]]:
        """Maximal runs [i, j) of equal recompute flag inside ops[start:end]; recompute runs break at
        enc-1st-layernorm."""
        segs, i, n = [], start, len(self.ops) if end is None else end
        while i < n:
            flag = bool(self.recompute[i])
            j = i + 1
            while j < n and bool(self.recompute[j]) == flag and not (flag and self.ops[j].name == "enc-1st-layernorm"):
                j += 1
            segs.append((i, j, flag))
            i = j
        return segs

    # ------------------------------------------------------------------ execution
    def _run(self, op, phase, fn, *a):
        """Run one op step; when `op_events` is a list, bracket it with CUDA events."""
        if self.op_events is None:
            return fn(*a)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = fn(*a)
        e.record()
        self.op_events.append((op.name, phase, s, e))
        return out

    def op_time_table(self):
        """{(op name, phase): total ms} from the recorded events (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for name, phase, s, e in self.op_events or []:
            out[(name, phase)] = out.get((name, phase), 0.0) + s.elapsed_time(e)
        return out

    def _key(self, mb_index: int, chunk: int):
        return mb_index if len(self.chunk_ranges) == 1 else (mb_index, chunk)

    def forward(self, mb: MicroBatch, inputs: Dict[str, torch.Tensor], chunk: int = 0) -> Dict[str, torch.Tensor]:
        env = dict(inputs)
        ctxs: Dict[int, dict] = {}
        mb.ctxs = ctxs
        saved_envs: Dict[int, dict] = {}
        for (i, j, recompute) in self._segments_by_chunk[chunk]:
            if recompute:
                # tensors that live in a short-lived ring slot must be copied to survive until backward
                saved_envs[i] = {k: (v.clone() if getattr(v, "_ethb_ring", False) else v) for k, v in env.items()}
                scratch: Dict[int, dict] = {}
                mb.ctxs = scratch
                for op in self.ops[i:j]:
                    scratch[op.op_index] = {}
                    self._run(op, "fwd", op.fwd, env, scratch[op.op_index], mb)
                mb.ctxs = ctxs
            else:
                for op in self.ops[i:j]:
                    ctxs[op.op_index] = {}
                    self._run(op, "fwd", op.fwd, env, ctxs[op.op_index], mb)
        self._contexts[self._key(mb.index, chunk)] = {"ctxs": ctxs, "envs": saved_envs, "mb": mb}
        last_chunk = chunk == len(self.chunk_ranges) - 1
        keep = {name for name, *_ in self.chunk_specs[chunk][1]} | ({"output"} if (self.is_last and last_chunk) else set())
        # a tensor that lives in a short-lived ring slot is copied: what leaves the stage is read later,
        # by a transfer on another stream
        return {k: (v.clone() if getattr(v, "_ethb_ring", False) else v) for k, v in env.items() if k in keep}

    def context_of(self, mb_index: int, chunk: int = 0) -> dict:
        return self._contexts[self._key(mb_index, chunk)]

    def backward(self, mb_index: int, grad_outputs: Dict[str, torch.Tensor], chunk: int = 0) -> Dict[str, torch.Tensor]:
        rec = self._contexts.pop(self._key(mb_index, chunk))
        ctxs, saved_envs, mb = rec["ctxs"], rec["envs"], rec["mb"]
        mb.ctxs = ctxs
        genv = dict(grad_outputs)
        for (i, j, recompute) in reversed(self._segments_by_chunk[chunk]):
            if recompute:
                env = saved_envs.pop(i)
                for op in self.ops[i:j]:
                    ctxs[op.op_index] = {}
                    self._run(op, "refwd", op.fwd, env, ctxs[op.op_index], mb)
            for op in reversed(self.ops[i:j]):
                self._run(op, "bwd", op.bwd, genv, ctxs.pop(op.op_index), mb)
                if self.after_op_backward is not None:
                    self.after_op_backward(op.op_index)
        keep = {name for name, *_ in self.chunk_specs[chunk][0]}
        return {k: v for k, v in genv.items() if k in keep and isinstance(v, torch.Tensor)}

    def drop_context(self, mb_index: int, chunk: int = 0) -> None:
        self._contexts.pop(self._key(mb_index, chunk), None)

    # ------------------------------------------------------------------ boundary shapes
    def boundary_shapes(self, spec, tokens: int) -> Dict[str, Tuple[int, ...]]:
        out = {}
        h = self.cfg.hidden_size
        for name, mult, tp_sharded, per_token in spec:
            feat = mult * h // (self.tp.size if tp_sharded else 1)
            out[name] = (tokens, feat) if per_token else (feat,)
        return out


def build_full_model(cfg: GPTModelConfig, device="cpu", tp: Optional[TPComm] = None, **kw) -> GPTStage:
    """The whole op list as a single stage (PP = 1)."""
    per_layer = 13 if getattr(cfg, "model_impl", "gpt") == "gpt-legacy13" else 10
    return GPTStage(cfg, 0, 3 + per_layer * cfg.num_layers, tp=tp, device=device, **kw)
