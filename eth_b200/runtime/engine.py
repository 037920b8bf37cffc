"""Training engine of one rank: stage program, pipeline schedule, loss contract, canonical
gradient sync and the optimizer step.

One iteration (reference call stack: eth/runtime/megatron/training.py:904-1034):
    zero the gradient buffer
    forward/backward over this pipeline's micro-batches (no-pipeline or 1F1B schedule)
    all-reduce [loss_sum, loss_weight] over the world  -> normalisation = nominal / weight
    canonical gradient sync (bucketed reductions across pipelines and DP replicas)
    optimizer: norm + overflow agreement over the world, clip, AdamW, refresh 16-bit weights
    learning-rate schedule and clock advance on success
The normalisation and the loss scale never go through the host: they are folded into one device
scalar that the optimizer kernels read.
"""
from __future__ import annotations

import os
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.gpt_ops import GPTModelConfig, TPComm
from ..models.stage import GPTStage, MicroBatch
from ..ops import raw as raw_ops
from ..optim.grad_scaler import ConstantGradScaler, DynamicGradScaler
from ..optim.lr import AnnealingLR
from ..optim.optimizer import FlatMixedPrecisionAdam, coalesce_ranges
from ..parallel.grad_sync.gpt_adapter import collect_gpt_gradient_metadata
from ..parallel.grad_sync.loss import SampleSchedule, TrainingClock, synthetic_gpt_batch
from ..parallel.grad_sync.manager import dump_gradient_sync_plan, initialize_gradient_sync
from ..parallel.p2p import PipelineComm
from ..parallel.state import ParallelState
from . import schedules
from .timers import Timers


class _SingleRank:
    """Stand-in for the process group of a single rank (collectives over it are no-ops)."""

    def __repr__(self):
        return "<single-rank group>"


SINGLE = _SingleRank()


class Collectives:
    """torch.distributed calls used by the engine, gathered in one place so tests can fake them.
    `group=None` means the world; groups of one rank are the `SINGLE` sentinel."""

    def __init__(self, world_size: int):
        self.world_size = world_size
        self.enabled = world_size > 1 and dist.is_available() and dist.is_initialized()

    def create_group(self, ranks):
        if len(ranks) <= 1:
            return SINGLE
        return dist.new_group(list(ranks)) if self.enabled else None

    def all_reduce_sum(self, t, group=None):
        if self.enabled and group is not SINGLE:
            dist.all_reduce(t, group=group)

    def all_reduce_max(self, t, group=None):
        if self.enabled and group is not SINGLE:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)

    def all_gather_object(self, out_list, obj, group=None):
        if self.enabled and group is not SINGLE:
            dist.all_gather_object(out_list, obj, group=group)
        else:
            out_list[0] = obj

    def broadcast(self, t, src, group=None):
        if self.enabled and group is not SINGLE:
            dist.broadcast(t, src, group=group)

    def barrier(self):
        if self.enabled:
            dist.barrier()


class TrainEngine:
    def __init__(self, args, device=None, collectives: Optional[Collectives] = None,
                 data_provider: Optional[Callable] = None):
        self.args = args
        self.device = torch.device(device if device is not None else
                                   ("cuda:%d" % torch.cuda.current_device() if torch.cuda.is_available() else "cpu"))
        self.coll = collectives or Collectives(args.world_size)
        self.timers = Timers()
        cfg = args.normalized_config
        self.pstate = ParallelState(cfg, args.rank, self.coll.create_group, topology=args.canonical_topology,
                                    interleave=getattr(args, "interleave_factor", 1))
        ps = self.pstate
        self.model_cfg = GPTModelConfig(
            num_layers=cfg["num_layers"], hidden_size=cfg["hidden_size"],
            num_attention_heads=cfg["num_attention_heads"], seq_length=cfg["seq_length"],
            max_position_embeddings=cfg.get("max_position_embeddings", cfg["seq_length"]),
            padded_vocab_size=args.padded_vocab_size, hidden_dropout=args.hidden_dropout,
            layernorm_epsilon=args.layernorm_epsilon, init_method_std=args.init_method_std,
            params_dtype=args.params_dtype, grad_dtype=args.grad_dtype, seed=args.seed,
            canonical_init=getattr(args, "grad_sync_evidence_canonical_init", False),
            zero_labels=getattr(args, "reference_zero_labels", False),
            model_impl=cfg.get("model_impl", "gpt"), attention_dropout=getattr(args, "attention_dropout", 0.0) or 0.0)
        self.tp = self._make_tp_comm()
        begin, end = ps.op_range
        chunks = ps.chunk_ranges if ps.interleave > 1 else None
        algo_ops = list(ps.pipe["algo_of_each_op"][ps.stage_id])
        if any(algo_ops) and ps.tp_size > 1 and not ps.pipe["resharding_stages"][ps.stage_id]:
            raise ValueError(f"pipeline {ps.pipeline_id} stage {ps.stage_id} asks for algo 1 (the swapped sharding of the "
                             "tensor-parallel GEMMs), which converts placements inside the stage: set "
                             "resharding_stages to true for it")
        self.stage = GPTStage(self.model_cfg, begin, end, tp=self.tp, device=self.device,
                              recompute_ops=ps.recompute_ops, chunks=chunks, algo_ops=algo_ops)
        self.seq_len = cfg["seq_length"]
        self.comm = PipelineComm(ps, cfg["hidden_size"], self.seq_len, self.stage.input_spec, self.stage.output_spec,
                                 args.params_dtype, self.device) if ps.num_stages > 1 else None
        # forward-only passes always use the NCCL channels; training may move to peer memory below
        self.eval_comm = self.comm
        self.p2p_backend = "nccl" if self.comm is not None else None
        self._setup_peer_p2p(cfg)
        # interleaved pipelining: one set of channels per model chunk, wired to the stage that holds
        # the previous / next virtual stage
        self.chunk_comms = None
        if ps.interleave > 1:
            self.chunk_comms = [
                PipelineComm(ps, cfg["hidden_size"], self.seq_len, spec_in, spec_out, args.params_dtype, self.device,
                             neighbours=(ps.chunk_neighbour(c, -1), ps.chunk_neighbour(c, +1)))
                for c, (spec_in, spec_out) in enumerate(self.stage.chunk_specs)]
        self.data_provider = data_provider
        self.eval_data_provider = None   # batches of eval_step; None = the training provider
        self.eval_cursor = 0             # position in the validation data (advanced by the evaluation loop)
        self.clock = TrainingClock(total_gbs=args.total_gbs)
        self.iteration = 0
        self._setup_grad_sync()
        self._setup_optimizer()
        evidence = getattr(args, "grad_sync_evidence_dir", None) or getattr(args, "grad_sync_runtime_evidence_dir", None)
        raw_ops.enable_async_wgrad(self.device, on=getattr(args, "async_wgrad", True) and not evidence)
        self.loss_acc = torch.zeros(2, dtype=torch.float32, device=self.device)
        self._gs_pairs = []
        self._sample_schedule = None
        self._defer_colsums = None   # decided at the first micro-batch (see _colsum_mode)
        self.last_stats: Dict[str, object] = {}

    # ------------------------------------------------------------------ set-up
    def _make_tp_comm(self) -> TPComm:
        ps = self.pstate
        if ps.tp_size == 1:
            return TPComm()
        backend = None
        mode = getattr(self.args, "tp_comm", "auto")
        if mode in ("auto", "fused") and self.device.type == "cuda":
            try:
                from ..parallel.fused_tp import FusedTPBackend
                backend = FusedTPBackend.create(ps, self.coll, self.device, self.args)
            except Exception as err:
                if mode == "fused":
                    raise
                # said once per rank: a broken peer-memory set-up must not pass as a slower number
                print(f"[rank {self.args.rank}] fused tensor-parallel kernels unavailable, using GEMM + NCCL "
                      f"all-reduce instead: {type(err).__name__}: {err}", flush=True)
                backend = None
        return TPComm(ps.tp_size, ps.tp_rank, ps.tp_group, backend)

    def _setup_grad_sync(self):
        args, ps = self.args, self.pstate
        topo = ps.topology
        peer_factory = None
        self._grad_symm = None
        backend = getattr(args, "grad_sync_backend", "auto")
        one_node = int(os.environ.get("LOCAL_WORLD_SIZE", args.world_size)) == args.world_size
        use_peer = backend in ("auto", "peer") and self.device.type == "cuda" and self.coll.enabled and one_node
        if use_peer:
            # Every rank takes this branch together (it depends on global facts only): the flat
            # gradient buffer moves into a symmetric allocation so peers can reduce it in place.
            # This comes before the gradient metadata is collected, which records `main_grad` views.
            from ..parallel.peer_memory import SymmetricBuffer
            gb = self.stage.grad_buf
            self._grad_symm = SymmetricBuffer(gb.numel() * gb.element_size(), tuple(range(args.world_size)),
                                              args.rank, None, self.device)
            self.stage.rebind_grad_buffer(self._grad_symm.tensor((gb.numel(),), gb.dtype))
        descriptors, bindings = collect_gpt_gradient_metadata(self.stage, ps, args.normalized_config)
        self.descriptors, self.bindings = descriptors, bindings
        if use_peer:
            evidence = bool(getattr(args, "grad_sync_runtime_evidence_dir", None))

            def peer_factory(plan, rank):
                from ..parallel.grad_sync.peer_backend import PeerReduceBackend
                if not any(1 < len(g.ranks) <= 8 for g in plan.process_groups):
                    return None     # no group the peer kernel would serve: plain scratch + collectives
                be = PeerReduceBackend(plan, rank, self.coll, self.device, max_group=8,
                                       grad_symm=self._grad_symm, grad_buf=self.stage.grad_buf)
                be.force_packed = evidence
                return be
        elif backend == "peer":
            raise RuntimeError("--grad-sync-backend peer needs CUDA ranks that all share one node")

        def group_gather(out, obj, handle):
            self.coll.all_gather_object(out, obj, group=handle)

        self.grad_sync = initialize_gradient_sync(
            local_descriptors=descriptors, local_runtime_bindings=bindings, topology=topo,
            model_impl=args.normalized_config["model_impl"], manifest_hash=args.manifest_hash,
            sync_mode=args.grad_sync_mode, bucket_cap_bytes=args.grad_sync_bucket_size_mb * 1024 * 1024,
            global_rank=args.rank, all_gather_object=lambda out, obj: self.coll.all_gather_object(out, obj),
            all_gather_group_object=group_gather, create_group=self.coll.create_group,
            all_reduce_sum=lambda t, handle: self.coll.all_reduce_sum(t, group=handle),
            control_device=self.device, runtime_evidence_dir=args.grad_sync_runtime_evidence_dir,
            peer_backend_factory=peer_factory)
        if args.grad_sync_dump_plan and args.rank == 0:
            dump_gradient_sync_plan(self.grad_sync.plan, args.grad_sync_dump_plan)
        # parameters of one logical fragment start equal on all holders
        self.grad_sync.synchronize_parameters(lambda t, src, handle: self.coll.broadcast(t, src, group=handle))
        groups = {g.process_group_id: g for g in self.grad_sync.plan.process_groups}
        self._needs_reduction = any(len(groups[b.process_group_id].ranks) > 1 for b in self.grad_sync.executor.buckets)
        self._setup_grad_overlap()

    # ------------------------------------------------------------------ gradient sync overlapped with backward
    def _setup_grad_overlap(self):
        """Buckets whose reduction runs on a side stream as soon as the last micro-batch's backward
        has passed their first op (reference: strictly after backward, grad_sync/executor.py:199-261).
        Only buckets served by the peer-memory backend take part: a library collective launched from
        a second stream could interleave differently with the main stream's collectives on other
        ranks. The peer backend's kernels never spin while they occupy an SM's worth of resources
        (waiting is left to a one-warp kernel), so an early rank cannot starve the persistent GEMMs
        of its own stage or, through a fused tensor-parallel GEMM, of its partner's."""
        a, ex = self.args, self.grad_sync.executor
        self._overlap_by_op, self._overlap_done = {}, set()
        self._sync_stream = None
        if (not getattr(a, "overlap_grad_sync", True) or self.device.type != "cuda"
                or getattr(a, "grad_sync_evidence_dir", None) or getattr(a, "grad_sync_runtime_evidence_dir", None)):
            return
        for b in ex.buckets:
            if ex.needs_reduction(b) and ex.uses_peer_backend(b):
                self._overlap_by_op.setdefault(ex.bucket_first_op(b), []).append(b)
        if self._overlap_by_op:
            self._sync_stream = torch.cuda.Stream(device=self.device)

    def _reduce_ready_buckets(self, op_index: Optional[int]) -> None:
        """Start the peer reduction of the buckets whose first op is `op_index` (None: of all buckets
        not started yet) on the sync stream, behind everything enqueued so far."""
        if op_index is None:
            # plan order: the same on every rank of a group, whatever ops the rank holds
            buckets = sorted((b for bs in self._overlap_by_op.values() for b in bs
                              if b.bucket_id not in self._overlap_done), key=lambda b: b.bucket_id)
        else:
            buckets = self._overlap_by_op.get(op_index)
        if not buckets:
            return
        ready = torch.cuda.Event()
        ready.record()
        self._sync_stream.wait_event(ready)
        # the weight gradients of these ops were enqueued on the side stream: wait for them too
        wgrad_done = raw_ops.async_wgrad_event(self.device)
        if wgrad_done is not None:
            self._sync_stream.wait_event(wgrad_done)
        with torch.cuda.stream(self._sync_stream):
            for b in buckets:
                self.grad_sync.executor.execute_bucket(b, 1.0)
                self._overlap_done.add(b.bucket_id)

    def _owned_ranges(self):
        """(offset, numel) ranges of the flat gradient buffer whose norm this rank is responsible for."""
        sem = self.grad_sync.optimizer_semantics
        base = self.stage.grad_buf.data_ptr()
        esize = self.stage.grad_buf.element_size()
        ranges = []
        for v in sem.owned_gradient_views():
            if v.is_contiguous():
                ranges.append(((v.data_ptr() - base) // esize, v.numel()))
            else:
                # a column slice of a row-parallel weight: one range per row
                flat = v.reshape(-1, v.shape[-1]) if v.dim() > 2 else v
                for r in range(flat.shape[0]):
                    row = flat[r]
                    ranges.append(((row.data_ptr() - base) // esize, row.numel()))
        return coalesce_ranges(ranges)

    def _setup_optimizer(self):
        a = self.args
        if a.fp16:
            if a.loss_scale:
                self.scaler = ConstantGradScaler(a.loss_scale, self.device)
            else:
                self.scaler = DynamicGradScaler(a.initial_loss_scale, a.min_loss_scale, 2.0, 0.5,
                                                int(a.loss_scale_window), a.hysteresis, self.device)
        else:
            self.scaler = None
        world_ar = (lambda t: self.coll.all_reduce_sum(t)) if self.coll.enabled else None
        self.optimizer = FlatMixedPrecisionAdam(
            self.stage, lr=a.lr, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_eps, weight_decay=a.weight_decay,
            clip_grad=a.clip_grad, grad_scaler=self.scaler, owned_ranges=self._owned_ranges(),
            world_all_reduce=world_ar)
        decay_samples = a.lr_decay_iters * a.total_gbs
        self.lr_scheduler = AnnealingLR(self.optimizer, a.lr, a.min_lr, a.lr_warmup_samples, decay_samples,
                                        a.lr_decay_style, a.use_checkpoint_lr_scheduler, a.override_lr_scheduler)

    # ------------------------------------------------------------------ data
    def _sample_ids(self, mb_index: int):
        a, ps = self.args, self.pstate
        if self._sample_schedule is None:
            self._sample_schedule = SampleSchedule(a.mbs_seq, a.pipeline_sample_offsets)
        return self._sample_schedule.slots(ps.pipeline_id, mb_index, ps.dp_size, ps.dp_rank,
                                           self.clock.global_data_cursor)

    def get_batch(self, mb_index: int):
        ids = self._sample_ids(mb_index)
        seq = self.args.mbs_seq[self.pstate.pipeline_id][mb_index][1]
        if self.data_provider is not None:
            return self.data_provider(ids, seq, self.device)
        tokens, mask, _pos, _attn, labels = synthetic_gpt_batch(ids, seq, self.args.vocab_size, self.device,
                                                                with_labels=True)
        if self.model_cfg.zero_labels:
            labels = torch.zeros_like(labels)
        return tokens, labels, mask

    # ------------------------------------------------------------------ steps used by the schedules
    def forward_step(self, mb_index: int, inputs: Optional[Dict[str, torch.Tensor]], chunk: int = 0):
        ps = self.pstate
        seq = self.args.mbs_seq[ps.pipeline_id][mb_index][1]
        mb = MicroBatch(index=mb_index, batch=ps.local_micro_batch, seq=seq, global_step=self.iteration,
                        dp_rank=ps.dp_rank, colsum_mode=self._colsum_mode(mb_index))
        env = dict(inputs) if inputs else {}
        first, last = ps.is_first_virtual(chunk), ps.is_last_virtual(chunk)
        if first or last:
            tokens, labels, mask = self.get_batch(mb_index)
            if first:
                env["enc_input_ids"] = tokens
            if last:
                env["labels"] = labels
                mb.loss_mask = mask.reshape(-1)
        out = self.stage.forward(mb, env, chunk)
        if last:
            losses = out.pop("output")
            if ps.tp_rank == 0:   # TP peers hold identical losses; count them once
                self.loss_acc[0] += torch.dot(losses, mb.loss_mask)
                self.loss_acc[1] += mb.loss_mask.sum()
        return out

    def _colsum_mode(self, mb_index: int) -> int:
        """Column-sum gradients (LayerNorm weights, biases behind a dropout) are summed once per step,
        with the backward of the last micro-batch, when every micro-batch has the same shape: each
        op sees its micro-batches in index order under all three schedules."""
        if self._defer_colsums is None:
            seqs = {int(entry[1]) for entry in self.args.mbs_seq[self.pstate.pipeline_id]}
            self._defer_colsums = (self.device.type == "cuda" and len(seqs) == 1
                                   and not getattr(self.args, "no_deferred_colsums", False))
        if not self._defer_colsums:
            return raw_ops.WS_IMMEDIATE
        return raw_ops.WS_FLUSH if mb_index == self.pstate.num_microbatches - 1 else raw_ops.WS_ACCUMULATE

    def backward_step(self, mb_index: int, grad_outputs: Optional[Dict[str, torch.Tensor]], chunk: int = 0):
        ps = self.pstate
        if ps.is_last_virtual(chunk):
            rec = self.stage.context_of(mb_index, chunk)["mb"]
            scale = self.scaler.value() if self.scaler is not None else 1.0
            grad_outputs = {"output": rec.loss_mask * (scale / self.args.nominal_global_loss_scale)}
        # Start reductions during the very last backward of the iteration -- without pipeline stages only.
        # A reduction begins with a wait for the group's peers. The tied embedding's group spans the
        # first and the last stage, and the first stage cannot arrive before it has received the last
        # gradient from downstream, which this rank sends after this backward: a wait enqueued now
        # could sit in front of that send (streams may share a hardware queue) and close a cycle
        # that only the wait limit breaks. With stages, reductions start after the schedule instead
        # (`train_step`), when every send of the iteration has been enqueued.
        last = (self._sync_stream is not None and mb_index == self.pstate.num_microbatches - 1 and ps.interleave == 1
                and ps.num_stages == 1)
        if last:
            self.stage.after_op_backward = self._reduce_ready_buckets
        try:
            return self.stage.backward(mb_index, grad_outputs or {}, chunk)
        finally:
            if last:
                self.stage.after_op_backward = None

    def _setup_peer_p2p(self, cfg) -> None:
        """Pipeline transfers of the 1F1B schedule through peer memory (`parallel/peer_p2p.py`) when
        the whole job sits in one NVLink domain. The decision is the same on every rank (the inboxes
        are allocated collectively), also on ranks whose pipeline has a single stage."""
        a, ps = self.args, self.pstate
        want = getattr(a, "p2p_backend", "auto")
        multi_stage = any(p["num_stages"] > 1 for p in cfg["pipe"])
        one_node = int(os.environ.get("LOCAL_WORLD_SIZE", a.world_size)) == a.world_size
        usable = (self.device.type == "cuda" and a.world_size > 1 and multi_stage and one_node and ps.interleave == 1
                  and a.world_size <= 8)
        if want == "nccl" or not usable:
            if want == "peer":
                raise RuntimeError("--p2p-backend peer needs CUDA ranks of one node, a pipeline with several stages "
                                   "and no interleaving")
            return
        from ..parallel.peer_p2p import PeerPipelineComm
        try:
            peer = PeerPipelineComm(ps, cfg["hidden_size"], self.seq_len, self.stage.input_spec, self.stage.output_spec,
                                    a.params_dtype, self.device, tuple(range(a.world_size)))
        except Exception as err:
            if want == "peer":
                raise
            print(f"[eth_b200] rank {a.rank}: peer-memory pipeline transfers unavailable ({err}); using NCCL",
                  flush=True)
            return
        if ps.num_stages > 1:
            self.comm, self.p2p_backend = peer, "peer"
        self._peer_p2p = peer

    # ------------------------------------------------------------------ one iteration
    def train_step(self, sync: Optional[bool] = None) -> Dict[str, object]:
        a = self.args
        if sync is None:
            sync = not getattr(a, "async_optimizer", False)
        evidence_dir = getattr(a, "grad_sync_evidence_dir", None)
        if evidence_dir and self.iteration == 0:
            self._evidence("init", evidence_dir)
        self.optimizer.zero_grad()
        self.loss_acc.zero_()
        n_mb = self.pstate.num_microbatches
        if self.pstate.num_stages == 1:
            schedules.forward_backward_no_pipelining(self, n_mb)
        elif self.pstate.interleave > 1:
            schedules.forward_backward_interleaved(self, n_mb)
        else:
            schedules.forward_backward_1f1b(self, n_mb)
            if self._sync_stream is not None:
                # later stages finish their last backward while earlier ones still drain the pipeline:
                # their reductions run beside that
                self._reduce_ready_buckets(None)
        raw_ops.join_async_wgrad(self.device)
        # global loss weight -> normalisation factor (device scalar)
        local_weight = float(self.loss_acc[1]) if evidence_dir else None
        self.coll.all_reduce_sum(self.loss_acc)
        normalization = a.nominal_global_loss_scale / self.loss_acc[1]
        if evidence_dir:
            self._evidence("pre_sync", evidence_dir, local_loss_weight=local_weight,
                           global_loss_weight=float(self.loss_acc[1]), normalization_scale=float(normalization))
        if self._needs_reduction:
            gs = self._grad_sync_events()
            if gs:
                gs[0].record()
            if self._sync_stream is not None:
                torch.cuda.current_stream().wait_stream(self._sync_stream)
            self.grad_sync.executor.execute(1.0, skip=self._overlap_done)
            self._overlap_done = set()
            if gs:
                gs[1].record()
        self.optimizer.set_grad_factor(normalization)
        if evidence_dir:
            self._evidence("post_sync", evidence_dir, grad_factor=float(self.optimizer.ctrl[2]))
        ok, grad_norm, _ = self.optimizer.step(sync=sync)
        if getattr(self.optimizer, "last_device_fault", False):
            # every rank sees the mark (it travels with the overflow flag), so all of them stop here
            # before a checkpoint could be written from stale data
            from ..ops import native
            detail = ""
            try:
                native.check_status(self.device)
            except RuntimeError as err:
                detail = f" (this rank: {err})"
            raise RuntimeError("a bounded device wait ran out on some rank during this iteration; the update was "
                               f"skipped on every rank{detail}")
        increment = self.clock.after_attempt(ok)
        if ok:
            self.lr_scheduler.step(increment)
        if evidence_dir:   # after the clock moved: the snapshot's clock is the state the next iteration starts from
            clip = min(1.0, a.clip_grad / (grad_norm + 1.0e-6)) if (ok and grad_norm is not None and a.clip_grad > 0) else 1.0
            self._evidence("post_step", evidence_dir, update_successful=bool(ok), grad_norm=grad_norm,
                           clip_coefficient=clip)
        self.iteration += 1
        stats = {"iteration": self.iteration, "update_successful": ok, "grad_norm": grad_norm,
                 "loss_scale": self.scaler.value() if self.scaler is not None else 1.0, "lr": self.optimizer.lr,
                 "loss_acc": self.loss_acc}
        self.last_stats = stats
        return stats

    # ------------------------------------------------------------------ exposed gradient-sync time
    def _grad_sync_events(self):
        """A fresh CUDA event pair for this iteration's post-backward gradient sync, or None on CPU.
        The pair brackets what the main stream spends on gradient reduction after the last backward
        (waiting for reductions started during backward included): the exposed part, the quantity
        the reference reports as its `backward-params-all-reduce` timer
        (eth/runtime/megatron/training.py:935-977, 1119-1169)."""
        if self.device.type != "cuda":
            return None
        pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        self._gs_pairs.append(pair)
        if len(self._gs_pairs) > 64:
            del self._gs_pairs[:-64]
        return pair

    def exposed_grad_sync_ms(self, last: int = 1) -> float:
        """Mean exposed gradient-sync time (ms per iteration) over the `last` iterations;
        synchronises on the newest event. 0.0 when nothing had to be reduced."""
        pairs = self._gs_pairs[-last:]
        if not pairs:
            return 0.0
        pairs[-1][1].synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)

    def eval_step(self) -> None:
        """Forward-only pass over one global batch with dropout disabled; accumulates the masked loss
        sum and weight into `loss_acc` (read them with `reduced_loss`). Gradients, optimizer state,
        the data cursor and the iteration counter are left untouched."""
        cfg = self.stage.cfg
        saved, provider = cfg.hidden_dropout, self.data_provider
        cfg.hidden_dropout = 0.0
        if self.eval_data_provider is not None:
            self.data_provider = self.eval_data_provider
        try:
            self.loss_acc.zero_()
            schedules.forward_only(self, self.pstate.num_microbatches)
            self.coll.all_reduce_sum(self.loss_acc)
        finally:
            cfg.hidden_dropout, self.data_provider = saved, provider

    def _evidence(self, phase, out_dir, **metrics):
        from ..parallel.grad_sync.evidence import snapshot_rank
        snapshot_rank(self, phase, self.iteration + 1, out_dir, metrics)

    def reduced_loss(self) -> float:
        """Mean masked LM loss of the last iteration (synchronises)."""
        s, w = self.loss_acc.tolist()
        return s / w if w > 0 else float("nan")
