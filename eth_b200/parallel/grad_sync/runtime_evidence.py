"""Opt-in observations around the real gradient collectives of a run.

What is recorded, per iteration and bucket: sha256 of the packed payload, byte counts, number of
collectives, and whether the set of process groups and the scratch buffers stayed the same
objects. One JSON file per rank (`rank-00000.json`) that
`tools/validation/compare_runtime_evidence.py` reads to compare a tensor-mode run with a block-mode
run; the JSON keys are that tool's input contract
(reference: eth/runtime/megatron/grad_sync/runtime_evidence.py:21-138).

The log is plain data (`EvidenceLog`); the functions below append to it and render it.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, List, Optional, Tuple

import torch

Signature = Tuple[Tuple[str, int, int], ...]     # (dtype name, numel, storage address) per scratch buffer


def scratch_signature(scratch) -> Signature:
    return tuple((name, int(t.numel()), int(t.untyped_storage().data_ptr())) for name, t in sorted(scratch.items()))


def _signature_rows(sig: Signature):
    return [{"dtype": d, "numel": n, "data_ptr": p} for d, n, p in sig]


@dataclass
class EnvironmentSample:
    """Things that must not change while training runs."""
    group_count: int
    groups_created: int
    scratch: Signature


@dataclass
class IterationRecord:
    index: int
    normalization_scale: float
    buckets: List[dict] = field(default_factory=list)
    payload_bytes: int = 0
    stream_digest: "hashlib._Hash" = field(default_factory=hashlib.sha256)
    environment: Optional[EnvironmentSample] = None


@dataclass
class EvidenceLog:
    rank: int
    directory: Path
    baseline: EnvironmentSample
    sample_environment: Callable[[], EnvironmentSample]
    finished: List[IterationRecord] = field(default_factory=list)
    open_record: Optional[IterationRecord] = None


def start_log(plan, global_rank: int, registry, scratch, output_dir) -> EvidenceLog:
    def sample() -> EnvironmentSample:
        return EnvironmentSample(int(registry.group_count), int(registry.creation_count), scratch_signature(scratch))
    return EvidenceLog(rank=int(global_rank), directory=Path(output_dir), baseline=sample(), sample_environment=sample)


def open_iteration(log: EvidenceLog, normalization_scale: float) -> None:
    if log.open_record is not None:
        raise RuntimeError("runtime evidence execution already active")
    log.open_record = IterationRecord(index=len(log.finished) + 1, normalization_scale=float(normalization_scale))


def record_bucket(log: EvidenceLog, bucket, payload: torch.Tensor) -> None:
    rec = log.open_record
    if rec is None:
        raise RuntimeError("runtime evidence execution is not active")
    raw = payload.detach().cpu().contiguous().view(dtype=torch.uint8).numpy().tobytes()
    rec.stream_digest.update(raw)
    rec.payload_bytes += len(raw)
    rec.buckets.append({
        "bucket_id": bucket.bucket_id, "semantic_hash": bucket.semantic_hash,
        "process_group_id": bucket.process_group_id, "exact_numel": int(bucket.exact_numel),
        "exact_bytes": int(bucket.exact_bytes), "packed_payload_sha256": hashlib.sha256(raw).hexdigest()})


def close_iteration(log: EvidenceLog) -> None:
    if log.open_record is None:
        raise RuntimeError("runtime evidence execution is not active")
    log.open_record.environment = log.sample_environment()
    log.finished.append(log.open_record)
    log.open_record = None


def render(log: EvidenceLog, plan) -> dict:
    """The report of one rank as the comparison tool expects it."""
    base = log.baseline
    envs = [it.environment for it in log.finished]
    iterations = [{
        "iteration": it.index, "normalization_scale": it.normalization_scale, "collective_count": len(it.buckets),
        "payload_bytes": it.payload_bytes, "buckets": it.buckets,
        "packed_payload_sha256": it.stream_digest.hexdigest(), "process_group_count": it.environment.group_count,
        "process_group_creation_count": it.environment.groups_created,
        "scratch_signature": _signature_rows(it.environment.scratch)} for it in log.finished]
    return {
        "version": 1, "global_rank": log.rank, "sync_mode": plan.sync_mode,
        "global_topology_hash": plan.global_topology_hash, "global_manifest_hash": plan.global_manifest_hash,
        "global_fragment_hash": plan.global_fragment_hash, "global_plan_hash": plan.global_plan_hash,
        "exact_payload_bytes_by_rank": [[int(r), int(v)] for r, v in plan.exact_payload_bytes_by_rank],
        "padding_payload_bytes": int(plan.padding_payload_bytes),
        "process_group_count": base.group_count, "process_group_creation_count": base.groups_created,
        "scratch": _signature_rows(base.scratch),
        "process_group_count_stable": all(e.group_count == base.group_count for e in envs),
        "process_group_creation_count_stable": all(e.groups_created == base.groups_created for e in envs),
        "scratch_stable": log.sample_environment().scratch == base.scratch
        and all(e.scratch == base.scratch for e in envs),
        "iterations": iterations,
    }


def write_report(log: EvidenceLog, plan) -> Path:
    log.directory.mkdir(parents=True, exist_ok=True)
    target = log.directory / f"rank-{log.rank:05d}.json"
    scratch_file = target.with_suffix(".json.tmp")
    scratch_file.write_text(json.dumps(render(log, plan), indent=2, sort_keys=True) + "\n", encoding="utf-8")
    scratch_file.replace(target)
    return target
