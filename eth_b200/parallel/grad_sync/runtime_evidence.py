"""Opt-in observations around the real gradient collectives of a run.

Per iteration and bucket: sha256 of the packed payload, byte counts, number of collectives, and
whether the set of process groups and the scratch buffers stayed the same objects. One JSON per
rank (`rank-00000.json`); `tools/validation/compare_runtime_evidence.py` compares a tensor-mode
run with a block-mode run (reference: eth/runtime/megatron/grad_sync/runtime_evidence.py:21-138).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch


def scratch_signature(scratch):
    return tuple((name, int(t.numel()), int(t.untyped_storage().data_ptr())) for name, t in sorted(scratch.items()))


class GradientRuntimeEvidenceRecorder:
    def __init__(self, plan, global_rank, registry, scratch, output_dir):
        self.plan, self.rank, self.registry, self.scratch = plan, int(global_rank), registry, scratch
        self.out = Path(output_dir)
        self.groups0 = int(registry.group_count)
        self.created0 = int(registry.creation_count)
        self.scratch0 = scratch_signature(scratch)
        self.iterations = []
        self.cur = None
        self.digest = None

    def begin_execution(self, normalization_scale):
        if self.cur is not None:
            raise RuntimeError("runtime evidence execution already active")
        self.digest = hashlib.sha256()
        self.cur = {"iteration": len(self.iterations) + 1, "normalization_scale": float(normalization_scale),
                    "collective_count": 0, "payload_bytes": 0, "buckets": []}

    def observe_packed_bucket(self, bucket, payload):
        if self.cur is None:
            raise RuntimeError("runtime evidence execution is not active")
        raw = payload.detach().cpu().contiguous().view(dtype=torch.uint8).numpy().tobytes()
        self.digest.update(raw)
        self.cur["collective_count"] += 1
        self.cur["payload_bytes"] += len(raw)
        self.cur["buckets"].append({
            "bucket_id": bucket.bucket_id, "semantic_hash": bucket.semantic_hash,
            "process_group_id": bucket.process_group_id, "exact_numel": int(bucket.exact_numel),
            "exact_bytes": int(bucket.exact_bytes), "packed_payload_sha256": hashlib.sha256(raw).hexdigest()})

    def finish_execution(self):
        if self.cur is None:
            raise RuntimeError("runtime evidence execution is not active")
        self.cur["packed_payload_sha256"] = self.digest.hexdigest()
        self.cur["process_group_count"] = int(self.registry.group_count)
        self.cur["process_group_creation_count"] = int(self.registry.creation_count)
        self.cur["scratch_signature"] = [{"dtype": d, "numel": n, "data_ptr": p}
                                         for d, n, p in scratch_signature(self.scratch)]
        self.iterations.append(self.cur)
        self.cur = self.digest = None
        self.write()

    def write(self):
        now = scratch_signature(self.scratch)
        report = {
            "version": 1, "global_rank": self.rank, "sync_mode": self.plan.sync_mode,
            "global_topology_hash": self.plan.global_topology_hash,
            "global_manifest_hash": self.plan.global_manifest_hash,
            "global_fragment_hash": self.plan.global_fragment_hash,
            "global_plan_hash": self.plan.global_plan_hash,
            "exact_payload_bytes_by_rank": [[int(r), int(v)] for r, v in self.plan.exact_payload_bytes_by_rank],
            "padding_payload_bytes": int(self.plan.padding_payload_bytes),
            "process_group_count": self.groups0, "process_group_creation_count": self.created0,
            "scratch": [{"dtype": d, "numel": n, "data_ptr": p} for d, n, p in self.scratch0],
            "process_group_count_stable": all(i["process_group_count"] == self.groups0 for i in self.iterations),
            "process_group_creation_count_stable": all(
                i["process_group_creation_count"] == self.created0 for i in self.iterations),
            "scratch_stable": now == self.scratch0 and all(
                tuple((e["dtype"], e["numel"], e["data_ptr"]) for e in i["scratch_signature"]) == self.scratch0
                for i in self.iterations),
            "iterations": self.iterations,
        }
        self.out.mkdir(parents=True, exist_ok=True)
        path = self.out / f"rank-{self.rank:05d}.json"
        tmp = path.with_suffix(".json.tmp")
        tmp.write_text(json.dumps(report, indent=2, sort_keys=True) + "\n", encoding="utf-8")
        tmp.replace(path)
