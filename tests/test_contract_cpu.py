"""The gpt_config.json contract: normalisation rules, hashes, runtime view."""
import copy
from types import SimpleNamespace

import pytest

from eth_b200.contract import config as C


def _cfg():
    return C.make_config([C.make_pipe([21, 22], [1, 2], [1, 1]), C.make_pipe([11, 32], [1, 1], [2, 1])])


def test_brief_and_expanded_forms_hash_identically():
    brief = _cfg()
    expanded = copy.deepcopy(brief)
    for p in expanded["pipe"]:
        for stem in C.TOPOLOGY_STEMS:
            vals = p.pop(f"{stem}_of_each_stage")
            p[f"{stem}_of_each_op"] = [[v] * n for v, n in zip(vals, p["num_ops_in_each_stage"])]
    a, b = C.normalize_flexpipe_config(brief), C.normalize_flexpipe_config(expanded)
    assert a["config_hash"] == b["config_hash"] and a["topology_fingerprint"] == b["topology_fingerprint"]
    assert a["world_size"] == 6 and a["total_gbs"] == 48 and a["pipeline_sample_offsets"] == [0, 24]
    assert len(a["manifest"]["ordered_ops"]) == 43 and a["manifest"]["ordered_ops"][1]["name"] == "enc-1st-layernorm"


@pytest.mark.parametrize("mutate,message", [
    (lambda c: c.update(bogus=1), "unknown top-level"),
    (lambda c: c["pipe"][0].update(bogus=1), "unknown field"),
    (lambda c: c["pipe"][0].update(model_parallel_size_of_each_stage=[1, 3], num_gpus=[1, 3]), "unsupported TP"),
    (lambda c: c["pipe"][0].update(context_parallel_size_of_each_stage=[1, 2]), "context parallel"),
    (lambda c: c["pipe"][0].update(num_gpus=[1, 4]), "stage product mismatch"),
    (lambda c: c["pipe"][0].update(micro_batch_size=5), "micro batch divisibility"),
    (lambda c: c["pipe"][1].update(micro_batch_size=3, global_batch_size=24), "micro batch divisibility"),
    (lambda c: c["pipe"][0].update(num_ops_in_each_stage=[21, 21]), "manifest size"),
    (lambda c: c.update(num_attention_heads=7), "TP constraint"),
    (lambda c: c["pipe"][0].update(recompute_ops=[[0] * 21, [0] * 21]), "recompute_ops"),
])
def test_violations_are_rejected(mutate, message):
    c = _cfg()
    mutate(c)
    with pytest.raises(ValueError, match=message):
        C.normalize_flexpipe_config(c)


def test_intra_stage_constancy():
    c = _cfg()
    p = c["pipe"][0]
    p.pop("model_parallel_size_of_each_stage")
    p["model_parallel_size_of_each_op"] = [[1] * 21, [2] * 21 + [1]]
    with pytest.raises(ValueError, match="intra-stage constancy"):
        C.normalize_flexpipe_config(c)


def test_world_size_check_and_model_impl_inference():
    with pytest.raises(ValueError, match="world size mismatch"):
        C.normalize_flexpipe_config(_cfg(), world_size=8)
    c = _cfg()
    c.pop("model_impl")
    with pytest.warns(UserWarning, match="inferred"):
        assert C.normalize_flexpipe_config(c)["model_impl"] == "gpt"


def test_runtime_view_rank_maps_and_loss_scale():
    n = C.normalize_flexpipe_config(_cfg())
    v = C.runtime_view(n, rank=4)
    assert v.rank_to_pipe == [0, 0, 0, 1, 1, 1] and v.rank_to_stage == [0, 1, 1, 0, 0, 1]
    assert v.current_pipe == 1 and v.offset == 3 and v.num_stages == 2
    assert v.nominal_global_loss_scale == 48 * 32 and len(v.mbs_seq[0]) == 3
    with pytest.raises(ValueError, match="sums to"):
        C.runtime_view(n, rank=0, mbs_seq=[[[8, 32]], [[8, 32]] * 3])


def test_validate_runtime_manifest():
    m = C.build_manifest("gpt", 2)
    ops = [{"op_index": o["op_index"], "name": o["name"]} for o in m["ordered_ops"]]
    C.validate_runtime_manifest(ops, m)
    ops[3]["name"] = "something-else"
    with pytest.raises(ValueError, match="mismatch at op 3"):
        C.validate_runtime_manifest(ops, m)


def test_fixture_sets_normalize():
    for cfg in C.heterogeneous_config_fixtures() + list(C.gpt_e2e_fixtures().values()):
        n = C.normalize_flexpipe_config(cfg)
        assert n["world_size"] == sum(sum(p["num_gpus"]) for p in n["pipe"])
