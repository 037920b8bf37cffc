"""The parts of bench.py that need no GPU: the layouts per GPU count are valid configs of the
benchmark's definition (weak scaling, micro-batch 4 per replica), the clock sampler summarises
nvidia-smi lines, and the reference arm's argument list asks the reference for the same job."""
import importlib.util
import os
import sys

import pytest

from eth_b200.contract.config import normalize_flexpipe_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("n,layout", [(1, (1, 1, 1)), (2, (1, 1, 2)), (4, (1, 1, 4)), (8, (2, 2, 2))])
def test_layouts_are_valid_weak_scaling_configs(bench, n, layout):
    config, got, gbs = bench.build_config(n)
    assert got == layout and gbs == 64 * n
    norm = normalize_flexpipe_config(config)
    assert norm["world_size"] == n and norm["total_gbs"] == gbs
    pipe = norm["pipe"][0]
    pp, tp, dp = layout
    assert pipe["num_stages"] == pp and pipe["num_gpus"] == [tp * dp] * pp
    assert pipe["micro_batch_size"] == 4 * dp                      # 4 samples per replica and micro-batch
    assert norm["num_layers"] == 24 and norm["hidden_size"] == 2048 and norm["num_attention_heads"] == 16


def test_clock_sampler_summary(bench):
    lines = ["0, 1450, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1500, 1965, 995.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1400, 1965, 999.9, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "garbage line"]
    out = bench.ClockSampler.summary(lines)
    assert out["sm_mhz"] == 1450 and out["sm_max_mhz"] == 1965 and out["samples"] == 3
    assert out["reasons"] == ["sw_power_cap"]


def test_reference_arm_asks_for_the_same_job(tmp_path):
    from baseline.reference_arm import reference_argv
    argv = reference_argv(str(tmp_path / "cfg.json"), str(tmp_path / "logs"), 7, "--fp16", 4096, 3)
    text = " ".join(argv)
    assert "--flexpipe-config " + str(tmp_path / "cfg.json") in text
    assert "--fp16" in argv and "--train-iters 7" in text and "--local_rank=3" in text
    assert "--grad-sync-mode block" in text and "--grad-sync-bucket-size-mb 32" in text
