"""CPU: the benchmark's host logic -- work per configuration, sharding of the workloads, the `config` object both
arms print, and the sizing of the CPU samples."""
import importlib.util
import os

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_flops_per_configuration(bench):
    """fwd + bwd = 3 GEMMs of 2*M*N*K per batch (6 for the attention-shaped configuration)."""
    want = {"c1": 0.805e9, "c2": 103.08e9, "c3": 19.33e9, "c4": 927.7e9, "c5a": 3298.5e9,
            "c5b1": 0.1007e9, "c5b4": 0.4027e9, "c5b16": 1.611e9}
    for name, flops in want.items():
        assert abs(bench.WORKLOADS[name].flops - flops) / flops < 1e-3, name
    assert bench.WORKLOADS["c3"].out_shape == (8, 12, 512, 512)
    assert bench.WORKLOADS["c3"].b_logical == (8, 12, 64, 512)          # K^T through the permute view
    assert bench.WORKLOADS["c4"].out_shape == (64, 1024, 3072)


def test_sharding_of_the_workloads(bench):
    c4, c5a, c2 = (bench.WORKLOADS[n] for n in ("c4", "c5a", "c2"))
    assert bench.shard_workload(c4, 3, 8).a_shape == (8, 1024, 768)
    assert bench.shard_workload(c4, 0, 8).b_shape == (768, 3072)          # the weight is replicated
    assert bench.shard_workload(c5a, 7, 8).a_shape == (1024, 8192)
    assert bench.shard_workload(c2, 1, 8).a_shape == c2.a_shape            # weak scaling: a full shard per rank
    assert sum(bench.shard_workload(c4, r, 8).flops for r in range(8)) == c4.flops
    assert bench.scaling_label(c4) == "strong" and bench.scaling_label(c2) == "weak"


def test_both_arms_print_the_same_config(bench):
    for name in ("c1", "c2", "c4", "c5a", "softmax", "adamw"):
        for world in (1, 8):
            a = bench.config_dict(bench.WORKLOADS[name], world, "3xtf32")
            b = bench.config_dict(bench.WORKLOADS[name], world, "3xtf32")
            assert a == b and a["workload"].startswith(name + ":")
    assert "NCCL reduce" in bench.config_dict(bench.WORKLOADS["c4"], 8, "3xtf32")["parallelism"]
    assert bench.config_dict(bench.WORKLOADS["c4"], 1, "3xtf32")["parallelism"] == "single GPU"


def test_cpu_samples_are_bounded_leading_slices(bench):
    c4 = bench.WORKLOADS["c4"]
    small, what = bench.cpu_sample_workload(c4, budget_gflop=150.0)
    assert small.a_shape[1:] == c4.a_shape[1:] and 1 <= small.a_shape[0] < 64 and small.flops <= 150e9
    assert "leading" in what
    whole, what = bench.cpu_sample_workload(bench.WORKLOADS["c1"], budget_gflop=150.0)
    assert whole.a_shape == (512, 512) and what == "whole step"
