"""Synthetic workload generators and benchmark statistics (CPU).

Mirrors the reference's generator tests (tests/test_routing.py:20-110) and timing test
(tests/test_timing.py:13-21) for the stand-ins used here: ``b200moe/workloads.py`` and the
percentile helpers of ``bench.py``.
"""

from __future__ import annotations

import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from b200moe import workloads

REPO = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("pattern", workloads.ROUTING_PATTERNS)
def test_routing_patterns_are_valid_and_seed_reproducible(pattern: str) -> None:
    T, E, K = 48, 32, 4
    a = workloads.make_routing(T, E, K, pattern, seed=11)
    b = workloads.make_routing(T, E, K, pattern, seed=11)
    c = workloads.make_routing(T, E, K, pattern, seed=12)
    assert a.dtype == torch.int64 and tuple(a.shape) == (T, K) and a.is_contiguous()
    assert int(a.min()) >= 0 and int(a.max()) < E
    assert torch.equal(a, b)
    assert not torch.equal(a, c)
    if pattern not in ("duplicates",):
        # every other pattern routes a token to K distinct experts
        assert all(len(set(row.tolist())) == K for row in a)


def test_uniform_is_balanced_and_skewed_patterns_are_not() -> None:
    T, E, K = 4096, 16, 2
    uniform = np.bincount(workloads.make_routing(T, E, K, "uniform", 3).reshape(-1).numpy(),
                          minlength=E)
    assert uniform.max() / uniform.mean() < 1.15
    zipf = np.bincount(workloads.make_routing(T, E, K, "zipf", 3).reshape(-1).numpy(),
                       minlength=E)
    assert zipf[0] > 3 * zipf[-1] and zipf.max() / zipf.mean() > 2.0
    hot = np.bincount(workloads.make_routing(T, 64, 8, "hotspot", 3).reshape(-1).numpy(),
                      minlength=64)
    assert hot[:4].sum() == T * 8 // 2                  # exactly half of all assignments
    half = workloads.make_routing(T, E, K, "empty_half", 3)
    assert len(torch.unique(half)) <= E // 2
    same = workloads.make_routing(T, E, K, "concentrated", 3)
    assert len(torch.unique(same)) == K and torch.equal(same[0], same[-1])


def test_unknown_pattern_and_weight_kind_are_rejected() -> None:
    with pytest.raises(ValueError, match="unknown routing pattern"):
        workloads.make_routing(4, 8, 2, "round_robin")
    with pytest.raises(ValueError, match="weight kind"):
        workloads.make_routing_weights(4, 2, kind="sigmoid")


@pytest.mark.parametrize("top_k", [1, 2, 4, 8])
def test_softmax_routing_weights_are_normalised_and_raw_ones_are_not(top_k: int) -> None:
    soft = workloads.make_routing_weights(64, top_k, "softmax", seed=5, dtype=torch.float32)
    assert torch.allclose(soft.sum(dim=-1), torch.ones(64), atol=1e-6) and float(soft.min()) > 0
    raw = workloads.make_routing_weights(64, top_k, "raw", seed=5, dtype=torch.float32)
    assert float(raw.min()) < 0                          # negatives are part of the contract
    assert torch.equal(soft, workloads.make_routing_weights(64, top_k, "softmax", seed=5,
                                                            dtype=torch.float32))


def test_make_case_shapes_dtypes_and_the_three_seeds() -> None:
    hidden, ids, weights, gate_up, down = workloads.make_case(5, 32, 48, 4, 2, seed=100)
    assert tuple(hidden.shape) == (5, 32) and hidden.dtype == torch.bfloat16
    assert tuple(ids.shape) == (5, 2) and tuple(weights.shape) == (5, 2)
    assert tuple(gate_up.shape) == (4, 96, 32) and tuple(down.shape) == (4, 32, 48)
    # seed, seed + 1, seed + 2: activations, routes (ids and weights), expert weights
    assert torch.equal(hidden, workloads.make_hidden(5, 32, seed=100))
    assert torch.equal(ids, workloads.make_routing(5, 4, 2, "uniform", 101))
    assert torch.equal(weights, workloads.make_routing_weights(5, 2, "softmax", 101))
    again = workloads.make_expert_weights(4, 32, 48, seed=102)
    assert torch.equal(gate_up, again[0]) and torch.equal(down, again[1])
    assert abs(float(gate_up.float().std()) - 0.02) < 0.002


def test_benchmark_configurations_match_the_named_shapes() -> None:
    c = workloads.CONFIGS
    assert (c["mixtral"].hidden_size, c["mixtral"].intermediate_size, c["mixtral"].num_experts,
            c["mixtral"].top_k, c["mixtral"].tokens) == (4096, 14336, 8, 2, (1, 2, 4, 8, 16, 32, 64))
    assert (c["wide"].num_experts, c["wide"].top_k, c["wide"].routing, c["wide"].weight_kind) == \
        (64, 8, "zipf", "raw")
    assert (c["deepseek"].hidden_size, c["deepseek"].intermediate_size,
            c["deepseek"].num_experts) == (7168, 2048, 256)
    assert c["irregular"].tokens == (1, 3, 17, 63)


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", REPO / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_percentiles_interpolate_linearly_on_sorted_samples() -> None:
    """benchmark/timing.py:23-29: position (n - 1) * q, linear between neighbours."""

    bench = _bench_module()
    samples = [1.0, 2.0, 3.0, 4.0, 10.0]
    assert bench.percentile(samples, 0.5) == 3.0
    assert bench.percentile(samples, 0.9) == pytest.approx(4.0 + 0.6 * 6.0)
    assert bench.percentile(samples, 0.0) == 1.0 and bench.percentile(samples, 1.0) == 10.0
    assert bench.percentile([7.0], 0.99) == 7.0
    s = bench.summary([5.0, 1.0, 3.0])
    assert s == {"p50": 3.0, "p90": 4.6, "p99": 4.96}
    assert s["p50"] <= s["p90"] <= s["p99"] <= 5.0


def test_algorithmic_weight_bytes_of_both_weight_formats() -> None:
    bench = _bench_module()
    bench.apply_config("mixtral")
    bf16 = bench.weight_bytes(2)
    assert bf16 == {"gate_up": 2 * 4 * 4096 * 14336, "down": 2 * 2 * 4096 * 14336,
                    "total": 2 * 6 * 4096 * 14336}
    bench.WEIGHT_ELEMENT_BYTES = 1
    fp8 = bench.weight_bytes(2)
    assert fp8["gate_up"] == 2 * (2 * 4096 * 14336 + 4 * 2 * 14336)
    assert fp8["down"] == 2 * (4096 * 14336 + 4 * 4096)
