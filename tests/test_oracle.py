"""The CPU oracle against the reference: golden fixtures and literal known answers."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES
from oracle import moe_oracle


def test_golden_fixtures_exist() -> None:
    assert len(GOLDEN_CASES) >= 15
    assert {c.group for c in GOLDEN_CASES} == {"e16_h32_i48", "e4_h72_i200", "e32_h32_i64"}


@pytest.mark.parametrize("case", GOLDEN_CASES, ids=lambda c: c.label)
def test_oracle_routing_is_bit_exact_against_reference(case) -> None:
    routing = moe_oracle.group_tokens(case.ids, case.num_experts)
    for key in ("permutation", "reverse_mapping", "expert_counts", "expert_offsets"):
        got = getattr(routing, key)
        want = case.routing[key].numpy()
        assert got.dtype == np.int64
        np.testing.assert_array_equal(got, want, err_msg=f"{case.label}:{key}")
    slow = moe_oracle.group_tokens_by_counting(case.ids, case.num_experts)
    np.testing.assert_array_equal(slow.permutation, routing.permutation)
    np.testing.assert_array_equal(slow.reverse_mapping, routing.reverse_mapping)
    np.testing.assert_array_equal(slow.expert_offsets, routing.expert_offsets)


@pytest.mark.parametrize("case", GOLDEN_CASES, ids=lambda c: c.label)
def test_oracle_output_matches_reference_fp32(case) -> None:
    out, _ = moe_oracle.routed_moe(
        *case.inputs(), num_experts=case.num_experts, top_k=case.top_k
    )
    # same FP32 algebra as the reference's torch backend on the same inputs;
    # tolerance of the reference's own oracle test (tests/test_goal_1b_correctness.py:77)
    torch.testing.assert_close(out, case.output_fp32, atol=3e-5, rtol=3e-5)


@pytest.mark.parametrize("case", [c for c in GOLDEN_CASES if c.hidden.shape[0] <= 8],
                         ids=lambda c: c.label)
def test_naive_loop_agrees(case) -> None:
    out = moe_oracle.routed_moe_naive(*case.inputs())
    torch.testing.assert_close(out, case.output_fp32, atol=3e-5, rtol=3e-5)


def test_repeated_route_known_answer() -> None:
    # literal expectation of the reference's routing test (tests/test_goal_1b_routing.py:46-54)
    ids = torch.tensor([[3, 3]] * 3, dtype=torch.int64)
    routing = moe_oracle.group_tokens(ids, 8)
    assert routing.expert_counts.tolist() == [0, 0, 0, 6, 0, 0, 0, 0]
    assert routing.expert_offsets.tolist() == [0, 0, 0, 0, 6, 6, 6, 6, 6]
    assert routing.permutation.tolist() == list(range(6))
    assert routing.reverse_mapping.tolist() == list(range(6))


def test_single_expert_concentration_known_answer() -> None:
    # tests/test_goal_1b_cuda.py:213-247: 8 tokens x 2 slots all on expert 5 of 16
    ids = torch.full((8, 2), 5, dtype=torch.int64)
    routing = moe_oracle.group_tokens(ids, 16)
    assert routing.expert_counts.tolist() == [0] * 5 + [16] + [0] * 10


def test_routing_rejects_bad_inputs() -> None:
    with pytest.raises(TypeError, match="int64"):
        moe_oracle.group_tokens(torch.zeros(2, 2, dtype=torch.int32), 4)
    with pytest.raises(ValueError, match="out-of-range"):
        moe_oracle.group_tokens(torch.full((2, 2), 4, dtype=torch.int64), 4)


def test_weights_are_used_as_supplied() -> None:
    # unnormalised, negative and zero weights scale linearly (reference.py:328-330)
    case = GOLDEN_CASES[3]
    hidden, ids, weights, gate_up, down = case.inputs()
    base, _ = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down,
                                    num_experts=case.num_experts, top_k=case.top_k)
    scaled, _ = moe_oracle.routed_moe(hidden, ids, (weights.float() * -2).to(torch.bfloat16),
                                      gate_up, down, num_experts=case.num_experts, top_k=case.top_k)
    torch.testing.assert_close(scaled, -2 * base, atol=1e-5, rtol=1e-5)
    zero, _ = moe_oracle.routed_moe(hidden, ids, torch.zeros_like(weights), gate_up, down,
                                    num_experts=case.num_experts, top_k=case.top_k)
    assert float(zero.abs().max()) == 0.0


def test_low_precision_variant_is_close_and_floor_is_reported() -> None:
    case = GOLDEN_CASES[6]
    ref, _ = moe_oracle.routed_moe(*case.inputs(), num_experts=case.num_experts, top_k=case.top_k)
    low, _ = moe_oracle.routed_moe(*case.inputs(), num_experts=case.num_experts,
                                   top_k=case.top_k, compute_dtype=torch.bfloat16)
    assert low.dtype == torch.bfloat16
    assert moe_oracle.relative_max_error(low.float(), ref) < 0.1
    floor = moe_oracle.bf16_floor(ref)
    assert 0.0 < floor < 2e-2


from conftest import ROUTER_CASES  # noqa: E402


@pytest.mark.parametrize("case", ROUTER_CASES, ids=lambda c: c["label"])
def test_oracle_router_matches_reference_topk_routing(case) -> None:
    ids, weights = moe_oracle.topk_routing(case["logits"], case["ids"].shape[1])
    # compare where the selection is tie-free (torch.topk leaves ties unspecified)
    selected = torch.gather(case["logits"].float(), 1, case["ids"])
    tie_free = (selected[:, :-1] != selected[:, 1:]).all(dim=1) if selected.shape[1] > 1 else \
        torch.ones(selected.shape[0], dtype=torch.bool)
    assert bool(tie_free.any())
    assert torch.equal(ids[tie_free], case["ids"][tie_free])
    torch.testing.assert_close(weights.float(), case["weights"].float(), atol=1e-6, rtol=1e-6)
    assert weights.dtype == case["weights"].dtype
