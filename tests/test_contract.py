"""CPU tests of the Python contract: validation order and messages, backend/quant
pairing, workspace bookkeeping.  They follow the reference's
tests/test_goal_1b_edge_cases.py:42-227 and tests/test_goal_1c_dispatch.py:173-203."""

from __future__ import annotations

import pytest
import torch

from b200moe import B300MoEWorkspace, b300_moe_forward, validate_routed_moe_inputs


def _case(tokens=4, experts=8, top_k=2, hidden=16, inter=24, dtype=torch.float32):
    g = torch.Generator().manual_seed(7)
    hidden_states = torch.randn(tokens, hidden, generator=g).to(dtype)
    ids = torch.randint(0, experts, (tokens, top_k), generator=g)
    weights = torch.rand(tokens, top_k, generator=g).to(dtype)
    gate_up = torch.randn(experts, 2 * inter, hidden, generator=g).to(dtype)
    down = torch.randn(experts, hidden, inter, generator=g).to(dtype)
    return [hidden_states, ids, weights, gate_up, down]


def _call(tensors, **kwargs):
    kwargs.setdefault("num_experts", 8)
    kwargs.setdefault("top_k", 2)
    return b300_moe_forward(*tensors, **kwargs)


@pytest.mark.parametrize(
    "mutate, error, match",
    [
        (lambda t: t.__setitem__(0, t[0][:3]), ValueError, "same num_tokens"),
        (lambda t: t.__setitem__(1, t[1].int()), TypeError, "int64"),
        (lambda t: t.__setitem__(3, t[3].half()), TypeError, "same dtype"),
        (lambda t: t.__setitem__(1, torch.full_like(t[1], 8)), ValueError, "out-of-range"),
        (lambda t: t.__setitem__(1, torch.full_like(t[1], -1)), ValueError, "out-of-range"),
        (lambda t: t.__setitem__(0, t[0].t().contiguous().t()), ValueError, "contiguous"),
        (lambda t: t.__setitem__(3, t[3][:, :47].contiguous()), ValueError, "positive even"),
        (lambda t: t.__setitem__(4, t[4][:, :, :23].contiguous()), ValueError, r"\[E, H, I\]"),
        (lambda t: t.__setitem__(3, t[3][:7].contiguous()), ValueError, "num_experts"),
    ],
)
def test_contract_violations_raise_like_the_reference(mutate, error, match) -> None:
    tensors = _case()
    mutate(tensors)
    with pytest.raises(error, match=match):
        _call(tensors)


def test_top_k_and_num_experts_arguments() -> None:
    with pytest.raises(ValueError, match="top_k must match"):
        _call(_case(), top_k=4)
    with pytest.raises(TypeError, match="num_experts"):
        _call(_case(), num_experts=True)
    with pytest.raises(ValueError, match="top_k"):
        _call(_case(top_k=3), top_k=3)
    with pytest.raises(ValueError, match="must not exceed"):
        _call(_case(experts=2, top_k=4), num_experts=2, top_k=4)


def test_argument_types_checked_before_tensors() -> None:
    with pytest.raises(TypeError, match="return_metadata"):
        _call(_case(), return_metadata=1)
    with pytest.raises(TypeError, match="backend"):
        _call(_case(), backend=3)
    with pytest.raises(ValueError, match="backend must be"):
        _call(_case(), backend="triton")
    with pytest.raises(TypeError, match="gemm_policy"):
        _call(_case(), gemm_policy=None)
    with pytest.raises(ValueError, match="gemm_policy"):
        _call(_case(), gemm_policy="fastest")
    # a bad return_metadata wins over a bad tensor
    broken = _case()
    broken[1] = broken[1].int()
    with pytest.raises(TypeError, match="return_metadata"):
        _call(broken, return_metadata="yes")


def test_backend_and_quant_mode_pairing() -> None:
    with pytest.raises(ValueError, match="cannot execute NVFP4"):
        _call(_case(), backend="torch", quant_mode="nvfp4")
    with pytest.raises(ValueError, match="requires quant_mode='bf16'"):
        _call(_case(), backend="cutlass_bf16", quant_mode="none")
    with pytest.raises(ValueError, match="requires quant_mode='bf16'"):
        _call(_case(), backend="b200_bf16", quant_mode="nvfp4")
    with pytest.raises(ValueError, match="requires quant_mode='nvfp4'"):
        _call(_case(), backend="cutlass_nvfp4", quant_mode="bf16")
    with pytest.raises(TypeError, match="quant_mode"):
        _call(_case(), quant_mode=1)


@pytest.mark.parametrize("backend", ["cutlass_bf16", "b200_bf16", "cutlass_nvfp4"])
def test_native_backends_on_cpu_tensors_raise_and_never_fall_back(backend) -> None:
    workspace = B300MoEWorkspace()
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        _call(_case(dtype=torch.bfloat16), backend=backend, workspace=workspace)
    assert workspace.allocation_count == 0


def test_torch_backend_is_not_an_execution_path() -> None:
    with pytest.raises(RuntimeError, match="not an execution path"):
        _call(_case(), backend="torch", quant_mode="none")


def test_workspace_type_and_autograd_rules() -> None:
    with pytest.raises(TypeError, match="B300MoEWorkspace"):
        _call(_case(), workspace=object())
    tensors = _case()
    tensors[0].requires_grad_(True)
    workspace = B300MoEWorkspace()
    with pytest.raises(ValueError, match="inference-only"):
        _call(tensors, workspace=workspace)
    assert workspace.allocation_count == 0


def test_invalid_call_leaves_workspace_untouched() -> None:
    workspace = B300MoEWorkspace(device="cpu")
    tensors = _case()
    tensors[1] = torch.full_like(tensors[1], 8)
    with pytest.raises(ValueError, match="out-of-range"):
        _call(tensors, workspace=workspace)
    assert (workspace.allocation_count, workspace.reuse_count) == (0, 0)
    with pytest.raises(ValueError, match="bound to device"):
        workspace.reserve(num_tokens=1, num_experts=8, top_k=1, hidden_size=8,
                          intermediate_size=8, device="meta", dtype=torch.float32)


def test_workspace_reserve_reuse_grow_rebind_on_cpu() -> None:
    workspace = B300MoEWorkspace(capacity_tokens=4, device="cpu")
    kwargs = dict(num_experts=8, top_k=2, hidden_size=16, intermediate_size=24, device="cpu",
                  dtype=torch.float32)
    assert workspace.reserve(num_tokens=3, **kwargs) is False
    first = workspace.buffer_data_ptrs()
    assert set(first) == {
        "expert_counts", "expert_offsets", "expert_offsets_i32", "permutation",
        "reverse_mapping", "permuted_token_indices", "permuted_expert_indices",
        "permuted_weights", "permuted_hidden", "gate_up_output", "swiglu_output",
        "expert_output",
    }
    assert workspace.buffers["expert_offsets"].dtype == torch.int64
    assert workspace.buffers["expert_offsets_i32"].dtype == torch.int32
    assert workspace.buffers["permuted_hidden"].shape == (8, 16)
    assert (workspace.allocation_count, workspace.reuse_count) == (1, 0)
    assert (workspace.capacity_tokens, workspace.capacity_assignments) == (4, 8)
    assert workspace.capacity_bytes > 0 and workspace.last_stream is None
    assert workspace.reserve(num_tokens=4, **kwargs) is True
    assert workspace.buffer_data_ptrs() == first
    assert (workspace.allocation_count, workspace.reuse_count) == (1, 1)
    assert workspace.reserve(num_tokens=6, **kwargs) is False
    assert workspace.allocation_count == 2 and workspace.capacity_tokens >= 8
    kwargs.update(top_k=1, hidden_size=9)
    assert workspace.reserve(num_tokens=2, **kwargs) is False
    assert workspace.allocation_count == 3
    assert workspace.last_shape == (2, 8, 1, 9, 24)
    assert workspace.capacity_tokens == 4  # a new layout restarts from max(hint, T)
    with pytest.raises(TypeError, match="num_tokens"):
        workspace.reserve(num_tokens=True, **kwargs)
    with pytest.raises(ValueError, match="top_k"):
        workspace.reserve(num_tokens=1, **{**kwargs, "top_k": 3})


def test_workspace_constructor_checks() -> None:
    with pytest.raises(TypeError):
        B300MoEWorkspace(capacity_tokens=1.5)
    with pytest.raises(ValueError):
        B300MoEWorkspace(capacity_tokens=-1)
    assert B300MoEWorkspace().status() == 0


def test_validate_returns_shape() -> None:
    shape = validate_routed_moe_inputs(*_case(), num_experts=8, top_k=2)
    assert (shape.num_tokens, shape.num_experts, shape.top_k) == (4, 8, 2)
    assert (shape.hidden_size, shape.intermediate_size, shape.num_assignments) == (16, 24, 8)


# ---------------------------------------------------------------------------
# FP8-weight entry point: host-side contract (no GPU needed to be rejected)
# ---------------------------------------------------------------------------
def _fp8_inputs(E=4, H=32, I=48, K=2, T=3):
    from b200moe import Fp8ExpertWeights

    hidden = torch.zeros(T, H, dtype=torch.bfloat16)
    ids = torch.zeros(T, K, dtype=torch.int64)
    ids[:, 1] = 1
    weights = torch.ones(T, K, dtype=torch.bfloat16)
    fw = Fp8ExpertWeights(
        torch.zeros(E, 2 * I, H, dtype=torch.uint8), torch.ones(E, 2 * I, dtype=torch.float32),
        torch.zeros(E, H, I, dtype=torch.uint8), torch.ones(E, H, dtype=torch.float32))
    return hidden, ids, weights, fw


def test_fp8_forward_rejects_bad_arguments_on_the_host() -> None:
    from b200moe import Fp8ExpertWeights, b300_moe_forward_fp8

    hidden, ids, weights, fw = _fp8_inputs()
    E, K = 4, 2
    with pytest.raises(TypeError, match="Fp8ExpertWeights"):
        b300_moe_forward_fp8(hidden, ids, weights, (fw.gate_up_q, fw.down_q), num_experts=E, top_k=K)
    with pytest.raises(TypeError, match="return_metadata"):
        b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K, return_metadata=1)
    with pytest.raises(TypeError, match="int64"):
        b300_moe_forward_fp8(hidden, ids.int(), weights, fw, num_experts=E, top_k=K)
    with pytest.raises(ValueError, match="num_experts"):
        b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E + 1, top_k=K)
    with pytest.raises(ValueError, match="hidden dimension"):
        b300_moe_forward_fp8(hidden[:, :16].contiguous(), ids, weights, fw, num_experts=E, top_k=K)
    with pytest.raises(TypeError, match="uint8"):
        bad = Fp8ExpertWeights(fw.gate_up_q.to(torch.int8), fw.gate_up_scale, fw.down_q, fw.down_scale)
        b300_moe_forward_fp8(hidden, ids, weights, bad, num_experts=E, top_k=K)
    with pytest.raises(TypeError, match="float32"):
        bad = Fp8ExpertWeights(fw.gate_up_q, fw.gate_up_scale.double(), fw.down_q, fw.down_scale)
        b300_moe_forward_fp8(hidden, ids, weights, bad, num_experts=E, top_k=K)
    with pytest.raises(TypeError, match="bfloat16"):
        b300_moe_forward_fp8(hidden.float(), ids, weights.float(), fw, num_experts=E, top_k=K)
    with pytest.raises(ValueError, match="out-of-range"):
        b300_moe_forward_fp8(hidden, ids + 7, weights, fw, num_experts=E, top_k=K)
    # H = 40 is a multiple of 8 (enough for BF16 weights) but not of 16
    h40, i40, w40, fw40 = _fp8_inputs(H=40)
    with pytest.raises(ValueError, match="divisible by 16"):
        b300_moe_forward_fp8(h40, i40, w40, fw40, num_experts=E, top_k=K)
    # a valid call still needs a CUDA device: there is no CPU path
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K)


def test_fp8_weight_container_reports_its_geometry() -> None:
    _, _, _, fw = _fp8_inputs(E=4, H=32, I=48)
    assert (fw.num_experts, fw.hidden_size, fw.intermediate_size) == (4, 32, 48)
    assert fw.nbytes == 4 * (2 * 48 * 32 + 32 * 48) + 4 * 4 * (2 * 48 + 32)


def test_graphed_layer_rejects_bad_construction_on_the_host() -> None:
    from b200moe import GraphedMoEDecodeLayer

    gate_up = torch.zeros(4, 96, 32, dtype=torch.bfloat16)
    down = torch.zeros(4, 32, 48, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="requires CUDA weights"):
        GraphedMoEDecodeLayer(gate_up, down, num_experts=4, top_k=2)
    with pytest.raises(ValueError, match="pass gate_up_weight and down_weight"):
        GraphedMoEDecodeLayer(None, None, num_experts=4, top_k=2)
    with pytest.raises(TypeError, match="Fp8ExpertWeights"):
        GraphedMoEDecodeLayer(None, None, num_experts=4, top_k=2, fp8_weights=(gate_up, down))


def test_out_tensor_rules() -> None:
    """``out=`` of ``b300_moe_forward`` (not in the reference's signature): same shape and
    dtype as the activations, contiguous, on their device or in pinned host memory."""

    import torch

    from b200moe.forward import _check_out

    hidden = torch.empty(3, 8, dtype=torch.bfloat16, device="meta")
    _check_out(torch.empty(3, 8, dtype=torch.bfloat16, device="meta"), hidden)
    with pytest.raises(TypeError, match="out must be a torch.Tensor"):
        _check_out([0.0], hidden)
    for bad in (torch.empty(4, 8, dtype=torch.bfloat16, device="meta"),
                torch.empty(3, 8, dtype=torch.float32, device="meta"),
                torch.empty(8, 3, dtype=torch.bfloat16, device="meta").t()):
        with pytest.raises(ValueError, match="out must be a contiguous"):
            _check_out(bad, hidden)
    with pytest.raises(ValueError, match="pinned host memory"):
        _check_out(torch.empty(3, 8, dtype=torch.bfloat16), hidden)  # pageable host memory
