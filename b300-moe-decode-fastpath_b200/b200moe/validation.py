"""Input contract of the explicitly routed MoE layer.

Behavioural mirror of the reference's validators
(fastpath/reference.py:57-183, fastpath/b300_moe.py:350-384,
fastpath/gemm_dispatch.py:44-51): the same conditions raise the same exception
types with messages containing the same key phrases, checked in the same
order, because callers and tests depend on which error wins.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

SUPPORTED_TOP_K = (1, 2, 4, 8)
SUPPORTED_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
MAX_EXPERTS = 256

BACKENDS = ("torch", "cutlass_bf16", "cutlass_nvfp4", "b200_bf16")
QUANT_MODES = ("none", "bf16", "nvfp4")
GEMM_POLICIES = ("auto", "grouped", "per_expert")


@dataclass(frozen=True)
class RoutedMoEShape:
    """Dimensions of one validated call: T tokens, E experts, K slots, H, I."""

    num_tokens: int
    num_experts: int
    top_k: int
    hidden_size: int
    intermediate_size: int

    @property
    def num_assignments(self) -> int:
        return self.num_tokens * self.top_k


def _tensor(name: str, value: object) -> torch.Tensor:
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    return value


def _positive_int(name: str, value: object) -> int:
    # bool is an int subclass; the reference rejects it explicitly (reference.py:49-51)
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer")
    if value < 1:
        raise ValueError(f"{name} must be positive")
    return value


def validate_routing(
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    num_experts: int,
    top_k: int | None = None,
    *,
    check_range_on_device: bool = False,
) -> tuple[int, int]:
    """Checks on the two routing tensors (reference.py:57-106).

    The id range check runs on the host only for CPU tensors.  For CUDA tensors
    the reference issues a device-side assert (reference.py:99-103), which
    destroys the CUDA context when it fires; here the routing kernel reports
    out-of-range ids through the workspace status word instead and drops the
    row, unless ``check_range_on_device`` asks for a synchronising check.
    """

    _tensor("expert_indices", expert_indices)
    _tensor("expert_weights", expert_weights)
    num_experts = _positive_int("num_experts", num_experts)

    if expert_indices.ndim != 2:
        raise ValueError("expert_indices must have shape [num_tokens, top_k]")
    if expert_weights.ndim != 2:
        raise ValueError("expert_weights must have shape [num_tokens, top_k]")
    if expert_weights.shape != expert_indices.shape:
        raise ValueError("expert_indices and expert_weights must have the same shape")
    tokens, slots = expert_indices.shape
    if tokens < 1:
        raise ValueError("num_tokens must be positive")
    if slots not in SUPPORTED_TOP_K:
        raise ValueError(f"top_k must be one of {SUPPORTED_TOP_K}, got {slots}")
    if slots > num_experts:
        raise ValueError("top_k must not exceed num_experts")
    if top_k is not None:
        if _positive_int("top_k", top_k) != slots:
            raise ValueError(
                "top_k must match expert_indices.shape[1] and expert_weights.shape[1]"
            )
    if expert_indices.dtype != torch.int64:
        raise TypeError("expert_indices must have dtype torch.int64")
    if expert_weights.dtype not in SUPPORTED_DTYPES:
        raise TypeError("expert_weights dtype must be float32, float16, or bfloat16")
    if expert_indices.device != expert_weights.device:
        raise ValueError("expert_indices and expert_weights must be on the same device")
    if not (expert_indices.is_contiguous() and expert_weights.is_contiguous()):
        raise ValueError("expert_indices and expert_weights must be contiguous")

    if expert_indices.device.type != "cuda" or check_range_on_device:
        low = int(expert_indices.min())
        high = int(expert_indices.max())
        if low < 0 or high >= num_experts:
            raise ValueError("expert_indices contains an out-of-range expert index")
    return tokens, slots


def validate_routed_moe_inputs(
    hidden_states: torch.Tensor,
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    gate_up_weight: torch.Tensor,
    down_weight: torch.Tensor,
    *,
    num_experts: int,
    top_k: int,
    check_range_on_device: bool = False,
    expert_weights_on_other_device: bool = False,
) -> RoutedMoEShape:
    """Full tensor contract (reference.py:109-183); returns the dimensions.

    ``expert_weights_on_other_device`` relaxes the one-device rule for the pinned-host
    entry point: the three per-step tensors share a device and the two weight tensors share
    a device.
    """

    named = {
        "hidden_states": hidden_states,
        "expert_indices": expert_indices,
        "expert_weights": expert_weights,
        "gate_up_weight": gate_up_weight,
        "down_weight": down_weight,
    }
    for name, value in named.items():
        _tensor(name, value)
    num_experts = _positive_int("num_experts", num_experts)
    top_k = _positive_int("top_k", top_k)
    tokens, slots = validate_routing(
        expert_indices,
        expert_weights,
        num_experts,
        top_k,
        check_range_on_device=check_range_on_device,
    )

    if hidden_states.ndim != 2:
        raise ValueError("hidden_states must have shape [num_tokens, hidden_size]")
    if hidden_states.shape[0] != tokens:
        raise ValueError(
            "hidden_states, expert_indices, and expert_weights must have the same num_tokens"
        )
    hidden = hidden_states.shape[1]
    if hidden < 1:
        raise ValueError("hidden_size must be positive")
    if gate_up_weight.ndim != 3:
        raise ValueError("gate_up_weight must have shape [E, 2I, H]")
    if gate_up_weight.shape[0] != num_experts:
        raise ValueError("gate_up_weight.shape[0] must equal num_experts")
    if gate_up_weight.shape[2] != hidden:
        raise ValueError("gate_up_weight hidden dimension must match hidden_states")
    two_i = gate_up_weight.shape[1]
    if two_i < 2 or two_i % 2 != 0:
        raise ValueError("gate_up_weight dimension 1 must be a positive even size 2I")
    inter = two_i // 2
    want_down = (num_experts, hidden, inter)
    if tuple(down_weight.shape) != want_down:
        raise ValueError(
            "down_weight must have shape [E, H, I] compatible with gate_up_weight; "
            f"expected {want_down}, got {tuple(down_weight.shape)}"
        )

    if hidden_states.dtype not in SUPPORTED_DTYPES:
        raise TypeError("hidden_states dtype must be float32, float16, or bfloat16")
    for other in (expert_weights, gate_up_weight, down_weight):
        if other.dtype != hidden_states.dtype:
            raise TypeError("all floating-point inputs must have the same dtype")
    for name, value in named.items():
        anchor = hidden_states
        if expert_weights_on_other_device and name in ("gate_up_weight", "down_weight"):
            anchor = gate_up_weight
        if value.device != anchor.device:
            raise ValueError("all inputs must be on the same device")
    for value in named.values():
        if not value.is_contiguous():
            raise ValueError("all inputs must be contiguous")

    return RoutedMoEShape(tokens, num_experts, slots, hidden, inter)


def normalize_backend(backend: object) -> str:
    """Accepted backend names (b300_moe.py:350-357 plus the native name).

    ``cutlass_bf16`` is accepted as the drop-in alias of this library's one
    BF16 path (``b200_bf16``).  ``torch`` is a known name, but the pure-PyTorch
    path is the oracle and is not shipped as an execution path.
    """

    if not isinstance(backend, str):
        raise TypeError("backend must be a string")
    if backend not in BACKENDS:
        raise ValueError(
            "backend must be 'torch', 'cutlass_bf16', 'cutlass_nvfp4', or 'b200_bf16'"
        )
    return backend


def normalize_quant_mode(backend: str, quant_mode: object, dtype: torch.dtype) -> str:
    """Backend/quantisation pairing rules (b300_moe.py:360-384)."""

    if quant_mode is None:
        quant_mode = {
            "torch": "none",
            "cutlass_bf16": "bf16",
            "b200_bf16": "bf16",
            "cutlass_nvfp4": "nvfp4",
        }[backend]
    if not isinstance(quant_mode, str):
        raise TypeError("quant_mode must be a string or None")
    if quant_mode not in QUANT_MODES:
        raise ValueError("quant_mode must be 'none', 'bf16', or 'nvfp4'")
    if backend == "torch":
        if quant_mode == "nvfp4":
            raise ValueError(
                "backend='torch' cannot execute NVFP4; select cutlass_nvfp4 explicitly"
            )
        if quant_mode == "bf16" and dtype != torch.bfloat16:
            raise TypeError("torch quant_mode='bf16' requires bfloat16 inputs")
    elif backend in ("cutlass_bf16", "b200_bf16"):
        if quant_mode != "bf16":
            raise ValueError(f"{backend} requires quant_mode='bf16'")
    elif quant_mode != "nvfp4":
        raise ValueError("cutlass_nvfp4 requires quant_mode='nvfp4'")
    return quant_mode


def normalize_gemm_policy(policy: object) -> str:
    """``gemm_policy`` is validated for compatibility (gemm_dispatch.py:44-51).

    The reference uses it to choose between its grouped kernel and a host loop
    of per-expert matmuls; this library has one grouped kernel, so the value
    only travels into the metadata.
    """

    if not isinstance(policy, str):
        raise TypeError("gemm_policy must be a string")
    if policy not in GEMM_POLICIES:
        raise ValueError("gemm_policy must be 'auto', 'grouped', or 'per_expert'")
    return policy
