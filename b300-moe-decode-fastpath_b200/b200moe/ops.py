"""The reference's older dispatch / combine API on the sm_100a kernels.

``fastpath/ops.py`` exposes ``dispatch_tokens`` (expert-major grouping of the token rows
with both mappings) and ``combine_tokens`` (reverse-map weighted sum) with a ``torch`` and a
``cuda_ext`` backend.  Here both run the native kernels only: ``dispatch_tokens`` is the
routing kernel plus the gather kernel (``b200moe_dispatch``), ``combine_tokens`` the BF16
combine kernel (``b200moe_combine_bf16``).  ``backend="torch"`` is refused like everywhere
else in this library: the PyTorch formulas are the test oracle.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .forward import _enqueue

_SCRATCH_ALIGN = 256


@dataclass(frozen=True)
class DispatchResult:
    """Same fields as the reference's ``DispatchResult`` (fastpath/ops.py:19-32).

    Assignment ids are token-major (``token * top_k + slot``);
    ``assignment_to_permuted[a]`` is assignment ``a``'s expert-major row and
    ``permuted_to_assignment`` its exact inverse.
    """

    permuted_hidden: torch.Tensor
    expert_counts: torch.Tensor
    expert_offsets: torch.Tensor
    assignment_to_permuted: torch.Tensor
    permuted_to_assignment: torch.Tensor


def _native_backend(backend: str) -> None:
    if backend not in ("torch", "cuda", "cuda_ext"):
        raise ValueError("backend must be 'torch', 'cuda', or 'cuda_ext'")
    if backend == "torch":
        raise RuntimeError(
            "backend='torch' is the reference oracle and is not an execution path of this "
            "library; use backend='cuda_ext'"
        )


def dispatch_tokens(
    hidden_states: torch.Tensor,
    expert_ids: torch.Tensor,
    num_experts: int,
    *,
    backend: str = "cuda_ext",
    validate_values: bool = True,
) -> DispatchResult:
    """Group token assignments by expert (checks follow fastpath/ops.py:78-131).

    ``validate_values`` is accepted for compatibility; ids outside ``[0, E)`` never trap:
    their rows are dropped and show as ``-1`` in the mappings.
    """

    _native_backend(backend)
    if hidden_states.ndim != 2 or expert_ids.ndim != 2:
        raise ValueError("dispatch expects hidden_states [T, H] and expert_ids [T, K]")
    tokens, hidden = hidden_states.shape
    if expert_ids.shape[0] != tokens:
        raise ValueError("hidden_states and expert_ids must have the same num_tokens")
    top_k = expert_ids.shape[1]
    if top_k not in (1, 2, 4, 8):
        raise ValueError(f"top_k must be one of 1, 2, 4, or 8, got {top_k}")
    if isinstance(num_experts, bool) or not isinstance(num_experts, int):
        raise TypeError("num_experts must be an integer")
    if not 1 <= num_experts <= 256:
        raise ValueError("num_experts must be in [1, 256]")
    if expert_ids.dtype != torch.int64:
        raise TypeError("expert_ids must have dtype torch.int64")
    if hidden_states.device.type != "cuda" or expert_ids.device != hidden_states.device:
        raise ValueError("cuda_ext backend requires CUDA tensors on one device")
    if hidden_states.dtype != torch.bfloat16:
        raise TypeError("the native dispatch supports bfloat16 hidden states")
    if hidden % 8:
        raise ValueError("hidden_size must be divisible by 8 (16-byte BF16 alignment)")
    if not (hidden_states.is_contiguous() and expert_ids.is_contiguous()):
        raise ValueError("dispatch inputs must be contiguous")

    device = hidden_states.device
    rows = tokens * top_k
    long = dict(dtype=torch.int64, device=device)
    counts = torch.empty(num_experts, **long)
    offsets = torch.empty(num_experts + 1, **long)
    offsets_i32 = torch.empty(num_experts, dtype=torch.int32, device=device)
    assignment_to_permuted = torch.empty(rows, **long)
    permuted_to_assignment = torch.empty(rows, **long)
    permuted_hidden = torch.empty(rows, hidden, dtype=hidden_states.dtype, device=device)
    need = _lib.dispatch_scratch_bytes(rows, num_experts)
    base = torch.empty(need + _SCRATCH_ALIGN, dtype=torch.uint8, device=device)
    skew = (-base.data_ptr()) % _SCRATCH_ALIGN

    args = _lib.B200MoeArgs()
    args.hidden_states = hidden_states.data_ptr()
    args.expert_indices = expert_ids.data_ptr()
    args.num_tokens, args.top_k, args.num_experts = tokens, top_k, num_experts
    args.hidden_size, args.intermediate_size, args.rows_cap = hidden, 8, rows
    args.expert_counts = counts.data_ptr()
    args.expert_offsets = offsets.data_ptr()
    args.expert_offsets_i32 = offsets_i32.data_ptr()
    args.permutation = permuted_to_assignment.data_ptr()
    args.reverse_mapping = assignment_to_permuted.data_ptr()
    args.permuted_hidden = permuted_hidden.data_ptr()
    args.scratch = base.data_ptr() + skew
    args.scratch_bytes = need
    args.flags = _lib.FLAG_PDL
    code = _enqueue(_lib.load().b200moe_dispatch, args, device)
    if code:
        _lib.check(code, "b200moe_dispatch")
    base.record_stream(torch.cuda.current_stream(device))
    return DispatchResult(permuted_hidden, counts, offsets, assignment_to_permuted,
                          permuted_to_assignment)


def combine_tokens(
    expert_outputs: torch.Tensor,
    assignment_to_permuted: torch.Tensor,
    routing_weights: torch.Tensor,
    *,
    backend: str = "cuda_ext",
    validate_values: bool = True,
) -> torch.Tensor:
    """Weighted sum of each token's expert rows (checks follow fastpath/ops.py:181-239)."""

    _native_backend(backend)
    if expert_outputs.ndim != 2:
        raise ValueError("expert_outputs must have shape [num_assignments, hidden_size]")
    if assignment_to_permuted.ndim != 1:
        raise ValueError("assignment_to_permuted must have shape [num_assignments]")
    if routing_weights.ndim != 2:
        raise ValueError("routing_weights must have shape [num_tokens, top_k]")
    tokens, top_k = routing_weights.shape
    rows, hidden = expert_outputs.shape
    if tokens < 1 or hidden < 1:
        raise ValueError("num_tokens and hidden_size must be positive")
    if top_k not in (1, 2, 4, 8):
        raise ValueError(f"top_k must be one of 1, 2, 4, or 8, got {top_k}")
    if rows != tokens * top_k:
        raise ValueError("expert_outputs first dimension must equal num_tokens * top_k")
    if assignment_to_permuted.numel() != rows:
        raise ValueError("assignment_to_permuted length must equal num_tokens * top_k")
    if expert_outputs.dtype != torch.bfloat16:
        raise TypeError("the native combine supports bfloat16 expert outputs")
    if routing_weights.dtype != expert_outputs.dtype:
        raise TypeError("routing_weights and expert_outputs must have the same dtype")
    if assignment_to_permuted.dtype != torch.int64:
        raise TypeError("assignment_to_permuted must have dtype torch.int64")
    tensors = (expert_outputs, assignment_to_permuted, routing_weights)
    if expert_outputs.device.type != "cuda" or any(t.device != expert_outputs.device
                                                    for t in tensors):
        raise ValueError("cuda_ext backend requires CUDA tensors on one device")
    if any(not t.is_contiguous() for t in tensors):
        raise ValueError("all combine inputs must be contiguous")
    if hidden % 8:
        raise ValueError("hidden_size must be divisible by 8 (16-byte BF16 alignment)")
    device = expert_outputs.device
    output = torch.empty(tokens, hidden, dtype=expert_outputs.dtype, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    with torch.cuda.device(device):
        code = _lib.load().b200moe_combine_bf16(
            expert_outputs.data_ptr(), assignment_to_permuted.data_ptr(),
            routing_weights.data_ptr(), tokens, top_k, hidden, output.data_ptr(), stream)
    _lib.check(code, "b200moe_combine_bf16")
    return output
