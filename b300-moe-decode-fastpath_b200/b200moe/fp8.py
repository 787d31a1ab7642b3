"""FP8 (E4M3) expert weights for the decode layer: half the bytes to stream per forward.

No counterpart in the reference: its quantised backend name (``cutlass_nvfp4``) always
raises (fastpath/b300_moe.py:571-596) and FP8/NVFP4 weights are listed as future work
(docs/goal_1b_report.md:313-314).  ``b300_moe_forward(backend="cutlass_nvfp4")`` keeps
raising here too; this module is a separate, explicitly named entry point and never stands
in for another backend.

Format: one E4M3 byte per weight plus one FP32 scale per weight row
(``scale = max|row| / 448``).  Routing, routing weights, accumulation (FP32) and the output
stay as in the BF16 path.  The weights feed ``tcgen05.mma kind::f8f6f4`` as they are; the
token rows are split into E4M3 planes (two exact planes for the BF16 hidden rows, three for
the activation rows: twelve significant bits, BF16 has eight) and the scales are applied to
the FP32 accumulators, so the layer equals the FP32 reference evaluated on the dequantised
weights within the usual 2e-2 x RMS bar.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .forward import (_check_out, _enqueue, _native_args, _remember_plan, _repeat_call,
                      _resolve_native_backend)
from .validation import RoutedMoEShape, validate_routing
from .workspace import B300MoEWorkspace


@dataclass(frozen=True)
class Fp8ExpertWeights:
    """Quantised expert weights of one layer (all on one CUDA device, contiguous)."""

    gate_up_q: torch.Tensor      # uint8 [E, 2I, H], E4M3 codes, gate rows first
    gate_up_scale: torch.Tensor  # float32 [E, 2I]
    down_q: torch.Tensor         # uint8 [E, H, I]
    down_scale: torch.Tensor     # float32 [E, H]

    @property
    def num_experts(self) -> int:
        return self.gate_up_q.shape[0]

    @property
    def hidden_size(self) -> int:
        return self.gate_up_q.shape[2]

    @property
    def intermediate_size(self) -> int:
        return self.gate_up_q.shape[1] // 2

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.gate_up_q, self.gate_up_scale, self.down_q, self.down_scale))


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def quantize_rows_fp8(weights: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 ``[..., rows, cols]`` -> (uint8 E4M3 codes of the same shape, FP32 ``[..., rows]``
    scales) by ``b200moe_fp8_quantize_rows``.  ``cols`` must be a multiple of 16."""

    if weights.device.type != "cuda" or weights.dtype != torch.bfloat16:
        raise TypeError("quantize_rows_fp8 needs a CUDA bfloat16 tensor")
    if not weights.is_contiguous():
        raise ValueError("weights must be contiguous")
    if weights.ndim < 2 or weights.shape[-1] % 16:
        raise ValueError("the last dimension must be a multiple of 16")
    cols = weights.shape[-1]
    rows = weights.numel() // cols
    q = torch.empty(weights.shape, dtype=torch.uint8, device=weights.device)
    scale = torch.empty(weights.shape[:-1], dtype=torch.float32, device=weights.device)
    with torch.cuda.device(weights.device):
        code = _lib.load().b200moe_fp8_quantize_rows(
            weights.data_ptr(), rows, cols, q.data_ptr(), scale.data_ptr(), _stream(weights.device))
    _lib.check(code, "b200moe_fp8_quantize_rows")
    return q, scale


def dequantize_rows_fp8(q: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    """E4M3 codes (+ per-row scales, or ``None`` for the bare E4M3 values) -> BF16.  For
    inspection and tests; the GEMM kernels consume the E4M3 bytes as they are."""

    if q.device.type != "cuda" or q.dtype != torch.uint8 or not q.is_contiguous():
        raise TypeError("dequantize_rows_fp8 needs a contiguous CUDA uint8 tensor")
    cols = q.shape[-1]
    if cols % 16:
        raise ValueError("the last dimension must be a multiple of 16")
    rows = q.numel() // cols
    if scale is not None:
        if scale.dtype != torch.float32 or scale.numel() != rows or not scale.is_contiguous():
            raise ValueError("scale must be contiguous float32 with one entry per row")
    out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        code = _lib.load().b200moe_fp8_dequantize_rows(
            q.data_ptr(), scale.data_ptr() if scale is not None else None, rows, cols,
            out.data_ptr(), _stream(q.device))
    _lib.check(code, "b200moe_fp8_dequantize_rows")
    return out


def quantize_expert_weights_fp8(gate_up_weight: torch.Tensor,
                                down_weight: torch.Tensor) -> Fp8ExpertWeights:
    """Quantise a layer's BF16 expert weights (``[E,2I,H]``, ``[E,H,I]``) once, at load time."""

    if gate_up_weight.ndim != 3 or down_weight.ndim != 3:
        raise ValueError("gate_up_weight must be [E,2I,H] and down_weight [E,H,I]")
    experts, two_i, hidden = gate_up_weight.shape
    if two_i % 2 or tuple(down_weight.shape) != (experts, hidden, two_i // 2):
        raise ValueError("down_weight must have shape [E, H, I] compatible with gate_up_weight")
    gq, gs = quantize_rows_fp8(gate_up_weight)
    dq, ds = quantize_rows_fp8(down_weight)
    return Fp8ExpertWeights(gq, gs, dq, ds)


def dequantize_expert_weights_fp8(weights: Fp8ExpertWeights) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 ``bf16(E4M3 value * scale)`` tensors (rounded once; the FP8 kernels themselves
    keep the scale in FP32 and do not round)."""

    return (dequantize_rows_fp8(weights.gate_up_q, weights.gate_up_scale),
            dequantize_rows_fp8(weights.down_q, weights.down_scale))


def _validate(hidden_states, expert_indices, expert_weights, weights: Fp8ExpertWeights,
              num_experts: int, top_k: int, *, weights_on_other_device: bool = False
              ) -> RoutedMoEShape:
    """Contract of the FP8-weight entry points.  ``weights_on_other_device`` relaxes the
    one-device rule for the pinned-host variant: the three per-step tensors share a device
    and the four weight tensors share a device."""

    if not isinstance(weights, Fp8ExpertWeights):
        raise TypeError("weights must be an Fp8ExpertWeights")
    tokens, slots = validate_routing(expert_indices, expert_weights, num_experts, top_k)
    if not isinstance(hidden_states, torch.Tensor):
        raise TypeError("hidden_states must be a torch.Tensor")
    if hidden_states.ndim != 2 or hidden_states.shape[0] != tokens:
        raise ValueError("hidden_states must have shape [num_tokens, hidden_size]")
    if weights.gate_up_q.ndim != 3 or weights.gate_up_q.shape[0] != num_experts:
        raise ValueError("gate_up_q.shape[0] must equal num_experts")
    hidden, inter = weights.hidden_size, weights.intermediate_size
    if hidden_states.shape[1] != hidden:
        raise ValueError("gate_up_q hidden dimension must match hidden_states")
    if weights.gate_up_q.shape[1] % 2:
        raise ValueError("gate_up_q dimension 1 must be an even size 2I")
    if tuple(weights.down_q.shape) != (num_experts, hidden, inter):
        raise ValueError("down_q must have shape [E, H, I] compatible with gate_up_q")
    if tuple(weights.gate_up_scale.shape) != (num_experts, 2 * inter) or \
            tuple(weights.down_scale.shape) != (num_experts, hidden):
        raise ValueError("scales must have shapes [E, 2I] and [E, H]")
    if weights.gate_up_q.dtype != torch.uint8 or weights.down_q.dtype != torch.uint8:
        raise TypeError("quantised weights must have dtype torch.uint8 (E4M3 codes)")
    if weights.gate_up_scale.dtype != torch.float32 or weights.down_scale.dtype != torch.float32:
        raise TypeError("scales must have dtype torch.float32")
    if hidden_states.dtype != torch.bfloat16 or expert_weights.dtype != torch.bfloat16:
        raise TypeError("the FP8-weight path requires bfloat16 activations and routing weights")
    per_step = (hidden_states, expert_indices, expert_weights)
    resident = (weights.gate_up_q, weights.gate_up_scale, weights.down_q, weights.down_scale)
    tensors = per_step + resident
    anchor = weights.gate_up_q.device if weights_on_other_device else hidden_states.device
    if any(t.device != hidden_states.device for t in per_step) or \
            any(t.device != anchor for t in resident):
        raise ValueError("all inputs must be on the same device")
    if not all(t.is_contiguous() for t in tensors):
        raise ValueError("all inputs must be contiguous")
    if hidden % 16 or inter % 16:
        raise ValueError("the FP8-weight path requires hidden_size and intermediate_size "
                         "divisible by 16")
    return RoutedMoEShape(tokens, num_experts, slots, hidden, inter)


def b300_moe_forward_fp8(
    hidden_states: torch.Tensor,
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    weights: Fp8ExpertWeights,
    *,
    num_experts: int,
    top_k: int,
    workspace: B300MoEWorkspace | None = None,
    return_metadata: bool = False,
    check_status: bool = False,
    use_pdl: bool = True,
    out: torch.Tensor | None = None,
) -> torch.Tensor | tuple[torch.Tensor, dict[str, object]]:
    """The layer of :func:`b300_moe_forward` with FP8 expert weights.

    Same routing contract, workspace protocol and metadata; ``metadata["backend"]`` is
    ``"b200_fp8"`` and ``quant_mode`` ``"fp8_e4m3_per_row"``.  Segments are 64 rows long
    (128 in the BF16 path), which only changes how the work is cut, not any result tensor.
    ``out``: as in :func:`b300_moe_forward`.
    """

    if not isinstance(return_metadata, bool):
        raise TypeError("return_metadata must be a bool")
    if out is not None and isinstance(hidden_states, torch.Tensor):
        _check_out(out, hidden_states)
    if workspace is not None and not return_metadata and not check_status and \
            type(workspace) is B300MoEWorkspace and hasattr(weights, "gate_up_q"):
        # a call that repeats the last fully checked one on this workspace (forward._CallPlan)
        repeated = _repeat_call(workspace, hidden_states, expert_indices, expert_weights,
                                weights.gate_up_q, weights.down_q, num_experts, top_k, "fp8",
                                "fp8", None, use_pdl, weights, out)
        if repeated is not None:
            return repeated
    shape = _validate(hidden_states, expert_indices, expert_weights, weights, num_experts, top_k)
    if workspace is not None and not isinstance(workspace, B300MoEWorkspace):
        raise TypeError("workspace must be a B300MoEWorkspace or None")
    build_info = _resolve_native_backend(
        "b200_fp8", hidden_states, expert_weights, weights.gate_up_scale, weights.down_scale, shape)
    active = workspace if workspace is not None else B300MoEWorkspace(device=hidden_states.device)
    with active._lock:
        reused = active.reserve(
            num_tokens=shape.num_tokens, num_experts=shape.num_experts, top_k=shape.top_k,
            hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size,
            device=hidden_states.device, dtype=hidden_states.dtype, backend="b200_bf16",
            quant_mode="bf16",
        )
        output = out if out is not None else \
            torch.empty_like(hidden_states, memory_format=torch.contiguous_format)
        flags = _lib.FLAG_FP8_WEIGHTS | (_lib.FLAG_PDL if use_pdl else 0)
        args = _native_args(hidden_states, expert_indices, expert_weights, weights.gate_up_q,
                            weights.down_q, shape, active, output, flags)
        args.gate_up_scale = weights.gate_up_scale.data_ptr()
        args.down_scale = weights.down_scale.data_ptr()
        code = _enqueue(_lib.load().b200moe_forward, args, hidden_states.device)
        if code:
            _lib.check(code, "b200moe_forward")
        metadata: dict[str, object] | None = None
        if return_metadata:
            buffers = active.buffers
            rows = shape.num_assignments
            metadata = {
                "backend": "b200_fp8",
                "architecture": "sm_100a",
                "quant_mode": "fp8_e4m3_per_row",
                "used_fallback": False,
                "expert_counts": buffers["expert_counts"][: shape.num_experts].clone(),
                "expert_offsets": buffers["expert_offsets"][: shape.num_experts + 1].clone(),
                "permutation": buffers["permutation"][:rows].clone(),
                "reverse_mapping": buffers["reverse_mapping"][:rows].clone(),
                "workspace": {
                    "capacity_tokens": active.capacity_tokens,
                    "capacity_assignments": active.capacity_assignments,
                    "capacity_bytes": active.capacity_bytes,
                    "allocation_count": active.allocation_count,
                    "reuse_count": active.reuse_count,
                    "reused": reused,
                    "shape_signature": active.shape_signature,
                },
                "build": dict(build_info),
                "weight_bytes": weights.nbytes,
            }
        active._record_use()
        if workspace is not None:
            _remember_plan(active, hidden_states, expert_indices, weights.gate_up_q,
                           weights.down_q, num_experts, top_k, "fp8", "fp8", None, use_pdl,
                           shape, flags, weights)
        if check_status:
            active.raise_for_status()
    if return_metadata:
        assert metadata is not None
        return output, metadata
    return output
