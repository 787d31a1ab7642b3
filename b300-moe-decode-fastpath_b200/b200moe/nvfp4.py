"""NVFP4 expert weights for the decode layer: 0.5625 bytes per weight to stream.

The reference names this backend and never had it: ``cutlass_nvfp4`` always raises there
(fastpath/b300_moe.py:571-596) and csrc/quantization_kernels.cu:3-6 lists what a real
implementation needs -- a 4-bit E2M1 payload and two levels of scales.  Here the name runs:
``b300_moe_forward(..., backend="cutlass_nvfp4", quant_mode="nvfp4")`` accepts the BF16 weight
tensors of the contract and uses their NVFP4 form, prepared once per weight tensor
(:func:`prepared_nvfp4_weights`); :func:`b300_moe_forward_nvfp4` takes the prepared weights
directly.  BF16 is never substituted.

Format (published NVFP4): element E2M1 (0, 0.5, 1, 1.5, 2, 3, 4, 6 and negatives, two per
byte), one unsigned-E4M3 scale per 16 elements of the reduction dimension, one FP32 scale per
expert matrix; ``weight = tensor_scale * block_scale * element``.  The weights feed
``tcgen05.mma kind::mxf4nvf4.block_scale`` as they are.  That instruction needs E2M1 on both
sides, so every token row is held as four E2M1 planes in fixed point (plane p rounds, in a unit
eight times finer, what planes 0..p-1 left over), all accumulated in FP32; the layer
equals the FP32 reference evaluated on the dequantised weights within the usual 2e-2 x RMS bar.
"""

from __future__ import annotations

import ctypes
import threading
import weakref
from dataclasses import dataclass

import torch

from . import _lib
from .forward import (_check_out, _enqueue, _native_args, _remember_plan, _repeat_call,
                      _resolve_native_backend)
from .validation import RoutedMoEShape, validate_routing
from .workspace import B300MoEWorkspace

PLANES = 4


@dataclass(frozen=True)
class Nvfp4ExpertWeights:
    """Quantised expert weights of one layer (all on one CUDA device, contiguous)."""

    gate_up_q: torch.Tensor            # uint8 [E, 2I, H/2], packed E2M1, gate rows first
    gate_up_block_scale: torch.Tensor  # uint8, 512-byte tiles [E][2][ceil(I/128)][H/64][512]
    gate_up_scale: torch.Tensor        # float32 [E]
    down_q: torch.Tensor               # uint8 [E, H, I/2]
    down_block_scale: torch.Tensor     # uint8 [E][ceil(H/128)][I/64][512]
    down_scale: torch.Tensor           # float32 [E]

    @property
    def num_experts(self) -> int:
        return self.gate_up_q.shape[0]

    @property
    def hidden_size(self) -> int:
        return self.gate_up_q.shape[2] * 2

    @property
    def intermediate_size(self) -> int:
        return self.gate_up_q.shape[1] // 2

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (
            self.gate_up_q, self.gate_up_block_scale, self.gate_up_scale, self.down_q,
            self.down_block_scale, self.down_scale))


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def scale_bytes_per_expert(rows: int, cols: int, halves: int) -> int:
    size = ctypes.c_size_t(0)
    _lib.check(_lib.load().b200moe_nvfp4_scale_bytes(rows, cols, halves, ctypes.byref(size)),
               "b200moe_nvfp4_scale_bytes")
    return int(size.value)


def quantize_matrix_nvfp4(weights: torch.Tensor, halves: int
                          ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """BF16 ``[E, halves * rows, cols]`` -> ``(packed uint8 [E, halves * rows, cols / 2],
    block scales uint8 [E, bytes], tensor scales float32 [E])`` by ``b200moe_nvfp4_quantize``.
    ``halves`` = 2 for the gate+up matrix (gate and up get separate scale tilings), 1 for down."""

    if weights.device.type != "cuda" or weights.dtype != torch.bfloat16:
        raise TypeError("quantize_matrix_nvfp4 needs a CUDA bfloat16 tensor")
    if weights.ndim != 3 or not weights.is_contiguous():
        raise ValueError("weights must be a contiguous [E, rows, cols] tensor")
    experts, all_rows, cols = weights.shape
    if cols % 64 or all_rows % halves:
        raise ValueError("the reduction dimension must be a multiple of 64")
    rows = all_rows // halves
    device = weights.device
    packed = torch.empty(experts, all_rows, cols // 2, dtype=torch.uint8, device=device)
    sf = torch.zeros(experts, scale_bytes_per_expert(rows, cols, halves), dtype=torch.uint8,
                     device=device)
    tensor_scale = torch.empty(experts, dtype=torch.float32, device=device)
    amax = torch.empty(experts, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        code = _lib.load().b200moe_nvfp4_quantize(
            weights.data_ptr(), experts, rows, cols, halves, packed.data_ptr(), sf.data_ptr(),
            tensor_scale.data_ptr(), amax.data_ptr(), _stream(device))
    _lib.check(code, "b200moe_nvfp4_quantize")
    return packed, sf, tensor_scale


def quantize_expert_weights_nvfp4(gate_up_weight: torch.Tensor, down_weight: torch.Tensor
                                  ) -> Nvfp4ExpertWeights:
    """BF16 ``[E,2I,H]`` / ``[E,H,I]`` expert weights -> their NVFP4 form (run once at load time)."""

    if gate_up_weight.ndim != 3 or down_weight.ndim != 3:
        raise ValueError("expert weights must be [E, 2I, H] and [E, H, I]")
    experts, two_i, hidden = gate_up_weight.shape
    if two_i % 2 or tuple(down_weight.shape) != (experts, hidden, two_i // 2):
        raise ValueError("down_weight must have shape [E, H, I] compatible with gate_up_weight")
    gq, gsf, gs = quantize_matrix_nvfp4(gate_up_weight, 2)
    dq, dsf, ds = quantize_matrix_nvfp4(down_weight, 1)
    return Nvfp4ExpertWeights(gq, gsf, gs, dq, dsf, ds)


def rows_to_planes_nvfp4(rows: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """FP32 ``[R, C]`` rows -> ``(planes uint8 [4, R, C/2], row scale float32 [R])`` by the
    rule the kernels use for token rows: ``row ~= t * (p0 + p1/8 + p2/64 + p3/512)`` (for
    tests)."""

    if rows.device.type != "cuda" or rows.dtype != torch.float32 or rows.ndim != 2 or \
            not rows.is_contiguous():
        raise TypeError("rows_to_planes_nvfp4 needs a contiguous CUDA float32 [R, C] tensor")
    count, cols = rows.shape
    planes = torch.empty(PLANES, count, cols // 2, dtype=torch.uint8, device=rows.device)
    row_scale = torch.empty(count, dtype=torch.float32, device=rows.device)
    with torch.cuda.device(rows.device):
        code = _lib.load().b200moe_nvfp4_rows_to_planes(
            rows.data_ptr(), count, cols, planes.data_ptr(), row_scale.data_ptr(),
            _stream(rows.device))
    _lib.check(code, "b200moe_nvfp4_rows_to_planes")
    return planes, row_scale


# ---------------------------------------------------------------------------------------
# prepared weights of BF16 tensors handed to b300_moe_forward(backend="cutlass_nvfp4")
# ---------------------------------------------------------------------------------------
_prepared_lock = threading.Lock()
_prepared: dict[tuple, tuple[weakref.ref, weakref.ref, Nvfp4ExpertWeights]] = {}


def prepared_nvfp4_weights(gate_up_weight: torch.Tensor, down_weight: torch.Tensor
                           ) -> Nvfp4ExpertWeights:
    """The NVFP4 form of a pair of BF16 weight tensors, quantised on first use and kept for as
    long as both tensors live and are not modified in place (their storage address, shape and
    version counter are the key).  ``b300_moe_forward(backend="cutlass_nvfp4")`` goes through
    here, so the contract's BF16 weight arguments keep working; servers that want control
    over when the quantisation runs call :func:`quantize_expert_weights_nvfp4` at load time
    and :func:`b300_moe_forward_nvfp4` per step."""

    key = (gate_up_weight.data_ptr(), down_weight.data_ptr(), tuple(gate_up_weight.shape),
           gate_up_weight._version, down_weight._version, gate_up_weight.device)
    with _prepared_lock:
        entry = _prepared.get(key)
        if entry is not None and entry[0]() is gate_up_weight and entry[1]() is down_weight:
            return entry[2]
        for stale in [k for k, e in _prepared.items() if e[0]() is None or e[1]() is None]:
            del _prepared[stale]
        weights = quantize_expert_weights_nvfp4(gate_up_weight, down_weight)
        _prepared[key] = (weakref.ref(gate_up_weight), weakref.ref(down_weight), weights)
        return weights


def _validate(hidden_states, expert_indices, expert_weights, weights: Nvfp4ExpertWeights,
              num_experts: int, top_k: int) -> RoutedMoEShape:
    if not isinstance(weights, Nvfp4ExpertWeights):
        raise TypeError("weights must be an Nvfp4ExpertWeights")
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
    if hidden % 64 or inter % 64:
        raise ValueError("the NVFP4-weight path requires hidden_size and intermediate_size "
                         "divisible by 64")
    if tuple(weights.down_q.shape) != (num_experts, hidden, inter // 2):
        raise ValueError("down_q must have shape [E, H, I/2] compatible with gate_up_q")
    want_gsf = scale_bytes_per_expert(inter, hidden, 2)
    want_dsf = scale_bytes_per_expert(hidden, inter, 1)
    if tuple(weights.gate_up_block_scale.shape) != (num_experts, want_gsf) or \
            tuple(weights.down_block_scale.shape) != (num_experts, want_dsf):
        raise ValueError("block scales do not have the size of this geometry's scale tiles")
    if tuple(weights.gate_up_scale.shape) != (num_experts,) or \
            tuple(weights.down_scale.shape) != (num_experts,):
        raise ValueError("tensor scales must have shape [E]")
    byte_tensors = (weights.gate_up_q, weights.down_q, weights.gate_up_block_scale,
                    weights.down_block_scale)
    if any(t.dtype != torch.uint8 for t in byte_tensors):
        raise TypeError("quantised weights and block scales must have dtype torch.uint8")
    if weights.gate_up_scale.dtype != torch.float32 or weights.down_scale.dtype != torch.float32:
        raise TypeError("tensor scales must have dtype torch.float32")
    if hidden_states.dtype != torch.bfloat16 or expert_weights.dtype != torch.bfloat16:
        raise TypeError("the NVFP4-weight path requires bfloat16 activations and routing weights")
    tensors = (hidden_states, expert_indices, expert_weights) + byte_tensors + (
        weights.gate_up_scale, weights.down_scale)
    if any(t.device != hidden_states.device for t in tensors):
        raise ValueError("all inputs must be on the same device")
    if not all(t.is_contiguous() for t in tensors):
        raise ValueError("all inputs must be contiguous")
    return RoutedMoEShape(tokens, num_experts, slots, hidden, inter)


def b300_moe_forward_nvfp4(
    hidden_states: torch.Tensor,
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    weights: Nvfp4ExpertWeights,
    *,
    num_experts: int,
    top_k: int,
    workspace: B300MoEWorkspace | None = None,
    return_metadata: bool = False,
    check_status: bool = False,
    use_pdl: bool = True,
    backend_name: str = "cutlass_nvfp4",
    out: torch.Tensor | None = None,
) -> torch.Tensor | tuple[torch.Tensor, dict[str, object]]:
    """The layer of :func:`b300_moe_forward` with NVFP4 expert weights.

    Same routing contract, workspace protocol and metadata; ``metadata["backend"]`` echoes
    ``backend_name`` and ``quant_mode`` is ``"nvfp4"``.  Segments are 64 rows long (128 in
    the BF16 path), which only changes how the work is cut, not any result tensor.
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
                                weights.gate_up_q, weights.down_q, num_experts, top_k, "nvfp4",
                                "nvfp4", None, use_pdl, weights, out)
        if repeated is not None:
            return repeated
    shape = _validate(hidden_states, expert_indices, expert_weights, weights, num_experts, top_k)
    if workspace is not None and not isinstance(workspace, B300MoEWorkspace):
        raise TypeError("workspace must be a B300MoEWorkspace or None")
    build_info = _resolve_native_backend(
        "b200_nvfp4", hidden_states, expert_weights, weights.gate_up_scale, weights.down_scale,
        shape)
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
        flags = _lib.FLAG_NVFP4_WEIGHTS | (_lib.FLAG_PDL if use_pdl else 0)
        args = _native_args(hidden_states, expert_indices, expert_weights, weights.gate_up_q,
                            weights.down_q, shape, active, output, flags)
        args.gate_up_scale = weights.gate_up_scale.data_ptr()
        args.down_scale = weights.down_scale.data_ptr()
        args.gate_up_block_scale = weights.gate_up_block_scale.data_ptr()
        args.down_block_scale = weights.down_block_scale.data_ptr()
        code = _enqueue(_lib.load().b200moe_forward, args, hidden_states.device)
        if code:
            _lib.check(code, "b200moe_forward")
        metadata: dict[str, object] | None = None
        if return_metadata:
            buffers = active.buffers
            rows = shape.num_assignments
            metadata = {
                "backend": backend_name,
                "architecture": "sm_100a",
                "quant_mode": "nvfp4",
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
                           weights.down_q, num_experts, top_k, "nvfp4", "nvfp4", None, use_pdl,
                           shape, flags, weights)
        if check_status:
            active.raise_for_status()
    if return_metadata:
        assert metadata is not None
        return output, metadata
    return output
