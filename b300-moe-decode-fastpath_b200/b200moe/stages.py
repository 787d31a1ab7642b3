"""Stage-by-stage access to the native layer, for tests and per-stage timing.

The reference times its stages by calling the extension's staged functions one
by one (benchmark/benchmark_goal_1b.py:389-500).  ``StagedLayer`` does the same
over the C ABI: it binds one set of inputs and one workspace to a
``B200MoeArgs`` struct once and can then enqueue any single stage, or the whole
layer, on the current stream without further Python work.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .forward import _native_args, _resolve_native_backend
from .validation import validate_routed_moe_inputs
from .workspace import B300MoEWorkspace

STAGES = ("routing", "gather", "gate_up_swiglu", "down", "combine")


class StagedLayer:
    """One bound call of the layer whose stages can be enqueued separately."""

    def __init__(
        self,
        hidden_states: torch.Tensor,
        expert_indices: torch.Tensor,
        expert_weights: torch.Tensor,
        gate_up_weight: torch.Tensor | None,
        down_weight: torch.Tensor | None,
        *,
        num_experts: int,
        top_k: int,
        workspace: B300MoEWorkspace | None = None,
        use_pdl: bool = True,
        fp8_weights=None,
        nvfp4_weights=None,
    ) -> None:
        """``fp8_weights`` (an ``Fp8ExpertWeights``) or ``nvfp4_weights`` (an
        ``Nvfp4ExpertWeights``) selects the kernels of that weight format; the two BF16 weight
        arguments are then ignored and may be ``None``."""

        flags = _lib.FLAG_PDL if use_pdl else 0
        if nvfp4_weights is not None:
            from .nvfp4 import _validate as validate_nvfp4

            self.shape = validate_nvfp4(hidden_states, expert_indices, expert_weights,
                                        nvfp4_weights, num_experts, top_k)
            gate_up_weight, down_weight = nvfp4_weights.gate_up_q, nvfp4_weights.down_q
            _resolve_native_backend("b200_nvfp4", hidden_states, expert_weights,
                                    nvfp4_weights.gate_up_scale, nvfp4_weights.down_scale,
                                    self.shape)
            flags |= _lib.FLAG_NVFP4_WEIGHTS
        elif fp8_weights is not None:
            from .fp8 import _validate as validate_fp8

            self.shape = validate_fp8(hidden_states, expert_indices, expert_weights, fp8_weights,
                                      num_experts, top_k)
            gate_up_weight, down_weight = fp8_weights.gate_up_q, fp8_weights.down_q
            _resolve_native_backend("b200_fp8", hidden_states, expert_weights,
                                    fp8_weights.gate_up_scale, fp8_weights.down_scale, self.shape)
            flags |= _lib.FLAG_FP8_WEIGHTS
        else:
            self.shape = validate_routed_moe_inputs(
                hidden_states,
                expert_indices,
                expert_weights,
                gate_up_weight,
                down_weight,
                num_experts=num_experts,
                top_k=top_k,
            )
            _resolve_native_backend(
                "b200_bf16", hidden_states, expert_weights, gate_up_weight, down_weight, self.shape
            )
        self.device = hidden_states.device
        self.workspace = workspace or B300MoEWorkspace(device=self.device)
        self.workspace.reserve(
            num_tokens=self.shape.num_tokens,
            num_experts=self.shape.num_experts,
            top_k=self.shape.top_k,
            hidden_size=self.shape.hidden_size,
            intermediate_size=self.shape.intermediate_size,
            device=self.device,
            dtype=hidden_states.dtype,
            backend="b200_bf16",
            quant_mode="bf16",
        )
        self.output = torch.empty_like(hidden_states)
        # keep the inputs alive for as long as their addresses sit in the struct
        self._inputs = (hidden_states, expert_indices, expert_weights, gate_up_weight, down_weight,
                        fp8_weights, nvfp4_weights)
        # a private struct: the workspace keeps its own bound struct for forward calls
        self._args = _lib.B200MoeArgs()
        bound = _native_args(
            hidden_states,
            expert_indices,
            expert_weights,
            gate_up_weight,
            down_weight,
            self.shape,
            self.workspace,
            self.output,
            flags,
        )
        ctypes.memmove(ctypes.byref(self._args), ctypes.byref(bound), ctypes.sizeof(bound))
        if fp8_weights is not None:
            self._args.gate_up_scale = fp8_weights.gate_up_scale.data_ptr()
            self._args.down_scale = fp8_weights.down_scale.data_ptr()
        if nvfp4_weights is not None:
            self._args.gate_up_scale = nvfp4_weights.gate_up_scale.data_ptr()
            self._args.down_scale = nvfp4_weights.down_scale.data_ptr()
            self._args.gate_up_block_scale = nvfp4_weights.gate_up_block_scale.data_ptr()
            self._args.down_block_scale = nvfp4_weights.down_block_scale.data_ptr()
        lib = _lib.load()
        self._calls = {
            "routing": lib.b200moe_routing,
            "gather": lib.b200moe_gather,
            "gate_up_swiglu": lib.b200moe_gate_up_swiglu,
            "down": lib.b200moe_down,
            "combine": lib.b200moe_combine,
            "forward": lib.b200moe_forward,
        }

    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def run_stage(self, name: str) -> None:
        """Enqueue one stage (or ``"forward"`` for all five) on the current stream."""

        code = self._calls[name](ctypes.byref(self._args), self._stream())
        _lib.check(code, f"b200moe_{name}")

    def forward(self) -> torch.Tensor:
        self.run_stage("forward")
        return self.output

    def routing_tensors(self) -> dict[str, torch.Tensor]:
        rows = self.shape.num_assignments
        buffers = self.workspace.buffers
        return {
            "expert_counts": buffers["expert_counts"][: self.shape.num_experts],
            "expert_offsets": buffers["expert_offsets"][: self.shape.num_experts + 1],
            "expert_offsets_i32": buffers["expert_offsets_i32"][: self.shape.num_experts],
            "permutation": buffers["permutation"][:rows],
            "reverse_mapping": buffers["reverse_mapping"][:rows],
            "permuted_token_indices": buffers["permuted_token_indices"][:rows],
            "permuted_expert_indices": buffers["permuted_expert_indices"][:rows],
            "permuted_weights": buffers["permuted_weights"][:rows],
        }
