"""b200moe: the explicitly routed SwiGLU MoE decode layer on hand-written sm_100a kernels.

Public names follow the reference package (fastpath/__init__.py:3-9) so that
``from fastpath import B300MoEWorkspace, b300_moe_forward`` becomes
``from b200moe import B300MoEWorkspace, b300_moe_forward``.
"""

from ._lib import available as cuda_extension_available
from ._lib import build_info
from .forward import ARCHITECTURE, b300_moe_forward, b300_moe_forward_pinned
from .fp8 import (Fp8ExpertWeights, b300_moe_forward_fp8, dequantize_expert_weights_fp8,
                  dequantize_rows_fp8, quantize_expert_weights_fp8, quantize_rows_fp8)
from .graphed import GraphedMoEDecodeLayer
from .nvfp4 import (Nvfp4ExpertWeights, b300_moe_forward_nvfp4, prepared_nvfp4_weights,
                    quantize_expert_weights_nvfp4)
from .ops import DispatchResult, combine_tokens, dispatch_tokens
from .router import topk_routing
from .stages import StagedLayer
from .validation import RoutedMoEShape, validate_routed_moe_inputs
from .workspace import B300MoEWorkspace

__all__ = [
    "ARCHITECTURE",
    "B300MoEWorkspace",
    "DispatchResult",
    "Fp8ExpertWeights",
    "GraphedMoEDecodeLayer",
    "Nvfp4ExpertWeights",
    "RoutedMoEShape",
    "StagedLayer",
    "b300_moe_forward",
    "b300_moe_forward_fp8",
    "b300_moe_forward_nvfp4",
    "b300_moe_forward_pinned",
    "build_info",
    "combine_tokens",
    "cuda_extension_available",
    "dequantize_expert_weights_fp8",
    "dequantize_rows_fp8",
    "dispatch_tokens",
    "prepared_nvfp4_weights",
    "quantize_expert_weights_fp8",
    "quantize_expert_weights_nvfp4",
    "quantize_rows_fp8",
    "topk_routing",
    "validate_routed_moe_inputs",
]
