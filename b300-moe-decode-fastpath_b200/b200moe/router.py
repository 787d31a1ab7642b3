"""Router front end on the GPU: ``topk_routing`` with the reference's semantics.

``baseline/routing.py:48-55`` selects the ``top_k`` largest logits per token with
``torch.topk`` and normalises them with a softmax computed in FP32, cast back to the
logits' dtype.  Here both steps are one kernel (``b200moe_router_topk``); its outputs
feed :func:`b200moe.b300_moe_forward` directly.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


def topk_routing(router_logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``(expert_indices [T,K] int64, expert_weights [T,K] logits.dtype)``.

    Indices are in descending logit order; equal logits resolve to the lower expert id.
    Checks follow ``_validate_logits`` (baseline/routing.py:34-45).
    """

    if router_logits.ndim != 2:
        raise ValueError(
            f"router_logits must have shape [num_tokens, num_experts], got "
            f"{tuple(router_logits.shape)}"
        )
    tokens, experts = router_logits.shape
    if tokens < 1 or experts < 1:
        raise ValueError("router_logits must contain at least one token and expert")
    if not router_logits.is_floating_point():
        raise TypeError("router_logits must use a floating-point dtype")
    if isinstance(top_k, bool) or not isinstance(top_k, int) or not 1 <= top_k <= experts:
        raise ValueError(f"top_k must be in [1, {experts}], got {top_k}")
    if router_logits.device.type != "cuda":
        raise ValueError("the native router requires CUDA tensors")
    if router_logits.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("the native router supports float32 and bfloat16 logits")
    if experts > 256 or top_k > 8:
        raise ValueError("the native router supports at most 256 experts and top_k <= 8")
    logits = router_logits.contiguous()
    device = logits.device
    ids = torch.empty(tokens, top_k, dtype=torch.int64, device=device)
    weights = torch.empty(tokens, top_k, dtype=logits.dtype, device=device)
    is_f32 = logits.dtype == torch.float32
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    with torch.cuda.device(device):
        code = _lib.load().b200moe_router_topk(
            logits.data_ptr(), 1 if is_f32 else 0, tokens, experts, top_k, ids.data_ptr(),
            None if is_f32 else weights.data_ptr(), weights.data_ptr() if is_f32 else None, stream,
        )
    _lib.check(code, "b200moe_router_topk")
    return ids, weights
