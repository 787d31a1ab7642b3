"""The decode layer packaged as replayable CUDA graphs, one per token count.

The reference lists "one persistent kernel or CUDA-graph packaging" of the layer as future
work and notes that its compiled path cannot be captured because the library GEMM allocates
(docs/goal_1b_report.md:189-194, 315-320).  The kernels here allocate nothing and never
synchronise, so a forward can be captured; this module does the bookkeeping a decode loop
needs around that: static input/output buffers per token count, one shared workspace,
capture after a warm-up call, and replay on the caller's stream.

A replay costs one launch call on the host instead of five or six plus the Python in
between, and computes bit-identical results to the eager call.
"""

from __future__ import annotations

import torch

from .forward import b300_moe_forward
from .fp8 import Fp8ExpertWeights, b300_moe_forward_fp8
from .router import topk_routing
from .workspace import B300MoEWorkspace


class GraphedMoEDecodeLayer:
    """Expert weights of one layer plus captured graphs of its forward for fixed token counts.

    ``gate_up_weight`` / ``down_weight`` are the BF16 tensors of :func:`b300_moe_forward`,
    or pass ``fp8_weights`` (an :class:`Fp8ExpertWeights`) instead.  ``token_counts`` are the
    batch sizes to capture; a call with another size runs eagerly.  With ``route_logits=True``
    the graph also holds the router front end: the call takes ``[T, E]`` router logits (BF16
    or FP32) and runs top-k + softmax + layer in one replay.

    Outputs are static buffers owned by the layer: a result is valid until the next call with
    the same token count (pass ``copy=True`` for a fresh tensor).  Calls are not thread-safe;
    replays are ordered on the current stream like any other work.
    """

    def __init__(
        self,
        gate_up_weight: torch.Tensor | None,
        down_weight: torch.Tensor | None,
        *,
        num_experts: int,
        top_k: int,
        token_counts: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64),
        fp8_weights: Fp8ExpertWeights | None = None,
        route_logits: bool = False,
        logits_dtype: torch.dtype = torch.bfloat16,
    ) -> None:
        if fp8_weights is not None:
            if not isinstance(fp8_weights, Fp8ExpertWeights):
                raise TypeError("fp8_weights must be an Fp8ExpertWeights")
            device, hidden = fp8_weights.gate_up_q.device, fp8_weights.hidden_size
        else:
            if gate_up_weight is None or down_weight is None:
                raise ValueError("pass gate_up_weight and down_weight, or fp8_weights")
            device, hidden = gate_up_weight.device, gate_up_weight.shape[2]
        if device.type != "cuda":
            raise ValueError("GraphedMoEDecodeLayer requires CUDA weights")
        if not token_counts or any((not isinstance(t, int)) or t < 1 for t in token_counts):
            raise ValueError("token_counts must be positive integers")
        self.gate_up_weight, self.down_weight, self.fp8_weights = gate_up_weight, down_weight, fp8_weights
        self.num_experts, self.top_k, self.hidden_size = num_experts, top_k, hidden
        self.route_logits = route_logits
        self.device = device
        # the captured graphs hold the addresses of this workspace's buffers, so it must never
        # be reallocated: calls with other token counts run on a second workspace
        self.workspace = B300MoEWorkspace(capacity_tokens=max(token_counts), device=device)
        self._eager_workspace = B300MoEWorkspace(device=device)
        self._static: dict[int, dict[str, object]] = {}
        self.replays = 0
        self.eager_calls = 0
        for tokens in sorted(set(token_counts)):
            self._capture(tokens, logits_dtype)

    # ------------------------------------------------------------------ internals
    def _eager(self, hidden, ids, weights, workspace=None):
        workspace = workspace if workspace is not None else self.workspace
        if self.fp8_weights is not None:
            return b300_moe_forward_fp8(hidden, ids, weights, self.fp8_weights,
                                        num_experts=self.num_experts, top_k=self.top_k,
                                        workspace=workspace)
        return b300_moe_forward(hidden, ids, weights, self.gate_up_weight, self.down_weight,
                                num_experts=self.num_experts, top_k=self.top_k,
                                backend="cutlass_bf16", workspace=workspace)

    def _run(self, slot):
        if self.route_logits:
            ids, weights = topk_routing(slot["logits"], self.top_k)
            if weights.dtype != torch.bfloat16:
                weights = weights.to(torch.bfloat16)
            slot["ids"], slot["weights"] = ids, weights
        return self._eager(slot["hidden"], slot["ids"], slot["weights"])

    def _capture(self, tokens: int, logits_dtype: torch.dtype) -> None:
        dev = self.device
        slot: dict[str, object] = {
            "hidden": torch.zeros(tokens, self.hidden_size, dtype=torch.bfloat16, device=dev),
        }
        if self.route_logits:
            # distinct logits so that the warm-up routes like a real call
            slot["logits"] = torch.arange(self.num_experts, device=dev).flip(0).to(logits_dtype) \
                .repeat(tokens, 1).contiguous()
        else:
            base = torch.arange(self.top_k, device=dev, dtype=torch.int64) % self.num_experts
            slot["ids"] = base.repeat(tokens, 1).contiguous()
            slot["weights"] = torch.full((tokens, self.top_k), 1.0 / self.top_k,
                                         dtype=torch.bfloat16, device=dev)
        with torch.cuda.device(dev):
            self._run(slot)                       # warm-up: workspace reserved, maps encoded
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                slot["output"] = self._run(slot)
        slot["graph"] = graph
        self._static[tokens] = slot

    # ------------------------------------------------------------------ calls
    @property
    def token_counts(self) -> tuple[int, ...]:
        return tuple(sorted(self._static))

    def __call__(self, hidden_states: torch.Tensor, expert_indices: torch.Tensor,
                 expert_weights: torch.Tensor, *, copy: bool = False) -> torch.Tensor:
        """Explicitly routed call (layers built with ``route_logits=False``)."""

        if self.route_logits:
            raise ValueError("this layer was captured with the router inside: call forward_logits")
        slot = self._static.get(hidden_states.shape[0])
        if slot is None:
            self.eager_calls += 1
            return self._eager(hidden_states, expert_indices, expert_weights,
                               self._eager_workspace)
        slot["hidden"].copy_(hidden_states, non_blocking=True)
        slot["ids"].copy_(expert_indices, non_blocking=True)
        slot["weights"].copy_(expert_weights, non_blocking=True)
        slot["graph"].replay()
        self.replays += 1
        return slot["output"].clone() if copy else slot["output"]

    def forward_logits(self, hidden_states: torch.Tensor, router_logits: torch.Tensor, *,
                       copy: bool = False) -> torch.Tensor:
        """Router logits in, layer output out (layers built with ``route_logits=True``)."""

        if not self.route_logits:
            raise ValueError("this layer was captured without the router: call it with ids and weights")
        slot = self._static.get(hidden_states.shape[0])
        if slot is None:
            self.eager_calls += 1
            ids, weights = topk_routing(router_logits, self.top_k)
            return self._eager(hidden_states, ids, weights.to(torch.bfloat16),
                               self._eager_workspace)
        slot["hidden"].copy_(hidden_states, non_blocking=True)
        slot["logits"].copy_(router_logits, non_blocking=True)
        slot["graph"].replay()
        self.replays += 1
        return slot["output"].clone() if copy else slot["output"]
