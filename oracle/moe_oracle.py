"""CPU oracle for the explicitly routed SwiGLU MoE layer.  TEST INFRASTRUCTURE.

This file is a checker, not a product path: only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / ``--impl reference`` legs of
``bench.py`` may import it.  The library under ``b300-moe-decode-fastpath_b200/``
never does, and fails loudly when its CUDA library is missing.

It restates, in NumPy (integer routing) and CPU PyTorch (dense FP32 algebra),
what the reference's ``backend="torch"`` computes:

* routing metadata      baseline/routing.py:76-99   (``group_tokens``)
* gather                baseline/torch_moe.py:96-99 (``permute_hidden_states``)
* per-expert SwiGLU FFN fastpath/reference.py:268-281, baseline/torch_moe.py:102-120
* weighted combine      baseline/torch_moe.py:123-133 (``combine_expert_outputs``)
* router top-k/softmax  baseline/routing.py:48-55   (``topk_routing``)
* an independent token/slot loop  tests/test_goal_1b_correctness.py:46-63

Parity is pinned: ``tests/golden/*.npz`` hold inputs and outputs produced by
importing the reference itself (``tests/golden/make_golden.py``), and
``tests/test_oracle.py`` checks every function here against them and against
the literal known answers in the reference's own tests.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass(frozen=True)
class Routing:
    """Same fields as the reference's ``RoutingResult`` (baseline/routing.py:14-31)."""

    permutation: np.ndarray  # [A] expert-major row -> assignment
    reverse_mapping: np.ndarray  # [A] assignment -> expert-major row
    permuted_token_indices: np.ndarray  # [A]
    permuted_expert_indices: np.ndarray  # [A]
    expert_counts: np.ndarray  # [E]
    expert_offsets: np.ndarray  # [E+1]


def group_tokens(expert_indices, num_experts: int) -> Routing:
    """Stable expert-major grouping of the flattened [T,K] ids (routing.py:76-99).

    ``permutation`` is the stable argsort of the ids, ``reverse_mapping`` its
    inverse, counts a bincount with ``minlength=E`` and offsets ``[0, cumsum]``,
    so an empty expert has equal adjacent offsets.  All int64.
    """

    ids = np.asarray(
        expert_indices.cpu().numpy() if isinstance(expert_indices, torch.Tensor) else expert_indices
    )
    if ids.ndim != 2:
        raise ValueError("expert_indices must be [T, K]")
    if ids.dtype != np.int64:
        raise TypeError("expert_indices must be int64")
    tokens, top_k = ids.shape
    flat = ids.reshape(-1)
    if flat.size == 0:
        raise ValueError("routing tensors must not be empty")
    if flat.min() < 0 or flat.max() >= num_experts:
        raise ValueError("expert_indices contains an out-of-range expert index")
    permutation = np.argsort(flat, kind="stable").astype(np.int64)
    reverse = np.empty_like(permutation)
    reverse[permutation] = np.arange(flat.size, dtype=np.int64)
    counts = np.bincount(flat, minlength=num_experts).astype(np.int64)
    offsets = np.concatenate([np.zeros(1, np.int64), np.cumsum(counts)]).astype(np.int64)
    flat_tokens = np.repeat(np.arange(tokens, dtype=np.int64), top_k)
    return Routing(
        permutation=permutation,
        reverse_mapping=reverse,
        permuted_token_indices=flat_tokens[permutation],
        permuted_expert_indices=flat[permutation].astype(np.int64),
        expert_counts=counts,
        expert_offsets=offsets,
    )


def group_tokens_by_counting(expert_indices, num_experts: int) -> Routing:
    """Second, loop-based statement of the same grouping (small inputs only).

    Follows the reference CUDA kernels instead of argsort
    (csrc/routing_kernels.cu:24-75): count, serial scan, then each expert walks
    the assignments in order.  Used to cross-check ``group_tokens``.
    """

    ids = np.asarray(
        expert_indices.cpu().numpy() if isinstance(expert_indices, torch.Tensor) else expert_indices
    )
    tokens, top_k = ids.shape
    flat = ids.reshape(-1)
    counts = np.zeros(num_experts, np.int64)
    for e in flat:
        counts[e] += 1
    offsets = np.zeros(num_experts + 1, np.int64)
    for e in range(num_experts):
        offsets[e + 1] = offsets[e] + counts[e]
    reverse = np.full(flat.size, -1, np.int64)
    permutation = np.full(flat.size, -1, np.int64)
    for e in range(num_experts):
        position = offsets[e]
        for a in range(flat.size):
            if flat[a] == e:
                reverse[a] = position
                permutation[position] = a
                position += 1
    return Routing(
        permutation=permutation,
        reverse_mapping=reverse,
        permuted_token_indices=permutation // top_k,
        permuted_expert_indices=flat[permutation].astype(np.int64),
        expert_counts=counts,
        expert_offsets=offsets,
    )


def topk_routing(router_logits: torch.Tensor, top_k: int):
    """Top-k experts per token and a softmax over the selected logits (routing.py:48-55).

    The softmax runs in FP32 and is cast back to the logits' dtype.  Ties between equal
    logits resolve to the lower expert id here (a stable descending sort); ``torch.topk``
    leaves that order unspecified, so parity is stated on tie-free selections.
    """

    order = torch.argsort(router_logits.float(), dim=-1, descending=True, stable=True)
    ids = order[:, :top_k].contiguous()
    selected = torch.gather(router_logits.float(), 1, ids)
    weights = torch.softmax(selected, dim=-1).to(router_logits.dtype)
    return ids, weights


def _silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def routed_moe(
    hidden_states: torch.Tensor,
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    gate_up_weight: torch.Tensor,
    down_weight: torch.Tensor,
    *,
    num_experts: int,
    top_k: int,
    compute_dtype: torch.dtype = torch.float32,
    return_intermediates: bool = False,
):
    """The layer as the reference's torch backend computes it, on the CPU.

    With ``compute_dtype=float32`` (default) every tensor is first converted to
    FP32: this is "the FP32 reference on identical inputs" results are judged
    against.  With another dtype the arithmetic runs in that dtype, operation
    for operation like fastpath/reference.py:260-284 (one linear on the fused
    [2I,H] weight, ``silu(gate) * up``, a second linear, then
    ``index_add_`` of weight-scaled rows in expert-major order,
    baseline/torch_moe.py:130-133): that variant is what the CPU baseline times.

    Routing weights are used exactly as supplied.  Duplicate experts inside a
    token are separate rows.
    """

    if expert_indices.shape[1] != top_k:
        raise ValueError("top_k must match expert_indices.shape[1]")
    routing = group_tokens(expert_indices, num_experts)
    tokens, hidden = hidden_states.shape
    inter = gate_up_weight.shape[1] // 2
    x = hidden_states.to(compute_dtype)
    weights = expert_weights.to(compute_dtype).reshape(-1)
    perm = torch.from_numpy(routing.permutation)
    perm_tokens = torch.from_numpy(routing.permuted_token_indices)
    rows = x.index_select(0, perm_tokens)
    act_rows = torch.empty((rows.shape[0], inter), dtype=compute_dtype)
    out_rows = torch.empty((rows.shape[0], hidden), dtype=compute_dtype)
    for e in range(num_experts):
        lo = int(routing.expert_offsets[e])
        hi = int(routing.expert_offsets[e + 1])
        if lo == hi:
            continue
        gate_up = torch.nn.functional.linear(rows[lo:hi], gate_up_weight[e].to(compute_dtype))
        gate, up = gate_up[:, :inter], gate_up[:, inter:]
        act = torch.nn.functional.silu(gate) * up
        act_rows[lo:hi] = act
        out_rows[lo:hi] = torch.nn.functional.linear(act, down_weight[e].to(compute_dtype))
    weighted = out_rows * weights.index_select(0, perm).unsqueeze(-1)
    output = torch.zeros((tokens, hidden), dtype=compute_dtype)
    output.index_add_(0, perm_tokens, weighted)
    if return_intermediates:
        return output, routing, {"permuted_hidden": rows, "activations": act_rows, "expert_rows": out_rows}
    return output, routing


def routed_moe_naive(
    hidden_states: torch.Tensor,
    expert_indices: torch.Tensor,
    expert_weights: torch.Tensor,
    gate_up_weight: torch.Tensor,
    down_weight: torch.Tensor,
) -> torch.Tensor:
    """Token/slot double loop in FP32 with no grouping at all (small cases).

    Independent statement following tests/test_goal_1b_correctness.py:46-63;
    it shares no routing code with ``routed_moe``.
    """

    inter = gate_up_weight.shape[1] // 2
    x = hidden_states.float()
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(expert_indices.shape[1]):
            e = int(expert_indices[t, k])
            w_gu = gate_up_weight[e].float()
            gate = w_gu[:inter] @ x[t]
            up = w_gu[inter:] @ x[t]
            act = _silu(gate) * up
            out[t] += float(expert_weights[t, k]) * (down_weight[e].float() @ act)
    return out


def rms(x: torch.Tensor) -> float:
    return float(torch.sqrt(torch.mean(x.double() ** 2)))


def relative_max_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """``max|actual - expected| / rms(expected)``: the layer's acceptance metric (bar 2e-2)."""

    err = float((actual.double() - expected.double()).abs().max())
    return err / max(rms(expected), 1e-30)


def bf16_floor(expected: torch.Tensor) -> float:
    """The metric of a perfect kernel: the FP32 reference rounded once to BF16.

    The output dtype is BF16, so no implementation can score below this.
    """

    return relative_max_error(expected.to(torch.bfloat16).float(), expected)
