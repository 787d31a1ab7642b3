"""Seeded synthetic inputs for the layer: shapes, routing patterns, value distributions.

These stand in for the reference's workload generators
(baseline/routing.py:111-168, baseline/torch_moe.py:29-55,
benchmark/benchmark_goal_1b.py:244-291) with the shapes and distributions of
the benchmark configurations below.  All routing randomness comes from a CPU
``torch.Generator`` so a seed defines the same routes on any device; weights
may be drawn on the GPU (tens of GiB do not fit a host-side draw in reasonable
time) from a seeded CUDA generator.  Seeds follow the reference's
``seed, seed+1, seed+2`` convention (benchmark_goal_1b.py:257-277).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

ROUTING_PATTERNS = (
    "uniform",       # K distinct experts per token, uniform
    "zipf",          # K distinct experts per token, p_e ~ (e+1)^-1.2
    "hotspot",       # half of every token's slots on 4 fixed hot experts
    "concentrated",  # every token routes to the same K experts
    "empty_half",    # ids drawn from a seeded half of the experts
    "duplicates",    # independent uniform ids, repeats inside a token allowed
)


@dataclass(frozen=True)
class LayerConfig:
    name: str
    hidden_size: int
    intermediate_size: int
    num_experts: int
    top_k: int
    tokens: tuple[int, ...]
    routing: str = "uniform"
    weight_kind: str = "softmax"   # "softmax" over K of N(0,1) logits, or "raw" N(0,1)
    dtype: torch.dtype = torch.bfloat16


CONFIGS = {
    # CPU-runnable reference case (FP32 in the reference; run here on its BF16 cast)
    "cpu_small": LayerConfig("cpu_small", 256, 512, 8, 2, (16,)),
    "mixtral": LayerConfig("mixtral", 4096, 14336, 8, 2, (1, 2, 4, 8, 16, 32, 64)),
    "wide": LayerConfig("wide", 4096, 14336, 64, 8, (64,), routing="zipf", weight_kind="raw"),
    "deepseek": LayerConfig("deepseek", 7168, 2048, 256, 8, (1, 8, 32, 64)),
    "irregular": LayerConfig("irregular", 2880, 2880, 32, 8, (1, 3, 17, 63)),
}


def make_routing(
    num_tokens: int,
    num_experts: int,
    top_k: int,
    pattern: str = "uniform",
    seed: int = 1235,
) -> torch.Tensor:
    """[T,K] int64 expert ids on the CPU for one of ``ROUTING_PATTERNS``."""

    if pattern not in ROUTING_PATTERNS:
        raise ValueError(f"unknown routing pattern {pattern!r}")
    g = torch.Generator(device="cpu").manual_seed(seed)
    T, E, K = num_tokens, num_experts, top_k
    if pattern == "uniform":
        ids = torch.rand(T, E, generator=g).argsort(dim=1)[:, :K]
    elif pattern == "zipf":
        p = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.2)
        ids = torch.multinomial((p / p.sum()).expand(T, E), K, replacement=False, generator=g)
    elif pattern == "hotspot":
        hot = min(4, E)
        ids = torch.empty(T, K, dtype=torch.int64)
        for t in range(T):
            n_hot = K // 2 if K >= 2 else t % 2
            n_hot = min(n_hot, hot)
            hot_ids = torch.randperm(hot, generator=g)[:n_hot]
            cold_pool = E - hot
            if cold_pool >= K - n_hot:
                cold = hot + torch.randperm(cold_pool, generator=g)[: K - n_hot]
            else:
                cold = torch.randint(0, E, (K - n_hot,), generator=g)
            ids[t] = torch.cat([hot_ids, cold])
    elif pattern == "concentrated":
        chosen = torch.randperm(E, generator=g)[:K]
        ids = chosen.unsqueeze(0).expand(T, K).clone()
    elif pattern == "empty_half":
        pool = torch.randperm(E, generator=g)[: max(K, E // 2)]
        pick = torch.rand(T, pool.numel(), generator=g).argsort(dim=1)[:, :K]
        ids = pool[pick]
    else:  # duplicates
        ids = torch.randint(0, E, (T, K), generator=g)
    return ids.to(torch.int64).contiguous()


def make_routing_weights(
    num_tokens: int, top_k: int, kind: str = "softmax", seed: int = 1235,
    dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """[T,K] routing weights: softmax of N(0,1) logits, or raw N(0,1) with negatives."""

    g = torch.Generator(device="cpu").manual_seed(seed + 7919)
    logits = torch.randn(num_tokens, top_k, generator=g)
    if kind == "softmax":
        logits = torch.softmax(logits, dim=-1)
    elif kind != "raw":
        raise ValueError("weight kind must be 'softmax' or 'raw'")
    return logits.to(dtype).contiguous()


def make_expert_weights(
    num_experts: int,
    hidden_size: int,
    intermediate_size: int,
    *,
    seed: int = 1236,
    std: float | None = 0.02,
    device: torch.device | str = "cpu",
    dtype: torch.dtype = torch.bfloat16,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``gate_up_weight`` [E,2I,H] and ``down_weight`` [E,H,I].

    ``std=None`` uses 1/sqrt(fan_in) like the reference's generator
    (baseline/torch_moe.py:41-55); the BF16 configurations use N(0, 0.02).
    Drawn expert by expert so the FP32 staging buffer stays one expert large.
    """

    device = torch.device(device)
    g = torch.Generator(device=device).manual_seed(seed)
    gate_up = torch.empty(num_experts, 2 * intermediate_size, hidden_size, device=device, dtype=dtype)
    down = torch.empty(num_experts, hidden_size, intermediate_size, device=device, dtype=dtype)
    s_in = hidden_size ** -0.5 if std is None else std
    s_down = intermediate_size ** -0.5 if std is None else std
    for e in range(num_experts):
        gate_up[e] = (
            torch.randn(2 * intermediate_size, hidden_size, generator=g, device=device) * s_in
        ).to(dtype)
        down[e] = (
            torch.randn(hidden_size, intermediate_size, generator=g, device=device) * s_down
        ).to(dtype)
    return gate_up, down


def make_hidden(
    num_tokens: int, hidden_size: int, *, seed: int = 1234, dtype: torch.dtype = torch.bfloat16
) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(num_tokens, hidden_size, generator=g).to(dtype).contiguous()


def make_case(
    num_tokens: int,
    hidden_size: int,
    intermediate_size: int,
    num_experts: int,
    top_k: int,
    *,
    routing: str = "uniform",
    weight_kind: str = "softmax",
    seed: int = 1234,
    std: float | None = 0.02,
    device: torch.device | str = "cpu",
    dtype: torch.dtype = torch.bfloat16,
    expert_weights_device: torch.device | str | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(hidden, ids, routing_weights, gate_up_weight, down_weight) on ``device``."""

    device = torch.device(device)
    hidden = make_hidden(num_tokens, hidden_size, seed=seed, dtype=dtype).to(device)
    ids = make_routing(num_tokens, num_experts, top_k, routing, seed + 1).to(device)
    weights = make_routing_weights(num_tokens, top_k, weight_kind, seed + 1, dtype).to(device)
    gate_up, down = make_expert_weights(
        num_experts,
        hidden_size,
        intermediate_size,
        seed=seed + 2,
        std=std,
        device=expert_weights_device if expert_weights_device is not None else device,
        dtype=dtype,
    )
    return hidden, ids, weights, gate_up.to(device), down.to(device)
