"""Expert-parallel host logic on CPU ranks (gloo, world size 2 and 4).

The per-rank compute is the oracle here (the tests may use it; the product's
default is the native kernels), so what is checked is the sharding of experts,
the token layouts, the cross-rank sum and the assembly of the global routing
tensors, which must be bit-exact against a single-rank run.
"""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_routing_from_oracle(ids: torch.Tensor, base: int, count: int):
    """What the routing kernel produces on one rank: stable order of the local ids only."""

    flat = ids.reshape(-1) - base
    valid = (flat >= 0) & (flat < count)
    order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, count)), stable=True)
    n_valid = int(valid.sum())
    permutation = torch.full_like(flat, -1)
    permutation[:n_valid] = order[:n_valid]
    reverse = torch.full_like(flat, -1)
    reverse[order[:n_valid]] = torch.arange(n_valid)
    counts = torch.bincount(flat[valid], minlength=count)
    offsets = torch.cat([counts.new_zeros(1), counts.cumsum(0)])
    return {"expert_counts": counts, "expert_offsets": offsets, "permutation": permutation,
            "reverse_mapping": reverse}


def _worker(rank: int, world: int, port: int, results) -> None:
    for entry in (str(REPO / "b300-moe-decode-fastpath_b200"), str(REPO)):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from b200moe import workloads
        from b200moe.expert_parallel import ExpertParallelMoE, assemble_global_routing, expert_range
        from oracle import moe_oracle

        T, H, I, E, K = 8, 32, 48, 8, 2
        hidden, ids, weights, gate_up, down = workloads.make_case(
            T, H, I, E, K, routing="zipf", weight_kind="raw", std=None, seed=77
        )
        base, count = expert_range(rank, world, E)

        def oracle_local(h, i, w):
            mine = (i >= base) & (i < base + count)
            out, _ = moe_oracle.routed_moe(
                h, torch.where(mine, i - base, torch.zeros_like(i)),
                torch.where(mine, w, torch.zeros_like(w)),
                gate_up[base:base + count], down[base:base + count],
                num_experts=count, top_k=K,
            )
            return out

        layer = ExpertParallelMoE(gate_up[base:base + count].contiguous(),
                                  down[base:base + count].contiguous(),
                                  num_experts=E, top_k=K, local_forward=oracle_local)
        full, routing = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down,
                                              num_experts=E, top_k=K)

        replicated = layer.forward(hidden, ids, weights, tokens="replicated")
        err_rep = moe_oracle.relative_max_error(replicated.float(), full)

        per = T // world
        mine = slice(rank * per, (rank + 1) * per)
        sharded = layer.forward(hidden[mine].contiguous(), ids[mine].contiguous(),
                                weights[mine].contiguous(), tokens="sharded")
        err_shard = moe_oracle.relative_max_error(sharded.float(), full[mine])

        assembled = assemble_global_routing(_local_routing_from_oracle(ids, base, count), world)
        exact = all(
            np.array_equal(assembled[k].numpy(), getattr(routing, k))
            for k in ("expert_counts", "expert_offsets", "permutation", "reverse_mapping")
        )
        results[rank] = (err_rep, err_shard, exact, tuple(sharded.shape), str(replicated.dtype))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_matches_single_rank(world: int) -> None:
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        err_rep, err_shard, exact, shape, dtype = results[rank]
        assert exact, f"rank {rank}: assembled routing tensors differ from the single-rank ones"
        assert dtype == "torch.bfloat16"
        assert shape == (8 // world, 32)
        # one BF16 rounding of an FP32 sum: the layer's 2e-2 x RMS bar
        assert err_rep <= 2e-2 and err_shard <= 2e-2, (rank, err_rep, err_shard)


def test_expert_range_rules() -> None:
    sys.path.insert(0, str(REPO / "b300-moe-decode-fastpath_b200"))
    from b200moe.expert_parallel import expert_range

    assert expert_range(0, 4, 64) == (0, 16)
    assert expert_range(3, 4, 64) == (48, 16)
    assert expert_range(7, 8, 8) == (7, 1)
    with pytest.raises(ValueError, match="divisible"):
        expert_range(0, 3, 8)
