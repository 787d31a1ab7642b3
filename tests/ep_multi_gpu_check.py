"""Multi-GPU check of the expert-parallel layer, run under torchrun (one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 tests/ep_multi_gpu_check.py

Every rank builds the same seeded problem, keeps its experts' weights, runs the layer with
both token layouts (replicated, sharded) and both transports (NCCL baseline, NVLink peer
memory) and compares with the CPU oracle of the whole layer; the assembled routing tensors
must be bit-exact against the single-rank ones.  Then 150 steps with changing token counts,
routing patterns and layouts on one engine, each against the oracle.  Prints one line per
rank, "EP_CHECK_OK".
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

REPO = Path(__file__).resolve().parent.parent
for entry in (str(REPO / "b300-moe-decode-fastpath_b200"), str(REPO)):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def mixed_steps(layer, gate_up, down, E, K, H, rank, world, device, steps: int = 150) -> int:
    """Steps with changing token counts, routing patterns and token layouts on one engine
    (peer transport): every output against the oracle, device status clean after every
    step.  The bar is the usual 2e-2 x RMS, or the BF16 rounding of the reference itself
    where an outlier row puts that above the bar."""

    import random

    from b200moe import workloads
    from oracle import moe_oracle

    rng = random.Random(5)  # the same sequence on every rank
    for step in range(steps):
        T = rng.choice([1, 2, 3, 4, 8, 16, 24, 32, 64])
        T = min(T, layer.capacity_tokens)
        sharded = T % world == 0 and rng.random() < 0.4
        hidden = workloads.make_hidden(T, H, seed=1000 + step)
        ids = workloads.make_routing(T, E, K, rng.choice(["uniform", "zipf"]), 2000 + step)
        weights = workloads.make_routing_weights(T, K, "softmax", 3000 + step)
        ref, _ = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
        dev = tuple(t.to(device) for t in (hidden, ids, weights))
        if sharded:
            per = T // world
            mine = slice(rank * per, (rank + 1) * per)
            out = layer.forward(*(t[mine].contiguous() for t in dev), tokens="sharded")
            want = torch.as_tensor(ref)[mine]
        else:
            out = layer.forward(*dev, tokens="replicated")
            want = torch.as_tensor(ref)
        rms = float(torch.as_tensor(ref).double().pow(2).mean().sqrt())
        err = float((out.float().cpu() - want).abs().max()) / rms
        bar = max(2e-2, 1.02 * moe_oracle.bf16_floor(ref))
        assert err <= bar, ("mixed step", step, T, sharded, err, bar)
        assert layer.workspace.status() == 0, ("mixed step", step, T, sharded)
    assert layer.repeated_steps > 0
    return steps


def main() -> int:
    from b200moe import workloads
    from b200moe.expert_parallel import ExpertParallelMoE, expert_range
    from oracle import moe_oracle

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    rank, world = dist.get_rank(), dist.get_world_size()
    try:
        T, H, I, E, K = 8 * world, 512, 768, 8 * world, 4
        hidden, ids, weights, gate_up, down = workloads.make_case(
            T, H, I, E, K, routing="zipf", weight_kind="raw", std=None, seed=321)
        ref, routing = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down,
                                             num_experts=E, top_k=K)
        base, count = expert_range(rank, world, E)
        gu = gate_up[base:base + count].to(device).contiguous()
        dn = down[base:base + count].to(device).contiguous()
        dev = tuple(t.to(device) for t in (hidden, ids, weights))
        per = T // world
        mine = slice(rank * per, (rank + 1) * per)
        shard = tuple(t[mine].contiguous() for t in dev)
        worst = 0.0
        for transport in ("nccl", "p2p"):
            layer = ExpertParallelMoE(gu, dn, num_experts=E, top_k=K, capacity_tokens=T,
                                      transport=transport)
            for repeat in range(3):  # several epochs: both buffer parities, flag reuse
                out = layer.forward(*dev, tokens="replicated")
                err = moe_oracle.relative_max_error(out.float().cpu(), ref)
                assembled = layer.global_routing()
                for key in ("expert_counts", "expert_offsets", "permutation", "reverse_mapping"):
                    assert np.array_equal(assembled[key].cpu().numpy(), getattr(routing, key)), \
                        (transport, key)
                out_s = layer.forward(*shard, tokens="sharded")
                err_s = moe_oracle.relative_max_error(out_s.float().cpu(), ref[mine])
                worst = max(worst, err, err_s)
                assert err <= 2e-2 and err_s <= 2e-2, (transport, repeat, err, err_s)
                assert layer.workspace.status() == 0
            if transport == "p2p":
                # back-to-back replicated steps with fresh tensors and changing token counts
                # take the plan remembered after one checked step, and give the same rows
                layer.forward(*dev, tokens="replicated")
                before = layer.repeated_steps
                for n in (T, T // 2, 2, T):
                    fresh = tuple(t[:n].clone() for t in dev)
                    out = layer.forward(*fresh, tokens="replicated")
                    err = moe_oracle.relative_max_error(out.float().cpu(), ref[:n])
                    worst = max(worst, err)
                    assert err <= 2e-2, ("repeated step", n, err)
                assert layer.repeated_steps == before + 4, layer.repeated_steps
                assert layer.workspace.status() == 0
                # out=: the combine kernel stores into the caller's tensor, on the device or
                # in pinned host memory, with the same bits
                want_rows = layer.forward(*dev, tokens="replicated").clone()
                for target in (torch.empty_like(want_rows),
                               torch.empty(T, H, dtype=want_rows.dtype).pin_memory()):
                    got = layer.forward(*dev, tokens="replicated", out=target)
                    torch.cuda.synchronize(device)
                    assert got is target and torch.equal(target.to(device), want_rows)
                mine_rows = layer.forward(*shard, tokens="sharded").clone()
                host_rows = torch.empty(per, H, dtype=mine_rows.dtype).pin_memory()
                layer.forward(*shard, tokens="sharded", out=host_rows)
                torch.cuda.synchronize(device)
                assert torch.equal(host_rows.to(device), mine_rows)
        torch.cuda.synchronize(device)
        soak_steps = mixed_steps(layer, gate_up, down, E, K, H, rank, world, device)
        print(f"EP_CHECK_OK rank={rank} world={world} worst_err_over_rms={worst:.5f} "
              f"floor={moe_oracle.bf16_floor(ref):.5f} mixed_steps={soak_steps}", flush=True)
    finally:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
