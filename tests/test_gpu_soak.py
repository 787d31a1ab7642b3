"""A few seconds of back-to-back forwards on one workspace, every output checked.

The kernels of one forward are chained by programmatic dependent launch, and the small-call
order lets the gate+up kernel start before the routing kernel has finished; consecutive calls
reuse the same workspace buffers without a host synchronisation in between.  A hand-over that
let a kernel read a buffer too early would show as an output that differs from the first
run of the same inputs, or as a non-zero device status.  The comparison runs on the device
(one flag accumulated per call), so the launch queue stays as deep as in production.
"""

from __future__ import annotations

import random
import time

import pytest
import torch

from oracle import moe_oracle

pytestmark = pytest.mark.gpu

SOAK_SECONDS = 4.0


def test_mixed_sizes_and_weight_formats_back_to_back(cuda_device) -> None:
    from b200moe import (B300MoEWorkspace, b300_moe_forward, b300_moe_forward_fp8,
                         b300_moe_forward_nvfp4, quantize_expert_weights_fp8,
                         quantize_expert_weights_nvfp4, workloads)

    H, I, E, K = 2048, 4096, 8, 2
    gate_up, down = workloads.make_expert_weights(E, H, I, seed=1236, std=0.02, device=cuda_device)
    fp8 = quantize_expert_weights_fp8(gate_up, down)
    fp4 = quantize_expert_weights_nvfp4(gate_up, down)
    runners = {
        "bf16": lambda c, ws: b300_moe_forward(*c, gate_up, down, num_experts=E, top_k=K, workspace=ws),
        "fp8": lambda c, ws: b300_moe_forward_fp8(*c, fp8, num_experts=E, top_k=K, workspace=ws),
        "nvfp4": lambda c, ws: b300_moe_forward_nvfp4(*c, fp4, num_experts=E, top_k=K, workspace=ws),
    }
    cases = {}
    for T in (1, 2, 4, 8, 16, 17, 32, 64):      # T*K <= 32 takes the small-call kernel order
        cases[T] = tuple(t.to(cuda_device) for t in (
            workloads.make_hidden(T, H, seed=T),
            workloads.make_routing(T, E, K, "zipf" if T % 2 else "uniform", 1235 + T),
            workloads.make_routing_weights(T, K, seed=T)))
    ws = B300MoEWorkspace(capacity_tokens=64, device=cuda_device)
    want = {}
    for T, case in cases.items():
        for name, run in runners.items():
            want[(T, name)] = run(case, ws).clone()
    torch.cuda.synchronize(cuda_device)
    assert ws.status() == 0
    # the first runs themselves are right (BF16 against the oracle; the other formats have
    # their own parity tests)
    for T in (1, 17, 64):
        ref, _ = moe_oracle.routed_moe(*(t.cpu() for t in cases[T]), gate_up.cpu(), down.cpu(),
                                       num_experts=E, top_k=K)
        assert moe_oracle.relative_max_error(want[(T, "bf16")].float().cpu(), ref) <= 2e-2

    allocations = ws.allocation_count
    rng = random.Random(1)
    keys = sorted(want)
    mismatches = torch.zeros((), dtype=torch.int64, device=cuda_device)
    forwards = 0
    start = time.time()
    while time.time() - start < SOAK_SECONDS:
        for _ in range(100):
            T, name = rng.choice(keys)
            out = runners[name](cases[T], ws)
            mismatches += (out != want[(T, name)]).any()
            forwards += 1
        torch.cuda.synchronize(cuda_device)
        assert ws.status() == 0
    print(f"soak: {forwards} forwards in {time.time() - start:.1f} s, "
          f"{int(mismatches)} mismatching outputs")
    assert int(mismatches) == 0
    assert forwards >= 1000
    assert ws.allocation_count == allocations
