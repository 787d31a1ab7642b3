"""The allocation-free routing entry point against the regular one (GPU).

``b200moe_routing_static`` exists for hosts that may not allocate device memory
when they need routing metadata -- a server whose memory arena owns the whole
GPU, a plugin interface that forbids allocation after start-up.  It keeps the
kernel's scratch inside the library.  This test drives both entry points through
the C ABI on the same inputs and requires identical tensors, twice in a row, the
second time with different routes so that anything left over from the first call
would show.  Routing is integer work: the comparison is exact.  The same outputs are also
compared with the CPU oracle's ``group_tokens`` directly, and a repeated call must leave the
device's free memory and PyTorch's allocation counter where they were.

The file name sorts last on purpose: if this test fails, a run that stops at the
first failure has already run everything else.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ROUTING_KEYS = (
    "expert_counts",
    "expert_offsets",
    "expert_offsets_i32",
    "permutation",
    "reverse_mapping",
    "permuted_token_indices",
    "permuted_expert_indices",
    "permuted_weights",
)


def _routing_outputs(device, experts: int, rows: int) -> dict[str, torch.Tensor]:
    """Caller-owned result buffers, pre-filled so that unwritten entries would be noticed."""

    def ints(n, dtype=torch.int64):
        return torch.full((n,), -7, dtype=dtype, device=device)

    return {
        "expert_counts": ints(experts),
        "expert_offsets": ints(experts + 1),
        "expert_offsets_i32": ints(experts, torch.int32),
        "permutation": ints(rows),
        "reverse_mapping": ints(rows),
        "permuted_token_indices": ints(rows),
        "permuted_expert_indices": ints(rows),
        "permuted_weights": torch.full((rows,), -7.0, dtype=torch.bfloat16, device=device),
    }


def _run_both(device, tokens, experts, top_k, pattern, seed, bad_id=False):
    from b200moe import StagedLayer, _lib, workloads

    hidden, ids, weights, gate_up, down = workloads.make_case(
        tokens, 64, 96, experts, top_k, routing=pattern, seed=seed, std=None, device=device
    )
    if bad_id:
        ids = ids.clone()
        ids[0, 0] = experts  # out of range: the row must be dropped by both entry points
    layer = StagedLayer(hidden, ids, weights, gate_up, down, num_experts=experts, top_k=top_k)
    layer.run_stage("routing")
    expected = {k: v.clone() for k, v in layer.routing_tensors().items()}

    rows = tokens * top_k
    outputs = _routing_outputs(device, experts, rows)
    args = _lib.B200MoeArgs()
    ctypes.memmove(ctypes.byref(args), ctypes.byref(layer._args), ctypes.sizeof(args))
    for name, tensor in outputs.items():
        setattr(args, name, tensor.data_ptr())
    args.scratch = None          # the static variant must not need caller scratch
    args.scratch_bytes = 0
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = _lib.load().b200moe_routing_static(ctypes.byref(args), stream)
    _lib.check(code, "b200moe_routing_static")
    torch.cuda.synchronize(device)
    return expected, outputs


def _assert_same(expected, outputs, label):
    for key in ROUTING_KEYS:
        assert torch.equal(outputs[key], expected[key]), f"{label}: {key} differs"


def _assert_matches_oracle(outputs, tokens, experts, top_k, pattern, seed, label):
    """The static entry point's tensors against the oracle's grouping of the same ids."""

    import numpy as np

    from b200moe import workloads
    from oracle import moe_oracle

    ids = workloads.make_case(tokens, 64, 96, experts, top_k, routing=pattern, seed=seed,
                              std=None)[1]
    want = moe_oracle.group_tokens(ids, experts)
    for key in ("expert_counts", "expert_offsets", "permutation", "reverse_mapping",
                "permuted_token_indices", "permuted_expert_indices"):
        assert np.array_equal(outputs[key].cpu().numpy(), getattr(want, key)), f"{label}: {key}"
    assert np.array_equal(outputs["expert_offsets_i32"].cpu().numpy(),
                          want.expert_offsets[1:].astype(np.int32)), label


def test_static_routing_matches_regular_routing_on_two_calls_in_a_row(cuda_device) -> None:
    first = _run_both(cuda_device, tokens=64, experts=32, top_k=8, pattern="zipf", seed=11)
    _assert_same(*first, "first call")
    _assert_matches_oracle(first[1], 64, 32, 8, "zipf", 11, "first call")
    second = _run_both(cuda_device, tokens=17, experts=16, top_k=2, pattern="empty_half", seed=12)
    _assert_same(*second, "second call")
    _assert_matches_oracle(second[1], 17, 16, 2, "empty_half", 12, "second call")


def test_static_routing_leaves_device_memory_alone(cuda_device) -> None:
    """The property the entry point exists for: after a first call (which looks up the
    array's address), another call changes neither the device's free memory nor PyTorch's
    count of allocated bytes."""

    from b200moe import StagedLayer, _lib, workloads

    hidden, ids, weights, gate_up, down = workloads.make_case(
        32, 64, 96, 16, 4, routing="uniform", seed=5, std=None, device=cuda_device)
    layer = StagedLayer(hidden, ids, weights, gate_up, down, num_experts=16, top_k=4)
    outputs = _routing_outputs(cuda_device, 16, 32 * 4)
    args = _lib.B200MoeArgs()
    ctypes.memmove(ctypes.byref(args), ctypes.byref(layer._args), ctypes.sizeof(args))
    for name, tensor in outputs.items():
        setattr(args, name, tensor.data_ptr())
    args.scratch, args.scratch_bytes = None, 0
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    lib = _lib.load()
    _lib.check(lib.b200moe_routing_static(ctypes.byref(args), stream), "b200moe_routing_static")
    torch.cuda.synchronize(cuda_device)
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    torch_before = torch.cuda.memory_allocated(cuda_device)
    for _ in range(3):
        _lib.check(lib.b200moe_routing_static(ctypes.byref(args), stream),
                   "b200moe_routing_static")
    torch.cuda.synchronize(cuda_device)
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after == free_before
    assert torch.cuda.memory_allocated(cuda_device) == torch_before


def test_static_routing_state_does_not_leak_between_calls(cuda_device) -> None:
    # a call that drops a row (bad id), then a clean call with other routes
    dropped = _run_both(cuda_device, tokens=9, experts=8, top_k=4, pattern="duplicates",
                        seed=21, bad_id=True)
    _assert_same(*dropped, "call with an out-of-range id")
    assert int(dropped[1]["reverse_mapping"][0]) == -1
    assert int(dropped[1]["expert_counts"].sum()) == 9 * 4 - 1
    clean = _run_both(cuda_device, tokens=300, experts=64, top_k=8, pattern="uniform", seed=22)
    _assert_same(*clean, "clean call after it")
    assert int(clean[1]["expert_counts"].sum()) == 300 * 8


def test_static_routing_rejects_sizes_beyond_its_maximum(cuda_device) -> None:
    from b200moe import _lib

    args = _lib.B200MoeArgs()
    args.num_tokens, args.top_k, args.num_experts = 513, 8, 64  # 4104 > 4096 assignments
    args.hidden_size = args.intermediate_size = 64
    dummy = torch.zeros(8, dtype=torch.int64, device=cuda_device)
    for name in ("expert_indices", "expert_counts", "expert_offsets", "expert_offsets_i32",
                 "permutation", "reverse_mapping"):
        setattr(args, name, dummy.data_ptr())
    code = _lib.load().b200moe_routing_static(ctypes.byref(args), None)
    assert code == -8
    assert "4096" in _lib.error_string(code)
