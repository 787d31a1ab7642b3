"""GPU tests of the API contract: workspace reuse, streams, metadata, explicit failures.

These replay, on the sm_100a kernels, the behaviours the reference's B300-only
suite pins (tests/test_goal_1b_cuda.py:139-175, 213-247, 316-400).
"""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import moe_oracle

pytestmark = pytest.mark.gpu


def _case(device, tokens=8, experts=16, top_k=2, hidden=64, inter=96, routing="uniform",
          weight_kind="softmax", seed=1234):
    from b200moe import workloads

    return workloads.make_case(tokens, hidden, inter, experts, top_k, routing=routing,
                               weight_kind=weight_kind, seed=seed, std=None, device=device)


def test_workspace_reuse_is_bitwise_repeatable_on_a_side_stream(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    tensors = _case(cuda_device, tokens=9, routing="empty_half", weight_kind="raw")
    workspace = B300MoEWorkspace(capacity_tokens=16, device=cuda_device)
    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        first, meta1 = b300_moe_forward(*tensors, num_experts=16, top_k=2, workspace=workspace,
                                        return_metadata=True)
        ptrs = workspace.buffer_data_ptrs()
        second, meta2 = b300_moe_forward(*tensors, num_experts=16, top_k=2, workspace=workspace,
                                         return_metadata=True)
    side.synchronize()
    assert torch.equal(first, second)
    assert workspace.buffer_data_ptrs() == ptrs
    assert workspace.allocation_count == 1 and workspace.reuse_count == 1
    assert meta1["workspace"]["reused"] is False and meta2["workspace"]["reused"] is True
    assert workspace.last_stream == int(side.cuda_stream)
    assert first.data_ptr() != second.data_ptr()
    for buffer in workspace.buffers.values():
        assert first.data_ptr() != buffer.data_ptr()
    ref, _ = moe_oracle.routed_moe(*(t.cpu() for t in tensors), num_experts=16, top_k=2)
    assert moe_oracle.relative_max_error(first.float().cpu(), ref) <= 2e-2


def test_metadata_survives_reuse_from_another_stream(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    workspace = B300MoEWorkspace(device=cuda_device)
    a = _case(cuda_device, seed=10)
    b = _case(cuda_device, seed=20, routing="concentrated")
    s1, s2 = torch.cuda.Stream(device=cuda_device), torch.cuda.Stream(device=cuda_device)
    with torch.cuda.stream(s1):
        _, meta_a = b300_moe_forward(*a, num_experts=16, top_k=2, workspace=workspace,
                                     return_metadata=True)
    with torch.cuda.stream(s2):
        _, meta_b = b300_moe_forward(*b, num_experts=16, top_k=2, workspace=workspace,
                                     return_metadata=True)
    torch.cuda.synchronize(cuda_device)
    want_a = moe_oracle.group_tokens(a[1].cpu(), 16)
    want_b = moe_oracle.group_tokens(b[1].cpu(), 16)
    assert meta_a["permutation"].cpu().tolist() == want_a.permutation.tolist()
    assert meta_b["permutation"].cpu().tolist() == want_b.permutation.tolist()
    assert meta_a["expert_offsets"].cpu().tolist() == want_a.expert_offsets.tolist()


def test_two_streams_with_own_workspaces_run_concurrently(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    cases = [_case(cuda_device, tokens=17, seed=s, hidden=256, inter=512) for s in (1, 2)]
    spaces = [B300MoEWorkspace(device=cuda_device) for _ in cases]
    streams = [torch.cuda.Stream(device=cuda_device) for _ in cases]
    outs = []
    torch.cuda.synchronize(cuda_device)
    for _ in range(3):
        outs = []
        for case, space, stream in zip(cases, spaces, streams):
            with torch.cuda.stream(stream):
                outs.append(b300_moe_forward(*case, num_experts=16, top_k=2, workspace=space))
    torch.cuda.synchronize(cuda_device)
    for case, out in zip(cases, outs):
        ref, _ = moe_oracle.routed_moe(*(t.cpu() for t in case), num_experts=16, top_k=2)
        assert moe_oracle.relative_max_error(out.float().cpu(), ref) <= 2e-2


def test_workspace_grows_and_rebinds(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    workspace = B300MoEWorkspace(capacity_tokens=4, device=cuda_device)
    b300_moe_forward(*_case(cuda_device, tokens=3), num_experts=16, top_k=2, workspace=workspace)
    assert (workspace.allocation_count, workspace.capacity_tokens) == (1, 4)
    assert workspace.capacity_assignments == 8
    b300_moe_forward(*_case(cuda_device, tokens=6), num_experts=16, top_k=2, workspace=workspace)
    assert workspace.allocation_count == 2 and workspace.capacity_tokens >= 8
    b300_moe_forward(*_case(cuda_device, tokens=2, top_k=1, hidden=72), num_experts=16, top_k=1,
                     workspace=workspace)
    assert workspace.allocation_count == 3
    assert workspace.last_shape == (2, 16, 1, 72, 96)
    assert workspace.private_bytes > 0 and workspace.capacity_bytes > workspace.private_bytes


def test_single_expert_in_both_slots_known_counts(cuda_device) -> None:
    from b200moe import b300_moe_forward

    hidden, ids, weights, gate_up, down = _case(cuda_device, tokens=8)
    ids = torch.full_like(ids, 5)
    out, meta = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=16, top_k=2,
                                 return_metadata=True)
    assert meta["expert_counts"].cpu().tolist() == [0] * 5 + [16] + [0] * 10
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                   down.cpu(), num_experts=16, top_k=2)
    assert moe_oracle.relative_max_error(out.float().cpu(), ref) <= 2e-2


def test_out_of_range_id_sets_status_and_never_traps(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    hidden, ids, weights, gate_up, down = _case(cuda_device, tokens=4)
    bad = ids.clone()
    bad[1, 0] = 16
    workspace = B300MoEWorkspace(device=cuda_device)
    with pytest.raises(ValueError, match="out-of-range"):
        b300_moe_forward(hidden, bad, weights, gate_up, down, num_experts=16, top_k=2,
                         workspace=workspace, check_status=True)
    # the context is intact and the dropped row contributed nothing
    out, meta = b300_moe_forward(hidden, bad, weights, gate_up, down, num_experts=16, top_k=2,
                                 workspace=workspace, return_metadata=True)
    assert int(meta["reverse_mapping"][2]) == -1
    assert int(meta["expert_counts"].sum()) == 7
    keep = weights.clone()
    keep[1, 0] = 0
    good = ids.clone()
    good[1, 0] = 0
    want = b300_moe_forward(hidden, good, keep, gate_up, down, num_experts=16, top_k=2)
    assert moe_oracle.relative_max_error(out.float().cpu(), want.float().cpu()) <= 2e-2
    clean = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=16, top_k=2,
                             workspace=workspace, check_status=True)
    assert clean.shape == hidden.shape


def test_explicit_failures_on_device(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward

    tensors = _case(cuda_device)
    # the NVFP4 backend runs (tests/test_gpu_nvfp4.py) but needs H and I divisible by 64;
    # it never falls back to the BF16 kernels
    with pytest.raises(ValueError, match="divisible by 64"):
        b300_moe_forward(*tensors, num_experts=16, top_k=2, backend="cutlass_nvfp4")
    with pytest.raises(RuntimeError, match="not an execution path"):
        b300_moe_forward(*tensors, num_experts=16, top_k=2, backend="torch")
    odd = _case(cuda_device, hidden=30 * 2 + 2, inter=46 * 2 + 2)  # 62, 94: not multiples of 8
    workspace = B300MoEWorkspace(device=cuda_device)
    with pytest.raises(ValueError, match="divisible by 8"):
        b300_moe_forward(*odd, num_experts=16, top_k=2, workspace=workspace)
    assert workspace.allocation_count == 0
    halves = tuple(t.half() if t.is_floating_point() else t for t in tensors)
    with pytest.raises(TypeError, match="requires bfloat16"):
        b300_moe_forward(*halves, num_experts=16, top_k=2)


def test_tokens_beyond_decode_sizes_stay_correct(cuda_device) -> None:
    """T is unbounded in the contract (reference.py:74-75): 300 tokens x 8 slots = 2400
    assignments exercises the multi-round routing kernel and many segments."""

    from b200moe import b300_moe_forward

    tensors = _case(cuda_device, tokens=300, top_k=8, experts=16, hidden=64, inter=128,
                    routing="zipf")
    out, meta = b300_moe_forward(*tensors, num_experts=16, top_k=8, return_metadata=True,
                                 check_status=True)
    want = moe_oracle.group_tokens(tensors[1].cpu(), 16)
    assert meta["permutation"].cpu().tolist() == want.permutation.tolist()
    assert meta["reverse_mapping"].cpu().tolist() == want.reverse_mapping.tolist()
    ref, _ = moe_oracle.routed_moe(*(t.cpu() for t in tensors), num_experts=16, top_k=8)
    # The 2e-2 bar is stated for T <= 64.  Over 300 x 64 outputs the largest |y| / rms grows,
    # and rounding the exact result to BF16 alone can exceed it; the kernels must then sit
    # on that floor.
    err = moe_oracle.relative_max_error(out.float().cpu(), ref)
    floor = moe_oracle.bf16_floor(ref)
    assert err <= max(2e-2, 1.03 * floor), (err, floor)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_ranks_emulated_on_one_gpu(world, cuda_device) -> None:
    """Each rank's share of an expert-parallel forward, run one after another on one GPU:
    the sum of the FP32 partial outputs must equal the layer, and every rank's routing
    must be the global stable order restricted to its experts."""

    from b200moe import B300MoEWorkspace, workloads
    from b200moe.expert_parallel import expert_range, local_partial_forward

    T, H, I, E, K = 16, 256, 384, 8, 2
    hidden, ids, weights, gate_up, down = workloads.make_case(
        T, H, I, E, K, routing="zipf", weight_kind="raw", std=None, device=cuda_device
    )
    total = torch.zeros(T, H, dtype=torch.float32, device=cuda_device)
    want = moe_oracle.group_tokens(ids.cpu(), E)
    for rank in range(world):
        base, count = expert_range(rank, world, E)
        workspace = B300MoEWorkspace(device=cuda_device)
        partial, _ = local_partial_forward(
            hidden, ids, weights, gate_up[base:base + count].contiguous(),
            down[base:base + count].contiguous(), top_k=K, expert_id_base=base,
            num_experts_global=E, workspace=workspace,
        )
        total += partial
        assert workspace.status() == 0  # other ranks' ids are not reported as bad ids
        rows = int(want.expert_offsets[base + count] - want.expert_offsets[base])
        lo = int(want.expert_offsets[base])
        perm = workspace.buffers["permutation"][: T * K].cpu()
        assert perm[:rows].tolist() == want.permutation[lo:lo + rows].tolist()
        assert (perm[rows:] == -1).all()
        rev = workspace.buffers["reverse_mapping"][: T * K].cpu()
        mine = torch.from_numpy((want.reverse_mapping >= lo) & (want.reverse_mapping < lo + rows))
        assert torch.equal(rev[mine], torch.from_numpy(want.reverse_mapping)[mine] - lo)
        assert (rev[~mine] == -1).all()
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                   down.cpu(), num_experts=E, top_k=K)
    err = moe_oracle.relative_max_error(total.to(torch.bfloat16).float().cpu(), ref)
    assert err <= 2e-2, err


def _ep_reduce_call(device, partials, flag_arrays, rank, epoch, limit_us, status, output):
    import ctypes

    from b200moe import _lib

    world = len(partials)
    args = _lib.B200MoeEpReduceArgs()
    p_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in partials])
    f_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in flag_arrays])
    args.partial_ptrs = ctypes.cast(p_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.flag_ptrs = ctypes.cast(f_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.world, args.rank = world, rank
    args.num_tokens, args.hidden_size = output.shape
    args.epoch, args.wait_limit_us = epoch, limit_us
    args.output, args.status, args.flags = output.data_ptr(), status.data_ptr(), 0
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = _lib.load().b200moe_ep_reduce(ctypes.byref(args), stream)
    _lib.check(code, "b200moe_ep_reduce")
    torch.cuda.synchronize(device)


def test_peer_reduce_kernel_with_all_ranks_buffers_on_one_gpu(cuda_device) -> None:
    """The expert-parallel combine kernel with the ranks' buffers all on this GPU and the
    peers' flags written by the host: rank-order FP32 sum, one BF16 rounding."""

    g = torch.Generator(device="cpu").manual_seed(3)
    world, T, H = 4, 17, 2880
    partials = [torch.randn(T, H, generator=g).to(cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    flags[1][:] = torch.tensor([5, 0, 5, 5, 0, 0, 0, 0], dtype=torch.int32)  # peers 0, 2, 3 arrived
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    output = torch.zeros(T, H, dtype=torch.bfloat16, device=cuda_device)
    _ep_reduce_call(cuda_device, partials, flags, rank=1, epoch=5, limit_us=0, status=status,
                    output=output)
    expected = partials[0].clone()
    for other in partials[1:]:
        expected += other
    assert torch.equal(output, expected.to(torch.bfloat16))
    assert int(status.item()) == 0
    # the kernel published this rank's epoch into slot `rank` of every rank's flag array
    assert [int(f[1]) for f in flags] == [5, 5, 5, 5]


def test_peer_reduce_wait_is_bounded_and_reports_a_missing_peer(cuda_device) -> None:
    """A peer that never publishes: the wait gives up after its limit, sets the status
    bit and writes zeros; the context stays usable."""

    world, T, H = 2, 3, 64
    partials = [torch.ones(T, H, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    output = torch.full((T, H), 7.0, dtype=torch.bfloat16, device=cuda_device)
    _ep_reduce_call(cuda_device, partials, flags, rank=0, epoch=1, limit_us=2000, status=status,
                    output=output)
    assert int(status.item()) & 0x4
    # the rows that could not be completed read as zeros, never as stale memory
    assert float(output.float().min()) == 0.0 and float(output.float().max()) == 0.0
    flags[0][1] = 1  # the peer arrives: the same call now completes
    status.zero_()
    _ep_reduce_call(cuda_device, partials, flags, rank=0, epoch=1, limit_us=2000, status=status,
                    output=output)
    assert int(status.item()) == 0
    assert float(output.float().min()) == 2.0


def _emulated_ranks(device, world, T, H, I, E, K, seed=9, routing="zipf"):
    """Every rank's local forward up to the down projection, one after another on one GPU."""

    from b200moe import B300MoEWorkspace, workloads
    from b200moe.expert_parallel import expert_range, local_partial_forward

    hidden, ids, weights, gate_up, down = workloads.make_case(
        T, H, I, E, K, routing=routing, weight_kind="raw", std=None, device=device, seed=seed)
    ranks = []
    for rank in range(world):
        base, count = expert_range(rank, world, E)
        workspace = B300MoEWorkspace(device=device)
        _, call = local_partial_forward(
            hidden, ids, weights, gate_up[base:base + count].contiguous(),
            down[base:base + count].contiguous(), top_k=K, expert_id_base=base,
            num_experts_global=E, workspace=workspace, skip_combine=True)
        ranks.append((workspace, call))
    torch.cuda.synchronize(device)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                   down.cpu(), num_experts=E, top_k=K)
    return ranks, ref


def _combine_reduce_call(device, ranks, rank, partials, flags, counter, epoch, first, rows,
                         limit_us=0):
    import ctypes

    from b200moe import _lib

    world = len(ranks)
    workspace, (layer_args, _keep) = ranks[rank]
    H = partials[0].shape[1]
    args = _lib.B200MoeEpReduceArgs()
    p_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in partials])
    f_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in flags])
    args.partial_ptrs = ctypes.cast(p_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.flag_ptrs = ctypes.cast(f_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.world, args.rank, args.hidden_size = world, rank, H
    args.num_tokens, args.first_token = rows, first
    args.epoch, args.wait_limit_us = epoch, limit_us
    output = torch.full((rows, H), 7.0, dtype=torch.bfloat16, device=device)
    args.output = output.data_ptr()
    args.status = workspace.scratch.data_ptr()
    args.block_counter = counter.data_ptr()
    args.flags = 0
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = _lib.load().b200moe_ep_combine_reduce(ctypes.byref(layer_args), ctypes.byref(args),
                                                 stream)
    _lib.check(code, "b200moe_ep_combine_reduce")
    torch.cuda.synchronize(device)
    return output


@pytest.mark.parametrize("spec", [(4, 16, 256, 384, 8, 2), (8, 64, 512, 256, 16, 4),
                                  (2, 1300, 64, 96, 8, 2)],
                         ids=["world4", "world8", "two_kernel_path_T1300"])
def test_fused_combine_reduce_with_all_ranks_buffers_on_one_gpu(spec, cuda_device) -> None:
    """The one-kernel combine + cross-rank reduce of an expert-parallel rank, with every
    rank's buffers on this GPU.  Kernels of different ranks are never in flight together
    here: every flag is pre-set to the epoch, and the ranks run twice in turn -- the first
    round leaves every rank's partial rows in its buffer, the second reads them all.  The
    result must meet the oracle bar, be identical on every rank, and a sharded caller's rows
    must equal the same rows of the replicated result.  The third case is large enough to
    take the two-kernel path inside the same entry point."""

    world, T, H, I, E, K = spec
    ranks, ref = _emulated_ranks(cuda_device, world, T, H, I, E, K)
    partials = [torch.full((T, H), float("nan"), device=cuda_device) for _ in range(world)]
    flags = [torch.full((8,), 3, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    outputs = None
    for _round in range(2):
        outputs = [_combine_reduce_call(cuda_device, ranks, r, partials, flags, counter, 3, 0, T)
                   for r in range(world)]
    for r in range(world):
        assert ranks[r][0].status() == 0
        assert torch.equal(outputs[r], outputs[0])
    assert int(counter.item()) == 0  # the last block of every launch reset it
    err = moe_oracle.relative_max_error(outputs[0].float().cpu(), ref)
    assert err <= 2e-2, err
    # a sharded caller: rank 1 outputs only its own T/world rows
    per = T // world
    mine = _combine_reduce_call(cuda_device, ranks, 1, partials, flags, counter, 3, per, per)
    assert torch.equal(mine, outputs[0][per:2 * per])


def _combine_push_call(device, ranks, rank, inboxes, flags, epoch, first, rows, cap,
                       tokens_per_rank, limit_us):
    import ctypes

    from b200moe import _lib

    world = len(ranks)
    workspace, (layer_args, _keep) = ranks[rank]
    H = layer_args.hidden_size
    args = _lib.B200MoeEpReduceArgs()
    i_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in inboxes])
    f_ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in flags])
    args.inbox_ptrs = ctypes.cast(i_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.flag_ptrs = ctypes.cast(f_ptrs, ctypes.POINTER(ctypes.c_void_p))
    args.world, args.rank, args.hidden_size = world, rank, H
    args.num_tokens, args.first_token = rows, first
    args.inbox_cap_tokens, args.tokens_per_rank = cap, tokens_per_rank
    args.epoch, args.wait_limit_us = epoch, limit_us
    output = torch.full((rows, H), 7.0, dtype=torch.bfloat16, device=device)
    args.output = output.data_ptr()
    args.status = workspace.scratch.data_ptr()
    args.flags = _lib.FLAG_EP_PUSH
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = _lib.load().b200moe_ep_combine_reduce(ctypes.byref(layer_args), ctypes.byref(args),
                                                 stream)
    _lib.check(code, "b200moe_ep_combine_reduce (push)")
    torch.cuda.synchronize(device)
    return output


@pytest.mark.parametrize("spec", [(4, 16, 256, 384, 8, 2), (8, 64, 512, 256, 16, 4),
                                  (2, 8, 1160, 256, 8, 2)],
                         ids=["world4", "world8", "world2_ragged_width"])
def test_push_combine_reduce_with_all_ranks_inboxes_on_one_gpu(spec, cuda_device) -> None:
    """The flagged-row push variant with every rank's inbox on this GPU.  Ranks run one after
    another, never together: in the first round a rank that runs before the owners of its
    tokens finds its inbox incomplete, gives up after its (short) limit, zeroes the rows and
    sets the status bit -- which is the bounded-wait behaviour -- while its own rows still land
    in every inbox; in the second round every inbox holds this epoch's rows and all ranks
    complete.  Results meet the oracle bar, agree across ranks and with the pull variant's
    rank-order sum; a sharded caller gets exactly its rows."""

    from b200moe import _lib

    world, T, H, I, E, K = spec
    ranks, ref = _emulated_ranks(cuda_device, world, T, H, I, E, K)
    cap = T
    inboxes = [torch.zeros(2 * world * cap * H * 2, dtype=torch.int32, device=cuda_device)
               for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    epoch = 1
    first_round = [_combine_push_call(cuda_device, ranks, r, inboxes, flags, epoch, 0, T, cap, 0,
                                      limit_us=1500) for r in range(world)]
    timed_out = [bool(ranks[r][0].status() & _lib.STATUS_PEER_TIMEOUT) for r in range(world)]
    assert timed_out[0]  # rank 0 ran before every other owner
    assert first_round[0].shape == (T, H)
    for r in range(world):
        ranks[r][0].scratch[:4].zero_()
    outputs = [_combine_push_call(cuda_device, ranks, r, inboxes, flags, epoch, 0, T, cap, 0,
                                  limit_us=1500) for r in range(world)]
    for r in range(world):
        assert ranks[r][0].status() == 0
        assert torch.equal(outputs[r], outputs[0])
    err = moe_oracle.relative_max_error(outputs[0].float().cpu(), ref)
    assert err <= 2e-2, err
    # every rank announced its epoch in slot `rank` of every rank's progress array
    assert all(int(f[r]) == epoch for f in flags for r in range(world))
    # same sum order as the pull variant: bit-identical results
    partials = [torch.zeros(T, H, device=cuda_device) for _ in range(world)]
    pflags = [torch.full((8,), 3, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    pulled = None
    for _round in range(2):
        pulled = [_combine_reduce_call(cuda_device, ranks, r, partials, pflags, counter, 3, 0, T)
                  for r in range(world)]
    assert torch.equal(pulled[0], outputs[0])
    # sharded tokens at the next epoch: rank 1 outputs its own T/world rows only, and only
    # pushes aimed at it land in its inbox
    per = T // world
    for r in range(world):
        flags[r][:] = epoch  # every rank has begun the previous epoch
    for _round in range(2):
        rows = [_combine_push_call(cuda_device, ranks, r, inboxes, flags, epoch + 1, r * per,
                                   per, cap, per, limit_us=1500) for r in range(world)]
        for r in range(world):
            if _round == 0:
                ranks[r][0].scratch[:4].zero_()
    for r in range(world):
        assert ranks[r][0].status() == 0
        assert torch.equal(rows[r], outputs[0][r * per:(r + 1) * per])


def test_fused_combine_reduce_reports_a_missing_peer(cuda_device) -> None:
    """A peer that never publishes its flag: the wait runs out after its limit, the rows come
    back as zeros with the status bit set, and the same call completes once the flag is there."""

    world, T, H, I, E, K = 2, 4, 128, 256, 4, 2
    ranks, _ = _emulated_ranks(cuda_device, world, T, H, I, E, K, routing="uniform")
    partials = [torch.zeros(T, H, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = _combine_reduce_call(cuda_device, ranks, 0, partials, flags, counter, 1, 0, T,
                               limit_us=2000)
    assert ranks[0][0].status() & 0x4
    assert not out.any()
    with pytest.raises(RuntimeError):
        ranks[0][0].raise_for_status()
    assert [int(f[0]) for f in flags] == [1, 1]  # rank 0 did publish its own epoch
    flags[0][1] = 1
    ranks[0][0].scratch[:4].zero_()
    out = _combine_reduce_call(cuda_device, ranks, 0, partials, flags, counter, 1, 0, T,
                               limit_us=2000)
    assert ranks[0][0].status() == 0


@pytest.mark.parametrize("use_pdl", [False, True])
def test_forward_replays_from_a_cuda_graph(use_pdl, cuda_device) -> None:
    """The whole layer is five launches and no allocation in the library, so a decode step
    can be captured once and replayed with new activations and routes.  (The reference
    could not do this: its grouped GEMM allocates inside ATen, docs/goal_1b_report.md:189-194.)"""

    from b200moe import B300MoEWorkspace, b300_moe_forward

    hidden, ids, weights, gate_up, down = _case(cuda_device, tokens=8, hidden=256, inter=384)
    workspace = B300MoEWorkspace(capacity_tokens=8, device=cuda_device)
    kwargs = dict(num_experts=16, top_k=2, workspace=workspace, use_pdl=use_pdl)
    b300_moe_forward(hidden, ids, weights, gate_up, down, **kwargs)  # reserve before capture
    torch.cuda.synchronize(cuda_device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = b300_moe_forward(hidden, ids, weights, gate_up, down, **kwargs)
    other = _case(cuda_device, tokens=8, hidden=256, inter=384, seed=99, routing="zipf")
    hidden.copy_(other[0])
    ids.copy_(other[1])
    weights.copy_(other[2])
    graph.replay()
    torch.cuda.synchronize(cuda_device)
    replayed = captured.clone()
    eager = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=16, top_k=2,
                             use_pdl=use_pdl)
    assert torch.equal(replayed, eager)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                   down.cpu(), num_experts=16, top_k=2)
    assert moe_oracle.relative_max_error(replayed.float().cpu(), ref) <= 2e-2


from conftest import ROUTER_CASES  # noqa: E402


@pytest.mark.parametrize("case", ROUTER_CASES, ids=lambda c: c["label"])
def test_router_topk_matches_reference_golden(case, cuda_device) -> None:
    """The router kernel against what the reference's topk_routing returned for the same
    logits: ids exact on tie-free selections, softmax weights to one ulp of their dtype."""

    from b200moe import topk_routing

    top_k = case["ids"].shape[1]
    ids, weights = topk_routing(case["logits"].to(cuda_device), top_k)
    assert ids.dtype == torch.int64 and weights.dtype == case["weights"].dtype
    selected = torch.gather(case["logits"].float(), 1, case["ids"])
    tie_free = (selected[:, :-1] != selected[:, 1:]).all(dim=1) if top_k > 1 else \
        torch.ones(selected.shape[0], dtype=torch.bool)
    assert torch.equal(ids.cpu()[tie_free], case["ids"][tie_free])
    # the logits the kernel picked are the reference's, ties or not
    torch.testing.assert_close(
        torch.gather(case["logits"].float(), 1, ids.cpu()), selected, atol=0, rtol=0)
    ulp = 2.0 ** -7 if weights.dtype == torch.bfloat16 else 2.0 ** -22
    torch.testing.assert_close(weights.float().cpu(), case["weights"].float(), atol=ulp,
                               rtol=ulp)


def test_router_keeps_ids_in_range_on_nan_and_infinite_logits(cuda_device) -> None:
    """A NaN logit ranks first, as in ``torch.topk``; rows of -inf or NaN still give top_k
    distinct experts in [0, E), so a poisoned router output cannot index past the weights."""

    from b200moe import topk_routing

    E, K = 40, 4
    logits = torch.randn(5, E, generator=torch.Generator().manual_seed(9))
    logits[1, 17] = float("nan")
    logits[2] = float("-inf")
    logits[3] = float("nan")
    logits[4, :38] = float("-inf")          # fewer finite logits than top_k
    ids, weights = topk_routing(logits.to(cuda_device), K)
    ids = ids.cpu()
    assert int(ids.min()) >= 0 and int(ids.max()) < E
    assert all(len(set(row.tolist())) == K for row in ids)
    want_ids, _ = moe_oracle.topk_routing(logits, K)
    assert torch.equal(ids[0], want_ids[0])
    assert int(ids[1, 0]) == 17 and torch.equal(ids[1, 1:], want_ids[0 + 1, 1:])
    assert ids[2].tolist() == [0, 1, 2, 3] and ids[3].tolist() == [0, 1, 2, 3]
    assert ids[4].tolist() == [38, 39, 0, 1] or ids[4].tolist() == [39, 38, 0, 1]
    assert torch.isfinite(weights[0]).all()


def test_router_then_layer_end_to_end(cuda_device) -> None:
    from b200moe import b300_moe_forward, topk_routing, workloads

    T, H, I, E, K = 16, 256, 384, 32, 4
    hidden, _, _, gate_up, down = workloads.make_case(T, H, I, E, K, std=None, device=cuda_device)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(4)).to(
        device=cuda_device, dtype=torch.bfloat16)
    ids, weights = topk_routing(logits, K)
    out = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
    ref_ids, ref_w = moe_oracle.topk_routing(logits.cpu(), K)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ref_ids, ref_w, gate_up.cpu(), down.cpu(),
                                   num_experts=E, top_k=K)
    assert moe_oracle.relative_max_error(out.float().cpu(), ref) <= 2e-2


def _forward_with_buffers(tensors, E, K, cuda_device, **kwargs):
    """One forward on a fresh workspace; returns the output, the metadata and copies of the
    public buffers a caller can observe."""

    from b200moe import B300MoEWorkspace, b300_moe_forward

    workspace = B300MoEWorkspace(device=cuda_device)
    out, meta = b300_moe_forward(*tensors, num_experts=E, top_k=K, workspace=workspace,
                                 return_metadata=True, **kwargs)
    torch.cuda.synchronize(cuda_device)
    rows = tensors[1].numel()
    valid = int(meta["expert_counts"].sum())
    buffers = {name: workspace.buffers[name][:rows].clone()
               for name in ("permuted_hidden", "swiglu_output", "permuted_token_indices",
                            "permuted_expert_indices", "permuted_weights", "expert_output")}
    return out, meta, buffers, valid, workspace


SMALL_CALL_CASES = [
    # T, H, I, E, K, routing
    (1, 512, 768, 8, 2, "uniform"),
    (4, 512, 768, 32, 8, "concentrated"),   # 32 assignments, 4 rows on each of 8 experts
    (16, 256, 384, 8, 2, "zipf"),           # 32 assignments
    (5, 512, 768, 16, 4, "zipf"),
    (3, 1024, 256, 256, 8, "uniform"),
    (2, 2880, 2880, 32, 8, "concentrated"),  # ragged tiles (I, H not multiples of 128)
    (1, 4096, 14336, 8, 2, "uniform"),      # Mixtral-shaped, one token
]


@pytest.mark.parametrize("spec", SMALL_CALL_CASES, ids=lambda s: "T{}_H{}_I{}_E{}_K{}_{}".format(*s))
@pytest.mark.parametrize("use_pdl", [True, False])
def test_small_call_order_equals_regular_order_bitwise(spec, use_pdl, cuda_device) -> None:
    """Calls with at most 32 assignments run gate+up first and the routing kernel beside it.
    That is a scheduling choice only: output, routing tensors and every public buffer are
    bit-identical to the regular order, and the output meets the oracle bar."""

    from b200moe import _lib, workloads
    from oracle import moe_oracle

    T, H, I, E, K, routing = spec
    tensors = workloads.make_case(T, H, I, E, K, routing=routing, std=0.02 if H >= 2048 else None,
                                  device=cuda_device, seed=77 + T)
    lib = _lib.load()
    results = {}
    try:
        for most in (0, 32):
            assert lib.b200moe_tune(_lib.TUNE_SMALL_CALL_MAX, most) == 0
            results[most] = _forward_with_buffers(tensors, E, K, cuda_device, use_pdl=use_pdl,
                                                  check_status=True)
    finally:
        lib.b200moe_tune(_lib.TUNE_SMALL_CALL_MAX, -1)   # back to the default rule
    (out0, meta0, buf0, valid0, _), (out1, meta1, buf1, valid1, ws1) = results[0], results[32]
    assert torch.equal(out0, out1)
    for key in ("expert_counts", "expert_offsets", "permutation", "reverse_mapping"):
        assert torch.equal(meta0[key], meta1[key]), key
    assert valid0 == valid1 == T * K
    for name in buf0:
        assert torch.equal(buf0[name], buf1[name]), name
    timeline = ws1.timeline()
    assert "gather" not in timeline  # the gate+up blocks did the gather
    assert timeline["gate_up"][0] <= timeline["routing"][0] + 50.0
    assert timeline["gate_up"][1] <= timeline["down"][1] <= timeline["combine"][1]
    assert timeline["down_first_data"][0] >= timeline["gate_up"][1]
    if H < 2048:  # the large shape is covered against the oracle in test_gpu_layer.py
        cpu = [t.float().cpu() if t.is_floating_point() else t.cpu() for t in tensors]
        ref, _ = moe_oracle.routed_moe(*cpu, num_experts=E, top_k=K)
        assert moe_oracle.relative_max_error(out1.float().cpu(), ref) <= 2e-2


HANDOVER_CASES = [
    # T, H, I, E, K, routing  (I <= H is where the host applies the hand-over by default)
    (40, 512, 256, 8, 2, "uniform"),
    (150, 512, 384, 4, 2, "uniform"),        # experts longer than one 128-row segment
    (64, 1024, 512, 64, 8, "zipf"),          # many small segments, empty experts
    (33, 2880, 2880, 32, 8, "concentrated"),  # ragged tiles
    (17, 256, 384, 8, 2, "uniform"),         # I > H: only reached through the knob
]


@pytest.mark.parametrize("spec", HANDOVER_CASES, ids=lambda s: "T{}_H{}_I{}_E{}_K{}_{}".format(*s))
def test_segment_handover_equals_the_grid_wait_bitwise(spec, cuda_device) -> None:
    """With the hand-over a down block waits for the gate+up tiles of its own segment (a
    counter in the schedule entry) instead of the whole gate+up grid.  A scheduling choice
    only: outputs and public buffers are bit-identical with it forced on and off, over
    repeated calls on one workspace, and the output meets the oracle bar."""

    from b200moe import B300MoEWorkspace, _lib, b300_moe_forward, workloads
    from oracle import moe_oracle

    T, H, I, E, K, routing = spec
    tensors = workloads.make_case(T, H, I, E, K, routing=routing, std=0.02 if H >= 2048 else None,
                                  device=cuda_device, seed=91 + T)
    lib = _lib.load()
    results = {}
    try:
        for mode in (0, 1):
            assert lib.b200moe_tune(_lib.TUNE_GEMM_OVERLAP, mode) == 0
            results[mode] = _forward_with_buffers(tensors, E, K, cuda_device, check_status=True)
        # many calls in a row: the counters are zeroed by every forward's routing kernel
        assert lib.b200moe_tune(_lib.TUNE_GEMM_OVERLAP, 1) == 0
        ws = B300MoEWorkspace(device=cuda_device)
        for _ in range(50):
            again = b300_moe_forward(*tensors, num_experts=E, top_k=K, workspace=ws)
        torch.cuda.synchronize(cuda_device)
        assert ws.status() == 0
    finally:
        lib.b200moe_tune(_lib.TUNE_GEMM_OVERLAP, -1)   # back to the default rule
    (out0, meta0, buf0, valid0, _), (out1, meta1, buf1, valid1, ws1) = results[0], results[1]
    assert torch.equal(out0, out1) and torch.equal(out1, again)
    for name in buf0:
        assert torch.equal(buf0[name], buf1[name]), name
    cpu = [t.float().cpu() if t.is_floating_point() else t.cpu() for t in tensors]
    ref, _ = moe_oracle.routed_moe(*cpu, num_experts=E, top_k=K)
    assert moe_oracle.relative_max_error(out1.float().cpu(), ref) <= 2e-2


def test_small_call_order_with_dropped_ids_and_local_experts(cuda_device) -> None:
    """Small-call order under the two conditions that change which rows exist: an id outside
    [0, E) (row dropped, status bit, zero-filled gather row) and an expert-parallel rank's
    local id range (foreign ids dropped silently)."""

    from b200moe import B300MoEWorkspace, _lib, b300_moe_forward, workloads
    from b200moe.expert_parallel import local_partial_forward

    lib = _lib.load()
    T, H, I, E, K = 6, 256, 384, 8, 4
    hidden, ids, weights, gate_up, down = workloads.make_case(
        T, H, I, E, K, routing="uniform", std=None, device=cuda_device, seed=5)
    bad = ids.clone()
    bad[1, 2] = E + 3
    bad[4, 0] = -1
    outs = {}
    try:
        for most in (0, 32):
            lib.b200moe_tune(_lib.TUNE_SMALL_CALL_MAX, most)
            ws = B300MoEWorkspace(device=cuda_device)
            out = b300_moe_forward(hidden, bad, weights, gate_up, down, num_experts=E, top_k=K,
                                   workspace=ws)
            torch.cuda.synchronize(cuda_device)
            assert ws.status() & _lib.STATUS_BAD_EXPERT_ID
            rows = T * K
            outs[most] = (out, ws.buffers["permuted_hidden"][:rows].clone(),
                          ws.buffers["reverse_mapping"][:rows].clone())
            # the two rows past the valid ones are zero, as the gather kernel leaves them
            assert not ws.buffers["permuted_hidden"][rows - 2:rows].any()
            # one rank of two: experts [4, 8) only
            ws2 = B300MoEWorkspace(device=cuda_device)
            part, _ = local_partial_forward(hidden, ids, weights, gate_up[4:].contiguous(),
                                            down[4:].contiguous(), top_k=K, expert_id_base=4,
                                            num_experts_global=E, workspace=ws2)
            torch.cuda.synchronize(cuda_device)
            assert ws2.status() == 0
            outs[most] += (part.clone(),)
    finally:
        lib.b200moe_tune(_lib.TUNE_SMALL_CALL_MAX, -1)   # back to the default rule
    for a, b in zip(outs[0], outs[32]):
        assert torch.equal(a, b)


def test_peer_dispatch_kernel_and_routing_wait_on_one_gpu(cuda_device) -> None:
    """Sharded-token dispatch with both "ranks'" buffers on this GPU: the push kernel lands
    this rank's shard in slot `rank` of every gathered buffer and publishes its flag; the
    forward waits on the flags, and a flag nothing sets ends the wait with a status bit and
    an all-zero result instead of a hang."""

    import ctypes

    from b200moe import B300MoEWorkspace, _lib, workloads
    from b200moe.expert_parallel import local_partial_forward

    world, rank, t_local, H, I, E, K = 2, 1, 3, 128, 192, 8, 2
    total = world * t_local
    hidden, ids, weights, gate_up, down = workloads.make_case(
        total, H, I, E, K, std=None, device=cuda_device)
    mine = slice(rank * t_local, (rank + 1) * t_local)
    g_hidden = [torch.zeros(total, H, dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    g_ids = [torch.full((total, K), -1, dtype=torch.int64, device=cuda_device) for _ in range(world)]
    g_w = [torch.zeros(total, K, dtype=torch.bfloat16, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device=cuda_device)

    def ptrs(tensors, row_bytes):
        return (ctypes.c_void_p * world)(*[t.data_ptr() + rank * t_local * row_bytes
                                           for t in tensors])

    args = _lib.B200MoeEpPushArgs()
    srcs = (hidden[mine].contiguous(), ids[mine].contiguous(), weights[mine].contiguous())
    args.hidden_states, args.expert_indices, args.expert_weights = (t.data_ptr() for t in srcs)
    keep = (ptrs(g_hidden, H * 2), ptrs(g_ids, K * 8), ptrs(g_w, K * 2),
            (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags]))
    cast = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_void_p))  # noqa: E731
    args.hidden_dst, args.indices_dst, args.weights_dst, args.flag_ptrs = (cast(a) for a in keep)
    args.block_counter = counter.data_ptr()
    args.world, args.rank, args.tokens_local, args.top_k, args.hidden_size = world, rank, t_local, K, H
    args.epoch = 7
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    _lib.check(_lib.load().b200moe_ep_push(ctypes.byref(args), stream), "b200moe_ep_push")
    torch.cuda.synchronize(cuda_device)
    for r in range(world):
        assert torch.equal(g_hidden[r][mine], hidden[mine])
        assert torch.equal(g_ids[r][mine], ids[mine])
        assert torch.equal(g_w[r][mine], weights[mine])
        assert int(g_ids[r][: rank * t_local].max()) == -1  # other slots untouched
        assert int(flags[r][rank]) == 7
    assert int(counter.item()) == 0

    # the consumer: rank 1's forward over the gathered inputs waits on its own flag array
    g_hidden[rank].copy_(hidden)
    g_ids[rank].copy_(ids)
    g_w[rank].copy_(weights)
    workspace = B300MoEWorkspace(device=cuda_device)
    wait = (flags[rank].data_ptr(), world, 7)
    partial, (native_args, _) = local_partial_forward(
        g_hidden[rank], g_ids[rank], g_w[rank], gate_up, down, top_k=K, expert_id_base=0,
        num_experts_global=E, workspace=workspace, ep_wait=wait)
    # rank 0 never published: bounded wait (default 1 s), status bit, nothing routed
    torch.cuda.synchronize(cuda_device)
    assert workspace.status() & 0x4
    assert float(partial.abs().max()) == 0.0
    flags[rank][0] = 7  # now "rank 0" has arrived
    partial, _ = local_partial_forward(
        g_hidden[rank], g_ids[rank], g_w[rank], gate_up, down, top_k=K, expert_id_base=0,
        num_experts_global=E, workspace=workspace, ep_wait=wait)
    torch.cuda.synchronize(cuda_device)
    assert workspace.status() == 0
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                   down.cpu(), num_experts=E, top_k=K)
    assert moe_oracle.relative_max_error(partial.to(torch.bfloat16).float().cpu(), ref) <= 2e-2


@pytest.mark.parametrize("tokens, experts, top_k", [(1, 256, 1), (7, 16, 2), (64, 64, 8),
                                                     (300, 32, 4)])
def test_legacy_dispatch_and_combine(tokens, experts, top_k, cuda_device) -> None:
    """The older dispatch/combine API (tests/test_cuda_ops.py:25-133 of the reference):
    mappings equal the stable argsort and its inverse, the gather is exact, the combine
    matches the FP32 formula of fastpath/ops.py:264-268."""

    from b200moe import combine_tokens, dispatch_tokens, workloads

    H = 256
    g = torch.Generator().manual_seed(tokens * 31 + top_k)
    hidden = torch.randn(tokens, H, generator=g).to(device=cuda_device, dtype=torch.bfloat16)
    ids = workloads.make_routing(tokens, experts, top_k, "duplicates", 5).to(cuda_device)
    weights = torch.randn(tokens, top_k, generator=g).to(device=cuda_device,
                                                         dtype=torch.bfloat16)
    result = dispatch_tokens(hidden, ids, experts)
    want = moe_oracle.group_tokens(ids.cpu(), experts)
    assert result.permuted_to_assignment.cpu().tolist() == want.permutation.tolist()
    assert result.assignment_to_permuted.cpu().tolist() == want.reverse_mapping.tolist()
    assert result.expert_counts.cpu().tolist() == want.expert_counts.tolist()
    assert result.expert_offsets.cpu().tolist() == want.expert_offsets.tolist()
    rows = hidden.cpu()[torch.from_numpy(want.permuted_token_indices)]
    assert torch.equal(result.permuted_hidden.cpu(), rows)

    expert_rows = torch.randn(tokens * top_k, H, generator=g).to(device=cuda_device,
                                                                 dtype=torch.bfloat16)
    out = combine_tokens(expert_rows, result.assignment_to_permuted, weights)
    ordered = expert_rows.cpu().float()[result.assignment_to_permuted.cpu()]
    expected = (ordered.reshape(tokens, top_k, H) * weights.cpu().float().unsqueeze(-1)).sum(1)
    torch.testing.assert_close(out.float().cpu(), expected, atol=1e-2 * max(1.0, top_k ** 0.5),
                               rtol=1e-2)
    with pytest.raises(RuntimeError, match="not an execution path"):
        dispatch_tokens(hidden, ids, experts, backend="torch")
    with pytest.raises(TypeError, match="int64"):
        dispatch_tokens(hidden, ids.int(), experts)


def test_pinned_host_io_matches_device_io(cuda_device) -> None:
    """Per-step tensors in pinned host memory, read and written by the kernels directly:
    same bits as the device-tensor entry point."""

    from b200moe import B300MoEWorkspace, b300_moe_forward, b300_moe_forward_pinned, workloads

    T, H, I, E, K = 9, 512, 768, 16, 4
    hidden, ids, weights, gate_up, down = workloads.make_case(
        T, H, I, E, K, routing="zipf", std=None, device=cuda_device)
    want = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
    host = tuple(t.cpu().pin_memory() for t in (hidden, ids, weights))
    workspace = B300MoEWorkspace(capacity_tokens=16, device=cuda_device)
    for _ in range(2):
        got = b300_moe_forward_pinned(*host, gate_up, down, num_experts=E, top_k=K,
                                      workspace=workspace)
        torch.cuda.synchronize(cuda_device)
        assert got.is_pinned() and got.device.type == "cpu"
        assert torch.equal(got, want.cpu())
    assert workspace.status() == 0
    with pytest.raises(ValueError, match="pinned"):
        b300_moe_forward_pinned(hidden.cpu(), *host[1:], gate_up, down, num_experts=E, top_k=K,
                                workspace=workspace)
    bad = host[1].clone().pin_memory()
    bad[0, 0] = E
    with pytest.raises(ValueError, match="out-of-range"):
        b300_moe_forward_pinned(host[0], bad, host[2], gate_up, down, num_experts=E, top_k=K,
                                workspace=workspace)


@pytest.mark.gpu
def test_out_tensor_on_the_device_or_in_pinned_host_memory(cuda_device) -> None:
    """``out=``: the combine kernel stores into the caller's tensor -- on the device, or in
    pinned host memory (no device-to-host copy) -- with the same bits as the returned
    tensor of a plain call, on the checked path and on the repeated-call path, for the
    small-call order (T * K <= 32) and the five-launch order."""

    from b200moe import B300MoEWorkspace, b300_moe_forward, workloads

    for T in (3, 40):
        H, I, E, K = 512, 768, 16, 2
        hidden, ids, weights, gate_up, down = workloads.make_case(
            T, H, I, E, K, routing="zipf", std=None, device=cuda_device)
        want = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
        workspace = B300MoEWorkspace(capacity_tokens=64, device=cuda_device)
        on_device = torch.empty_like(hidden)
        on_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        for _ in range(3):  # first call checked, then the remembered plan
            for out in (on_device, on_host):
                out.fill_(7.0)
                got = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E,
                                       top_k=K, workspace=workspace, out=out)
                torch.cuda.synchronize(cuda_device)
                assert got is out
                assert torch.equal(out.to(cuda_device), want)
        assert workspace.reuse_count >= 4 and workspace.status() == 0
        with pytest.raises(ValueError, match="out must be"):
            b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                             workspace=workspace, out=torch.empty(T + 1, H, dtype=torch.bfloat16,
                                                                  device=cuda_device))
        with pytest.raises(ValueError, match="pinned"):
            b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                             workspace=workspace, out=torch.empty(T, H, dtype=torch.bfloat16))
        # the quantised paths take it too
        from b200moe import b300_moe_forward_fp8, quantize_expert_weights_fp8

        fw = quantize_expert_weights_fp8(gate_up, down)
        want_fp8 = b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K)
        want_fp4 = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                                    backend="cutlass_nvfp4", quant_mode="nvfp4")
        for _ in range(2):
            b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K,
                                 workspace=workspace, out=on_host)
            torch.cuda.synchronize(cuda_device)
            assert torch.equal(on_host.to(cuda_device), want_fp8)
        fp4_workspace = B300MoEWorkspace(capacity_tokens=64, device=cuda_device)
        for _ in range(2):
            b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                             workspace=fp4_workspace, backend="cutlass_nvfp4",
                             quant_mode="nvfp4", out=on_host)
            torch.cuda.synchronize(cuda_device)
            assert torch.equal(on_host.to(cuda_device), want_fp4)


@pytest.mark.gpu
def test_bench_writes_reference_csv_schema(tmp_path):
    """``bench.py --csv`` emits the column set and stage names of the reference's result
    files (benchmark/benchmark_goal_1b.py:55-64, 77-122), one row per (T, stage)."""

    import csv
    import json
    import subprocess
    import sys

    repo = Path(__file__).resolve().parents[1]
    out = tmp_path / "stages.csv"
    proc = subprocess.run(
        [sys.executable, str(repo / "bench.py"), "--only-tokens", "1", "4", "--steps", "3",
         "--warmup", "3", "--no-cpu-baseline", "--csv", str(out)],
        capture_output=True, text=True, timeout=600, check=True,
    )
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["csv"]["rows"] == 16
    with out.open(newline="", encoding="utf-8") as handle:
        rows = list(csv.DictReader(handle))
    assert len(rows) == 16
    assert list(rows[0].keys())[:5] == ["backend_set_requested", "requested_backend",
                                        "actual_backend", "device", "gpu_name"]
    assert len(rows[0]) == 44
    stages = [r["stage"] for r in rows[:8]]
    assert stages == ["routing_us", "permutation_us", "quantization_us", "gate_up_gemm_us",
                      "swiglu_us", "down_gemm_us", "combine_us", "total_us"]
    by_stage = {r["stage"]: r for r in rows[:8]}
    assert by_stage["quantization_us"]["stage_status"] == "not_applicable"
    assert by_stage["swiglu_us"]["stage_status"] == "fused_in_gate_up"
    assert by_stage["total_us"]["stage_status"] == "measured"
    assert float(by_stage["total_us"]["p50_us"]) > 50.0
    assert all(r["used_fallback"] == "false" and r["architecture"] == "sm_100a" for r in rows)
    assert {r["num_tokens"] for r in rows} == {"1", "4"}


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8"])
def test_graphed_layer_replays_equal_eager_calls(fp8, cuda_device) -> None:
    """GraphedMoEDecodeLayer: one captured graph per token count, bit-identical to the eager
    call for changing inputs; other token counts fall back to an eager call on a separate
    workspace and leave the captured graphs intact."""

    from b200moe import (GraphedMoEDecodeLayer, b300_moe_forward, b300_moe_forward_fp8,
                         quantize_expert_weights_fp8, workloads)

    H, I, E, K = 256, 384, 8, 2
    _, _, _, gate_up, down = workloads.make_case(1, H, I, E, K, std=None, device=cuda_device)
    fw = quantize_expert_weights_fp8(gate_up, down) if fp8 else None
    layer = GraphedMoEDecodeLayer(None if fp8 else gate_up, None if fp8 else down, num_experts=E,
                                  top_k=K, token_counts=(1, 4, 16), fp8_weights=fw)
    assert layer.token_counts == (1, 4, 16)

    def eager(hidden, ids, weights):
        if fp8:
            return b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K)
        return b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)

    for seed, T in enumerate((4, 1, 16, 4, 5, 16, 1)):
        hidden, ids, weights, _, _ = workloads.make_case(T, H, I, E, K, seed=300 + 3 * seed,
                                                         routing="zipf", device="cpu")
        hidden, ids, weights = (t.to(cuda_device) for t in (hidden, ids, weights))
        got = layer(hidden, ids, weights, copy=True)
        assert torch.equal(got, eager(hidden, ids, weights)), (seed, T)
    assert layer.replays == 6 and layer.eager_calls == 1
    assert layer.workspace.allocation_count == 1


@pytest.mark.gpu
def test_graphed_layer_with_the_router_inside(cuda_device) -> None:
    """Router logits -> top-k + softmax -> layer in one graph replay."""

    from b200moe import GraphedMoEDecodeLayer, b300_moe_forward, topk_routing, workloads

    H, I, E, K = 256, 384, 16, 4
    _, _, _, gate_up, down = workloads.make_case(1, H, I, E, K, std=None, device=cuda_device)
    layer = GraphedMoEDecodeLayer(gate_up, down, num_experts=E, top_k=K, token_counts=(2, 8),
                                  route_logits=True)
    g = torch.Generator().manual_seed(17)
    for T in (8, 2, 8):
        hidden = workloads.make_hidden(T, H, seed=int(torch.randint(0, 1000, (1,), generator=g)))
        logits = torch.randn(T, E, generator=g).to(torch.bfloat16)
        hidden, logits = hidden.to(cuda_device), logits.to(cuda_device)
        got = layer.forward_logits(hidden, logits, copy=True)
        ids, weights = topk_routing(logits, K)
        want = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
        assert torch.equal(got, want)
    with pytest.raises(ValueError, match="router inside"):
        layer(hidden, ids, weights)
