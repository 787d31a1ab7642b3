"""GPU tests of the FP8 (E4M3) expert-weight path, through the C ABI.

There is no reference implementation of a quantised layer to compare with (the reference's
quantised backend always raises), so the bars are: the weight format bit-exact against the
format oracle (itself pinned to ``torch.float8_e4m3fn``); routing tensors bit-exact against
the routing oracle; the layer output within ``2e-2 x rms`` of the FP32 oracle evaluated on
the dequantised weights -- the BF16 path's bar.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import fp8_oracle, moe_oracle

pytestmark = pytest.mark.gpu

TOLERANCE = 2e-2
QUANTISATION_RMS_BOUND = 0.06   # FP8 layer against the unquantised layer, RMS over RMS


def _case(E, H, I, K, T, routing="uniform", seed=0, device=None):
    from b200moe import workloads

    gate_up, down = workloads.make_expert_weights(E, H, I, seed=1236 + seed, std=0.05, device="cpu")
    hidden = workloads.make_hidden(T, H, seed=1234 + seed)
    ids = workloads.make_routing(T, E, K, routing, 1235 + seed)
    weights = workloads.make_routing_weights(T, K, "softmax", 1235 + seed)
    return gate_up, down, hidden, ids, weights


def _reference(fw, hidden, ids, weights, E, K):
    gate_up = fp8_oracle.dequantize_rows(fw.gate_up_q.cpu().numpy(), fw.gate_up_scale.cpu().numpy())
    down = fp8_oracle.dequantize_rows(fw.down_q.cpu().numpy(), fw.down_scale.cpu().numpy())
    return moe_oracle.routed_moe(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)


def _check(out, ref, label):
    err = moe_oracle.relative_max_error(out.float().cpu(), ref)
    floor = moe_oracle.bf16_floor(ref)
    print(f"{label}: err/rms={err:.5f} floor={floor:.5f}")
    assert err <= max(TOLERANCE, 1.03 * floor), f"{label}: {err:.5f} (floor {floor:.5f})"


def test_every_e4m3_code_converts_exactly(cuda_device) -> None:
    from b200moe import dequantize_rows_fp8

    codes = torch.arange(256, dtype=torch.uint8).repeat(2).reshape(2, 256).contiguous()
    got = dequantize_rows_fp8(codes.to(cuda_device), None).float().cpu().numpy()
    table = fp8_oracle.e4m3_table()
    finite = ~np.isnan(table)
    for row in got:
        np.testing.assert_array_equal(row[finite], table[finite])
        assert abs(row[0x7F]) == 480.0 and abs(row[0xFF]) == 480.0  # documented for NaN codes


def test_row_quantiser_matches_the_oracle_bit_for_bit(cuda_device) -> None:
    from b200moe import dequantize_rows_fp8, quantize_rows_fp8

    g = torch.Generator().manual_seed(21)
    w = (torch.randn(3, 40, 272, generator=g) * 0.03).to(torch.bfloat16)
    w[0, 3] = 0
    w[1, 5, 100] = 7.0
    w[2, 7] *= 1e-3
    q, scale = quantize_rows_fp8(w.to(cuda_device))
    q_ref, scale_ref = fp8_oracle.quantize_rows(w)
    np.testing.assert_array_equal(q.cpu().numpy(), q_ref)
    np.testing.assert_array_equal(scale.cpu().numpy(), scale_ref)
    back = dequantize_rows_fp8(q, scale).float().cpu()
    want = fp8_oracle.dequantize_rows(q_ref, scale_ref).to(torch.bfloat16).float()
    assert torch.equal(back, want)


@pytest.mark.parametrize(
    "E,H,I,K,T,routing",
    [
        (8, 256, 512, 2, 16, "uniform"),
        (4, 80, 208, 2, 5, "uniform"),          # H, I not multiples of the 128-element stage
        (16, 128, 96, 4, 1, "uniform"),
        (8, 256, 512, 2, 64, "zipf"),
        (4, 128, 256, 2, 100, "uniform"),       # experts with more rows than one segment holds
        (8, 256, 512, 8, 33, "concentrated"),   # every token to the same experts
        (32, 64, 64, 1, 7, "empty_half"),
        (8, 2880, 2880, 4, 3, "uniform"),
    ],
)
def test_layer_matches_fp32_oracle_on_dequantised_weights(E, H, I, K, T, routing, cuda_device):
    from b200moe import B300MoEWorkspace, b300_moe_forward_fp8, quantize_expert_weights_fp8

    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, routing)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    ws = B300MoEWorkspace(device=cuda_device)
    out, meta = b300_moe_forward_fp8(
        hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device), fw,
        num_experts=E, top_k=K, workspace=ws, return_metadata=True, check_status=True)
    ref, routing_ref = _reference(fw, hidden, ids, weights, E, K)
    for key in ("permutation", "reverse_mapping", "expert_counts", "expert_offsets"):
        np.testing.assert_array_equal(meta[key].cpu().numpy(), getattr(routing_ref, key), err_msg=key)
    _check(out, ref, f"fp8 E{E} H{H} I{I} K{K} T{T} {routing}")
    # what the format itself costs against the unquantised layer: bounded, not only printed
    # (E4M3 keeps three mantissa bits; measured 4.2-4.7 % of the output RMS)
    exact, _ = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
    shift = float(((out.float().cpu() - exact) ** 2).mean().sqrt() / (exact ** 2).mean().sqrt())
    print(f"  fp8 quantisation: rms(out - unquantised) / rms = {shift:.4f}")
    assert shift <= QUANTISATION_RMS_BOUND, shift
    assert meta["backend"] == "b200_fp8" and meta["used_fallback"] is False
    assert meta["weight_bytes"] == fw.nbytes


def test_duplicates_negative_weights_and_repeatability(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, b300_moe_forward_fp8, quantize_expert_weights_fp8

    E, H, I, K, T = 8, 256, 384, 4, 9
    gate_up, down, hidden, ids, _ = _case(E, H, I, K, T, seed=2)
    ids[:, 1] = ids[:, 0]                      # the same expert twice in every token
    g = torch.Generator().manual_seed(8)
    weights = torch.randn(T, K, generator=g).to(torch.bfloat16)  # raw, some negative
    weights[0, 0] = 0
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    ws = B300MoEWorkspace(device=cuda_device)
    args = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device), fw)
    first = b300_moe_forward_fp8(*args, num_experts=E, top_k=K, workspace=ws, check_status=True)
    ref, _ = _reference(fw, hidden, ids, weights, E, K)
    _check(first, ref, "fp8 duplicates")
    for _ in range(3):
        again = b300_moe_forward_fp8(*args, num_experts=E, top_k=K, workspace=ws)
        assert torch.equal(first, again)
    assert ws.allocation_count == 1


def test_out_of_range_ids_are_dropped_and_reported(cuda_device) -> None:
    from b200moe import B300MoEWorkspace, _lib, b300_moe_forward_fp8, quantize_expert_weights_fp8

    E, H, I, K, T = 4, 128, 128, 2, 6
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, seed=3)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    bad = ids.clone()
    bad[2, 1] = E + 3
    ws = B300MoEWorkspace(device=cuda_device)
    out = b300_moe_forward_fp8(hidden.to(cuda_device), bad.to(cuda_device),
                               weights.to(cuda_device), fw, num_experts=E, top_k=K, workspace=ws)
    torch.cuda.synchronize()
    assert ws.status() & _lib.STATUS_BAD_EXPERT_ID
    with pytest.raises(ValueError, match="out-of-range"):
        ws.raise_for_status()
    # the dropped slot contributes nothing: same as a zero routing weight on a valid id
    fixed, zeroed = ids.clone(), weights.clone()
    fixed[2, 1] = 0
    zeroed[2, 1] = 0
    ref, _ = _reference(fw, hidden, fixed, zeroed, E, K)
    _check(out, ref, "fp8 dropped id")


def test_contract_errors(cuda_device) -> None:
    from b200moe import Fp8ExpertWeights, b300_moe_forward_fp8, quantize_expert_weights_fp8

    E, H, I, K, T = 4, 128, 128, 2, 4
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    dev = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device))
    with pytest.raises(TypeError, match="Fp8ExpertWeights"):
        b300_moe_forward_fp8(*dev, gate_up.to(cuda_device), num_experts=E, top_k=K)
    with pytest.raises(TypeError, match="bfloat16"):
        b300_moe_forward_fp8(dev[0].float(), dev[1], dev[2].float(), fw, num_experts=E, top_k=K)
    with pytest.raises(ValueError, match="top_k"):
        b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=4)
    wrong = Fp8ExpertWeights(fw.gate_up_q, fw.gate_up_scale[:, :-1].contiguous(), fw.down_q,
                             fw.down_scale)
    with pytest.raises(ValueError, match="scales"):
        b300_moe_forward_fp8(*dev, wrong, num_experts=E, top_k=K)
    # H = 72 is fine for the BF16 path (multiple of 8) but not here (multiple of 16)
    g72, d72, h72, i72, w72 = _case(4, 72, 128, 2, 3)
    with pytest.raises(ValueError, match="multiple of 16"):
        quantize_expert_weights_fp8(g72.to(cuda_device), d72.to(cuda_device))
    # FP8 weights are their own entry point: the backend names of b300_moe_forward never
    # select them, and a quantised backend name is never paired with another quant_mode
    from b200moe import b300_moe_forward

    with pytest.raises(ValueError, match="requires quant_mode='nvfp4'"):
        b300_moe_forward(*dev, gate_up.to(cuda_device), down.to(cuda_device), num_experts=E,
                         top_k=K, backend="cutlass_nvfp4", quant_mode="bf16")


def test_staged_calls_and_graph_replay_equal_the_forward(cuda_device) -> None:
    from b200moe import (B300MoEWorkspace, StagedLayer, b300_moe_forward_fp8,
                         quantize_expert_weights_fp8)

    E, H, I, K, T = 8, 256, 512, 2, 12
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, seed=5)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    dev = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device))
    ws = B300MoEWorkspace(device=cuda_device)
    want = b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=K, workspace=ws).clone()

    layer = StagedLayer(*dev, None, None, num_experts=E, top_k=K, fp8_weights=fw, use_pdl=False,
                        workspace=B300MoEWorkspace(device=cuda_device))
    for stage in ("routing", "gather", "gate_up_swiglu", "down", "combine"):
        layer.run_stage(stage)
    torch.cuda.synchronize()
    assert torch.equal(layer.output, want)

    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=K, workspace=ws)
    captured.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, want)


def test_mixtral_shaped_decode_step(cuda_device) -> None:
    """Full layer width on two experts' worth of weights: T=1 with the real H and I."""

    from b200moe import B300MoEWorkspace, b300_moe_forward_fp8, quantize_expert_weights_fp8, workloads

    E, H, I, K = 2, 4096, 14336, 2
    gate_up, down = workloads.make_expert_weights(E, H, I, seed=1236, std=0.02, device=cuda_device)
    fw = quantize_expert_weights_fp8(gate_up, down)
    for T in (1, 4):
        hidden = workloads.make_hidden(T, H, seed=1234)
        ids = workloads.make_routing(T, E, K, "uniform", 1235)
        weights = workloads.make_routing_weights(T, K, "softmax", 1235)
        out = b300_moe_forward_fp8(hidden.to(cuda_device), ids.to(cuda_device),
                                   weights.to(cuda_device), fw, num_experts=E, top_k=K,
                                   workspace=B300MoEWorkspace(device=cuda_device),
                                   check_status=True)
        ref, _ = _reference(fw, hidden, ids, weights, E, K)
        _check(out, ref, f"fp8 mixtral-shaped T={T}")


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_shares_with_fp8_weights(world, cuda_device) -> None:
    """Each rank's share of an expert-parallel forward with FP8 weights, run one after another
    on one GPU: the FP32 partial outputs add up to the FP8 layer."""

    from b200moe import B300MoEWorkspace, quantize_expert_weights_fp8
    from b200moe.expert_parallel import expert_range, local_partial_forward

    E, H, I, K, T = 8, 256, 384, 2, 16
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, "zipf", seed=7)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    dev = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device))
    total = torch.zeros(T, H, dtype=torch.float32, device=cuda_device)
    for rank in range(world):
        base, count = expert_range(rank, world, E)
        ws = B300MoEWorkspace(device=cuda_device)
        partial, _ = local_partial_forward(
            *dev, fw.gate_up_q[base:base + count].contiguous(),
            fw.down_q[base:base + count].contiguous(), top_k=K, expert_id_base=base,
            num_experts_global=E, workspace=ws,
            fp8_scales=(fw.gate_up_scale[base:base + count].contiguous(),
                        fw.down_scale[base:base + count].contiguous()))
        total += partial
        assert ws.status() == 0
    ref, _ = _reference(fw, hidden, ids, weights, E, K)
    _check(total.to(torch.bfloat16), ref, f"fp8 expert-parallel shares, world {world}")


def test_full_size_deepseek_shaped_layer_spot_checked(cuda_device) -> None:
    """E=256, K=8, H=7168, I=2048, T=64 with hot experts, all weights FP8 (10.5 GiB).  Three
    tokens are checked against the token/slot loop oracle on the dequantised weights of the
    experts they route to; routing tensors of the whole call bit-exact; two runs identical;
    and the output is exactly linear in a power-of-two scale of the routing weights."""

    from b200moe import B300MoEWorkspace, b300_moe_forward_fp8, quantize_expert_weights_fp8, workloads

    T, H, I, E, K = 64, 7168, 2048, 256, 8
    hidden, ids, weights, gate_up, down = workloads.make_case(
        T, H, I, E, K, routing="hotspot", weight_kind="softmax", device=cuda_device)
    fw = quantize_expert_weights_fp8(gate_up, down)
    del gate_up, down
    ws = B300MoEWorkspace(capacity_tokens=T, device=cuda_device)
    out, meta = b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K,
                                     workspace=ws, return_metadata=True, check_status=True)
    again = b300_moe_forward_fp8(hidden, ids, weights, fw, num_experts=E, top_k=K, workspace=ws)
    assert torch.equal(out, again)
    doubled = b300_moe_forward_fp8(hidden, ids, weights * 2, fw, num_experts=E, top_k=K,
                                   workspace=ws)
    assert torch.equal(doubled.float(), out.float() * 2)
    want = moe_oracle.group_tokens(ids.cpu(), E)
    for key in ("permutation", "reverse_mapping", "expert_counts", "expert_offsets"):
        np.testing.assert_array_equal(meta[key].cpu().numpy(), getattr(want, key), err_msg=key)

    tokens = [0, T // 2, T - 1]
    picked = ids[tokens].cpu()
    experts = sorted(set(picked.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(experts)}
    small_ids = torch.tensor([[remap[int(e)] for e in row] for row in picked])
    index = torch.tensor(experts, device=cuda_device)
    gate_up_ref = fp8_oracle.dequantize_rows(
        fw.gate_up_q.index_select(0, index).cpu().numpy(),
        fw.gate_up_scale.index_select(0, index).cpu().numpy())
    down_ref = fp8_oracle.dequantize_rows(
        fw.down_q.index_select(0, index).cpu().numpy(),
        fw.down_scale.index_select(0, index).cpu().numpy())
    ref = moe_oracle.routed_moe_naive(hidden[tokens].cpu(), small_ids, weights[tokens].cpu(),
                                      gate_up_ref, down_ref)
    got = out[tokens].float().cpu()
    err = float((got - ref).abs().max()) / moe_oracle.rms(ref)
    print(f"fp8 deepseek-shaped full size: err/rms={err:.5f} floor={moe_oracle.bf16_floor(ref):.5f}")
    assert err <= TOLERANCE


def test_one_workspace_serves_bf16_and_fp8_calls_alternately(cuda_device) -> None:
    """The two weight formats share a workspace layout; switching between them per call must
    neither reallocate nor leak state from one call into the next, with and without PDL."""

    from b200moe import (B300MoEWorkspace, b300_moe_forward, b300_moe_forward_fp8,
                         quantize_expert_weights_fp8)

    E, H, I, K, T = 8, 256, 384, 2, 10
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, seed=9)
    gate_up, down = gate_up.to(cuda_device), down.to(cuda_device)
    fw = quantize_expert_weights_fp8(gate_up, down)
    dev = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device))
    want_bf16 = b300_moe_forward(*dev, gate_up, down, num_experts=E, top_k=K)
    want_fp8 = b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=K)
    ws = B300MoEWorkspace(device=cuda_device)
    for use_pdl in (True, False, True):
        got_fp8 = b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=K, workspace=ws,
                                       use_pdl=use_pdl, check_status=True)
        got_bf16 = b300_moe_forward(*dev, gate_up, down, num_experts=E, top_k=K, workspace=ws,
                                    use_pdl=use_pdl, check_status=True)
        assert torch.equal(got_fp8, want_fp8)
        assert torch.equal(got_bf16, want_bf16)
    assert ws.allocation_count == 1


def test_pinned_host_io_with_fp8_weights(cuda_device) -> None:
    """Per-step tensors in pinned host memory, read and written by the kernels directly,
    with FP8 expert weights: same bits as the device-resident call."""

    from b200moe import (B300MoEWorkspace, b300_moe_forward_fp8, b300_moe_forward_pinned,
                         quantize_expert_weights_fp8)

    E, H, I, K, T = 8, 256, 384, 2, 7
    gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, seed=11)
    fw = quantize_expert_weights_fp8(gate_up.to(cuda_device), down.to(cuda_device))
    want = b300_moe_forward_fp8(hidden.to(cuda_device), ids.to(cuda_device),
                                weights.to(cuda_device), fw, num_experts=E, top_k=K)
    host = tuple(t.pin_memory() for t in (hidden, ids, weights))
    ws = B300MoEWorkspace(device=cuda_device)
    got = b300_moe_forward_pinned(*host, None, None, num_experts=E, top_k=K, workspace=ws,
                                  fp8_weights=fw)
    torch.cuda.synchronize(cuda_device)
    assert got.is_pinned() and got.device.type == "cpu"
    assert torch.equal(got, want.cpu())
    assert ws.status() == 0


def test_seeded_random_shapes_both_weight_formats(cuda_device) -> None:
    """Twenty-four seeded random geometries (ragged H and I, every top_k, all routing patterns,
    token counts up to 150 so that experts exceed one segment) through both weight formats:
    routing bit-exact, outputs within the bar of their FP32 oracles."""

    import random

    from b200moe import (B300MoEWorkspace, b300_moe_forward, b300_moe_forward_fp8,
                         quantize_expert_weights_fp8)

    rng = random.Random(20240607)
    patterns = ("uniform", "zipf", "concentrated", "empty_half", "duplicates")
    for trial in range(24):
        E = rng.choice((1, 2, 3, 8, 17, 64))
        K = rng.choice([k for k in (1, 2, 4, 8) if k <= E])
        H = 16 * rng.randint(1, 24)
        I = 16 * rng.randint(1, 24)
        T = rng.choice((1, 2, 3, 7, 16, 33, 64, 150))
        routing = rng.choice(patterns)
        if routing == "empty_half" and E < 2 * K:
            routing = "uniform"
        gate_up, down, hidden, ids, weights = _case(E, H, I, K, T, routing, seed=100 + trial)
        dev = (hidden.to(cuda_device), ids.to(cuda_device), weights.to(cuda_device))
        gate_up_d, down_d = gate_up.to(cuda_device), down.to(cuda_device)
        label = f"trial {trial}: E{E} K{K} H{H} I{I} T{T} {routing}"

        ws = B300MoEWorkspace(device=cuda_device)
        out, meta = b300_moe_forward(*dev, gate_up_d, down_d, num_experts=E, top_k=K,
                                     workspace=ws, return_metadata=True, check_status=True)
        ref, routing_ref = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down,
                                                 num_experts=E, top_k=K)
        for key in ("permutation", "reverse_mapping", "expert_counts", "expert_offsets"):
            np.testing.assert_array_equal(meta[key].cpu().numpy(), getattr(routing_ref, key),
                                          err_msg=f"{label} {key}")
        _check(out, ref, label + " bf16")

        fw = quantize_expert_weights_fp8(gate_up_d, down_d)
        out8, meta8 = b300_moe_forward_fp8(*dev, fw, num_experts=E, top_k=K, workspace=ws,
                                           return_metadata=True, check_status=True)
        ref8, _ = _reference(fw, hidden, ids, weights, E, K)
        np.testing.assert_array_equal(meta8["permutation"].cpu().numpy(), routing_ref.permutation,
                                      err_msg=label)
        _check(out8, ref8, label + " fp8")
