"""NVFP4 expert weights on the GPU: quantiser and token-plane rule bit-exact against the
format oracle, the layer against the FP32 oracle evaluated on the dequantised weights.

The reference has no NVFP4 arithmetic (its backend of that name always raises), so parity is
stated against this repository's format oracle (``oracle/nvfp4_oracle.py``, pinned by
enumeration) and the layer oracle; the bar is the BF16 path's: routing tensors bit-exact,
``max|y - y_ref| <= 2e-2 x rms(y_ref)``.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import moe_oracle, nvfp4_oracle as nv

pytestmark = pytest.mark.gpu
TOLERANCE = 2e-2
QUANTISATION_RMS_BOUND = 0.20   # NVFP4 layer against the unquantised layer, RMS over RMS


def _case(device, T, H, I, E, K, routing="uniform", weight_kind="softmax", seed=1234, std=None):
    from b200moe import workloads

    return workloads.make_case(T, H, I, E, K, routing=routing, weight_kind=weight_kind,
                               seed=seed, std=std, device=device)


def test_weight_quantiser_matches_the_oracle_bit_for_bit(cuda_device) -> None:
    from b200moe.nvfp4 import quantize_matrix_nvfp4

    g = torch.Generator().manual_seed(3)
    for experts, halves, rows, cols in [(3, 2, 200, 256), (2, 1, 128, 64), (1, 1, 72, 2880)]:
        w = (torch.randn(experts, halves * rows, cols, generator=g) * 0.02).bfloat16()
        w[0, 5] = 0
        if experts > 1:
            w[1] *= 11.0
        packed, sf, scale = quantize_matrix_nvfp4(w.to(cuda_device), halves)
        torch.cuda.synchronize(cuda_device)
        want_packed, want_sf, want_scale = nv.quantize_weights(w)
        assert np.array_equal(scale.cpu().numpy(), want_scale)
        assert np.array_equal(packed.cpu().numpy(), want_packed)
        # gate and up halves are tiled separately: [E][halves][row tiles][K tiles][512]
        tiles = nv.swizzle_block_scales(want_sf.reshape(experts, halves, rows, cols // 16))
        assert np.array_equal(sf.cpu().numpy(), tiles.reshape(experts, -1))


def test_token_plane_rule_matches_the_oracle_bit_for_bit(cuda_device) -> None:
    from b200moe.nvfp4 import rows_to_planes_nvfp4

    g = torch.Generator().manual_seed(4)
    rows = torch.randn(9, 2880, generator=g)
    rows[1] *= 1e-4
    rows[2] = 0
    rows[3, ::7] *= 300.0
    planes, t = rows_to_planes_nvfp4(rows.to(cuda_device))
    torch.cuda.synchronize(cuda_device)
    want_codes, want_t = nv.split_planes(rows.numpy(), 4)
    assert np.array_equal(t.cpu().numpy(), want_t)
    assert np.array_equal(planes.cpu().numpy(), nv.pack_nibbles(want_codes))


def _dequantised(fw):
    gate_up = nv.dequantize_weights(
        fw.gate_up_q.cpu().numpy(), _plain_scales(fw.gate_up_block_scale, fw.num_experts, 2,
                                                  fw.intermediate_size, fw.hidden_size),
        fw.gate_up_scale.cpu().numpy())
    down = nv.dequantize_weights(
        fw.down_q.cpu().numpy(), _plain_scales(fw.down_block_scale, fw.num_experts, 1,
                                               fw.hidden_size, fw.intermediate_size),
        fw.down_scale.cpu().numpy())
    return gate_up, down


def _plain_scales(tiled: torch.Tensor, experts: int, halves: int, rows: int, cols: int):
    """Undo the 512-byte tiling: -> [E, halves * rows, cols / 16] scale codes."""

    row_tiles, k_tiles = (rows + 127) // 128, (cols + 63) // 64
    t = tiled.cpu().numpy().reshape(experts, halves, row_tiles, k_tiles, 32, 4, 4)
    # tile byte (r % 32) * 16 + (r // 32) * 4 + k  ->  axes [.., r % 32, r // 32, k]
    plain = t.transpose(0, 1, 2, 5, 4, 3, 6).reshape(experts, halves, row_tiles * 128, k_tiles * 4)
    return np.ascontiguousarray(plain[:, :, :rows, : cols // 16]).reshape(
        experts, halves * rows, cols // 16)


SHAPES = [
    # T, H, I, E, K, routing, weight_kind
    (5, 256, 384, 8, 2, "uniform", "softmax"),
    (1, 512, 256, 4, 1, "uniform", "softmax"),
    (16, 2880, 2880, 8, 4, "concentrated", "softmax"),     # K not a multiple of 256: short last stage
    (64, 512, 768, 8, 8, "zipf", "raw"),                  # up to 64 rows per expert, +/- weights
    (150, 256, 320, 4, 2, "uniform", "softmax"),          # experts longer than one segment
    (33, 1024, 2048, 16, 2, "empty_half", "softmax"),
]


@pytest.mark.parametrize("spec", SHAPES, ids=lambda s: "T{}_H{}_I{}_E{}_K{}_{}".format(*s[:6]))
def test_layer_matches_fp32_oracle_on_dequantised_weights(spec, cuda_device) -> None:
    from b200moe import StagedLayer, b300_moe_forward_nvfp4, quantize_expert_weights_nvfp4

    T, H, I, E, K, routing, weight_kind = spec
    hidden, ids, weights, gate_up, down = _case(cuda_device, T, H, I, E, K, routing, weight_kind)
    fw = quantize_expert_weights_nvfp4(gate_up, down)
    out, meta = b300_moe_forward_nvfp4(hidden, ids, weights, fw, num_experts=E, top_k=K,
                                       return_metadata=True, check_status=True)
    torch.cuda.synchronize(cuda_device)
    gu_deq, dn_deq = _dequantised(fw)
    ref, routing_ref, mid = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gu_deq,
                                                  dn_deq, num_experts=E, top_k=K,
                                                  return_intermediates=True)
    for key in ("expert_counts", "expert_offsets", "permutation", "reverse_mapping"):
        assert np.array_equal(meta[key].cpu().numpy(), getattr(routing_ref, key)), key
    err = moe_oracle.relative_max_error(out.float().cpu(), ref)
    floor = moe_oracle.bf16_floor(ref)
    print(f"nvfp4 {spec}: err/rms={err:.5f} floor={floor:.5f}")
    assert meta["backend"] == "cutlass_nvfp4" and meta["quant_mode"] == "nvfp4"
    assert meta["used_fallback"] is False
    assert err <= TOLERANCE, (err, floor)
    # what the format itself costs against the unquantised layer: bounded, not only printed
    # (E2M1 keeps one mantissa bit under a 16-element block scale; measured 16-17 % of the output RMS)
    exact, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gate_up.cpu(),
                                     down.cpu(), num_experts=E, top_k=K)
    shift = float(((out.float().cpu() - exact) ** 2).mean().sqrt() / (exact ** 2).mean().sqrt())
    print(f"  nvfp4 quantisation: rms(out - unquantised) / rms = {shift:.4f}")
    assert shift <= QUANTISATION_RMS_BOUND, shift


def test_gate_up_stage_reproduces_the_oracle_activations(cuda_device) -> None:
    """The first GEMM on its own: hi + lo activations against the oracle's, row by row."""

    from b200moe import B300MoEWorkspace, StagedLayer, _lib, quantize_expert_weights_nvfp4

    T, H, I, E, K = 12, 512, 384, 4, 2
    hidden, ids, weights, gate_up, down = _case(cuda_device, T, H, I, E, K, seed=77)
    fw = quantize_expert_weights_nvfp4(gate_up, down)
    layer = StagedLayer(hidden, ids, weights, None, None, num_experts=E, top_k=K,
                        nvfp4_weights=fw, use_pdl=False)
    for stage in ("routing", "gather", "gate_up_swiglu"):
        layer.run_stage(stage)
    torch.cuda.synchronize(cuda_device)
    assert layer.workspace.status() == 0
    gu_deq, dn_deq = _dequantised(fw)
    _, _, mid = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gu_deq, dn_deq,
                                      num_experts=E, top_k=K, return_intermediates=True)
    rows = T * K
    hi = layer.workspace.buffers["swiglu_output"][:rows].float().cpu()
    want = mid["activations"]
    scale = float(want.abs().max())
    # hi alone is the BF16 rounding of the activation
    assert float((hi - want).abs().max()) <= scale * 2 ** -7, float((hi - want).abs().max()) / scale


def test_backend_name_of_the_reference_runs_nvfp4(cuda_device) -> None:
    """``b300_moe_forward(backend="cutlass_nvfp4")`` -- the name that always fails in the
    reference -- runs the NVFP4 kernels on the contract's BF16 weight tensors (quantised once,
    on first use) and never the BF16 kernels."""

    from b200moe import B300MoEWorkspace, b300_moe_forward, prepared_nvfp4_weights

    T, H, I, E, K = 7, 256, 320, 8, 2
    hidden, ids, weights, gate_up, down = _case(cuda_device, T, H, I, E, K)
    ws = B300MoEWorkspace(device=cuda_device)
    out, meta = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                                 backend="cutlass_nvfp4", quant_mode="nvfp4", workspace=ws,
                                 return_metadata=True, check_status=True)
    again = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                             backend="cutlass_nvfp4", workspace=ws)
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(out, again)
    assert meta["backend"] == "cutlass_nvfp4" and meta["quant_mode"] == "nvfp4"
    fw = prepared_nvfp4_weights(gate_up, down)
    assert fw is prepared_nvfp4_weights(gate_up, down)       # prepared once
    gu_deq, dn_deq = _dequantised(fw)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gu_deq, dn_deq,
                                   num_experts=E, top_k=K)
    assert moe_oracle.relative_max_error(out.float().cpu(), ref) <= TOLERANCE
    # and it differs from the BF16 layer by the quantisation, i.e. BF16 was not substituted
    bf16 = b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K)
    assert not torch.equal(out, bf16)
    with pytest.raises(ValueError, match="requires quant_mode='nvfp4'|cutlass_nvfp4 requires"):
        b300_moe_forward(hidden, ids, weights, gate_up, down, num_experts=E, top_k=K,
                         backend="cutlass_nvfp4", quant_mode="bf16")


def test_mixtral_shaped_decode_step_with_nvfp4_weights(cuda_device) -> None:
    """Full-size expert matrices (H=4096, I=14336), four experts to bound host memory."""

    from b200moe import b300_moe_forward_nvfp4, quantize_expert_weights_nvfp4

    T, H, I, E, K = 8, 4096, 14336, 4, 2
    hidden, ids, weights, gate_up, down = _case(cuda_device, T, H, I, E, K, std=0.02)
    fw = quantize_expert_weights_nvfp4(gate_up, down)
    del gate_up, down
    out = b300_moe_forward_nvfp4(hidden, ids, weights, fw, num_experts=E, top_k=K,
                                 check_status=True)
    again = b300_moe_forward_nvfp4(hidden, ids, weights, fw, num_experts=E, top_k=K)
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(out, again)
    gu_deq, dn_deq = _dequantised(fw)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gu_deq, dn_deq,
                                   num_experts=E, top_k=K)
    err = moe_oracle.relative_max_error(out.float().cpu(), ref)
    print(f"nvfp4 mixtral-shaped T=8: err/rms={err:.5f} floor={moe_oracle.bf16_floor(ref):.5f} "
          f"weight bytes {fw.nbytes / 1e6:.1f} MB")
    assert err <= TOLERANCE


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_shares_with_nvfp4_weights(world, cuda_device) -> None:
    """Each rank's share of an expert-parallel forward with NVFP4 weights, run one after
    another on one GPU: the FP32 partial outputs add up to the NVFP4 layer."""

    from b200moe import B300MoEWorkspace, quantize_expert_weights_nvfp4
    from b200moe.expert_parallel import expert_range, local_partial_forward

    T, H, I, E, K = 16, 256, 384, 8, 2
    hidden, ids, weights, gate_up, down = _case(cuda_device, T, H, I, E, K, routing="zipf", seed=7)
    fw = quantize_expert_weights_nvfp4(gate_up, down)
    total = torch.zeros(T, H, dtype=torch.float32, device=cuda_device)
    for rank in range(world):
        base, count = expert_range(rank, world, E)
        ws = B300MoEWorkspace(device=cuda_device)
        own = slice(base, base + count)
        partial, _ = local_partial_forward(
            hidden, ids, weights, fw.gate_up_q[own].contiguous(), fw.down_q[own].contiguous(),
            top_k=K, expert_id_base=base, num_experts_global=E, workspace=ws,
            nvfp4_scales=(fw.gate_up_scale[own].contiguous(), fw.down_scale[own].contiguous(),
                          fw.gate_up_block_scale[own].contiguous(),
                          fw.down_block_scale[own].contiguous()))
        torch.cuda.synchronize(cuda_device)
        assert ws.status() == 0
        total += partial
    gu_deq, dn_deq = _dequantised(fw)
    ref, _ = moe_oracle.routed_moe(hidden.cpu(), ids.cpu(), weights.cpu(), gu_deq, dn_deq,
                                   num_experts=E, top_k=K)
    err = moe_oracle.relative_max_error(total.cpu(), ref)
    print(f"nvfp4 expert-parallel shares, world {world}: err/rms={err:.5f}")
    assert err <= TOLERANCE
