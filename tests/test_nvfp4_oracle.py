"""The NVFP4 format oracle, pinned by enumeration (CPU).

E2M1 has sixteen codes, so the element half of the format is checked exhaustively: every code's
value, every midpoint between neighbouring magnitudes (round to nearest, ties to the even
mantissa bit), saturation, signs, and nibble packing.  The block-scale half is the E4M3 oracle
already pinned to ``torch.float8_e4m3fn``.  The weight rule and the token-plane rule are
checked through their defining properties.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import fp8_oracle, nvfp4_oracle as nv


def test_every_e2m1_code_has_its_published_value() -> None:
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    table = nv.e2m1_table()
    assert table[:8].tolist() == want and table[8:].tolist() == [-v for v in want]
    # sign, two exponent bits (bias 1), one mantissa bit; exponent field 0 is subnormal
    for code in range(8):
        exponent, mantissa = code >> 1, code & 1
        value = mantissa * 0.5 if exponent == 0 else (1 + mantissa * 0.5) * 2.0 ** (exponent - 1)
        assert table[code] == value


def test_rounding_is_nearest_with_ties_to_the_even_mantissa() -> None:
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i in range(7):
        lo, hi = grid[i], grid[i + 1]
        mid = (lo + hi) / 2
        even = lo if i % 2 == 0 else hi          # the code with mantissa bit 0
        below, above = np.nextafter(np.float32(mid), np.float32(-1)), np.nextafter(np.float32(mid), np.float32(10))
        got = nv.dequantize_e2m1(nv.quantize_e2m1(np.array([below, mid, above, -mid], np.float32)))
        assert got.tolist() == [lo, even, hi, -even]
    big = nv.dequantize_e2m1(nv.quantize_e2m1(np.array([6.0, 7.5, 1e9, -1e9, np.inf], np.float32)))
    assert big.tolist() == [6.0, 6.0, 6.0, -6.0, 6.0]
    assert nv.quantize_e2m1(np.array([-0.0, -0.1], np.float32)).tolist() == [8, 8]


def test_nibble_packing_puts_the_even_element_low() -> None:
    codes = np.arange(16, dtype=np.uint8)
    packed = nv.pack_nibbles(codes)
    assert packed.tolist() == [(2 * j) | ((2 * j + 1) << 4) for j in range(8)]
    assert np.array_equal(nv.unpack_nibbles(packed), codes)
    if hasattr(torch, "float4_e2m1fn_x2"):
        # PyTorch's packed FP4 storage type holds the same bytes (no arithmetic is defined on it)
        as_torch = torch.from_numpy(packed.copy()).view(torch.float4_e2m1fn_x2)
        assert as_torch.view(torch.uint8).tolist() == packed.tolist()


def test_weight_quantisation_follows_its_rule_and_bounds_its_error() -> None:
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(3, 40, 128, generator=g) * 0.02).bfloat16()
    w[1, 3] = 0                      # an all-zero row: zero scales, zero elements
    w[2] *= 37.0                     # another expert on another scale
    packed, sf, tensor_scale = nv.quantize_weights(w)
    assert packed.shape == (3, 40, 64) and sf.shape == (3, 40, 8) and tensor_scale.shape == (3,)
    wf = w.float().numpy()
    for e in range(3):
        assert tensor_scale[e] == np.float32(np.abs(wf[e]).max()) / np.float32(6 * 448)
    assert not sf[1, 3].any() and not packed[1, 3].any()
    deq = nv.dequantize_weights(packed, sf, tensor_scale).numpy()
    # within a block every element is within half a step of the block's grid: step <= block max / 3
    blocks = wf.reshape(3, 40, 8, 16)
    err = np.abs(deq.reshape(3, 40, 8, 16) - blocks)
    bound = np.abs(blocks).max(-1, keepdims=True) * (1 / 6 + 0.07) + 1e-12
    assert (err <= bound).all()
    # the block maximum itself is reproduced to E4M3 precision of its scale (1/16 relative)
    top = np.abs(blocks).max(-1)
    top_deq = np.abs(deq.reshape(3, 40, 8, 16)).max(-1)
    assert np.allclose(top_deq, top, rtol=0.0701, atol=1e-12)


def test_scale_tiles_have_the_tensor_core_byte_order() -> None:
    rows, nsf = 200, 6                # two row tiles (the second partial), two K tiles
    sf = (np.arange(rows * nsf) % 251).astype(np.uint8).reshape(rows, nsf)
    tiles = nv.swizzle_block_scales(sf)
    assert tiles.shape == (2, 2, 512)
    for r in (0, 1, 31, 32, 33, 127, 128, 199):
        for s in range(nsf):
            tile = tiles[r // 128, s // 4]
            rr = r % 128
            assert tile[(rr % 32) * 16 + (rr // 32) * 4 + s % 4] == sf[r, s]
    assert not tiles[1, :, :].reshape(2, 32, 4, 4)[:, :, 3, :].any()   # rows 224..255 do not exist
    assert not tiles[:, 1].reshape(2, 32, 4, 4)[..., 2:].any()         # scales 6, 7 do not exist


@pytest.mark.parametrize("planes", [1, 2, 3, 4])
def test_token_planes_remove_three_bits_each(planes: int) -> None:
    g = torch.Generator().manual_seed(9)
    x = torch.randn(6, 512, generator=g).bfloat16().float().numpy()
    x[2] *= 1e-3
    x[3] = 0
    x[4, 7] = 3.999 * np.abs(x[4]).max()          # a row maximum just under the top of its octave
    codes, t = nv.split_planes(x, planes)
    assert codes.shape == (planes, 6, 512) and codes.dtype == np.uint8 and int(codes.max()) < 16
    rebuilt = nv.join_planes(codes, t)
    # |x - rebuilt| <= t * 8**-(planes-1) / 2 for every element, i.e. max|row| * 2**-(3*planes-1)
    bound = t.astype(np.float64) * 8.0 ** -(planes - 1) / 2
    assert (np.abs(rebuilt - x) <= bound[:, None]).all()
    assert not rebuilt[3].any() and t[3] == 1.0
    # the row scale is the power of two that puts the row maximum into [2, 4): no element
    # reaches the part of the E2M1 grid that is 2 apart
    for r in (0, 1, 2, 4, 5):
        assert 2 <= np.abs(x[r]).max() / t[r] < 4 and np.log2(t[r]) == int(np.log2(t[r]))
    assert int((codes[0] & 7).max()) <= 6          # magnitude 6 is never needed in plane 0
    if planes == 4:
        rms = np.sqrt((x.astype(np.float64) ** 2).mean(1))
        err = np.sqrt(((rebuilt - x) ** 2).mean(1))
        # Gaussian rows: 1e-4 of the row's RMS, a twentieth of what BF16 rounding costs
        assert (err[[0, 1, 5]] / rms[[0, 1, 5]] <= 2e-4).all()
