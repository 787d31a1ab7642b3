"""The FP8 (E4M3) oracle against an independent implementation of the number format.

The reference has no quantised path, so there are no reference vectors for these functions;
the format restatement in ``oracle/fp8_oracle.py`` is pinned against PyTorch's
``torch.float8_e4m3fn`` conversion (a third implementation of the same published format),
and the library-specific rules (per-row scale, three-plane split) are checked through
their defining properties.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import fp8_oracle


def test_table_matches_torch_float8() -> None:
    mine = fp8_oracle.e4m3_table()
    theirs = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(mine), np.isnan(theirs))
    finite = ~np.isnan(mine)
    np.testing.assert_array_equal(mine[finite], theirs[finite])
    assert mine[0x7E] == 448.0 and mine[0x01] == 2.0 ** -9 and mine[0x08] == 2.0 ** -6


def test_quantise_matches_torch_float8_including_ties() -> None:
    g = torch.Generator().manual_seed(11)
    table = fp8_oracle.e4m3_table()[:0x7F].astype(np.float64)
    midpoints = torch.tensor(((table[:-1] + table[1:]) / 2).astype(np.float32))
    x = torch.cat([
        (torch.randn(100_000, generator=g) * 100).clamp(-448, 448),
        torch.randn(100_000, generator=g) * 0.01,
        torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10]),
        midpoints, -midpoints,
    ])
    mine = fp8_oracle.quantize_e4m3(x.numpy())
    theirs = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(mine, theirs)


def test_quantise_saturates_instead_of_nan() -> None:
    codes = fp8_oracle.quantize_e4m3(np.array([449.0, 1e6, -1e6, np.inf, -np.inf], np.float32))
    np.testing.assert_array_equal(codes, [0x7E, 0x7E, 0xFE, 0x7E, 0xFE])


def test_round_trip_of_every_code_is_exact() -> None:
    table = fp8_oracle.e4m3_table()
    finite = ~np.isnan(table)
    codes = np.arange(256, dtype=np.uint8)[finite]
    again = fp8_oracle.quantize_e4m3(table[finite])
    # +0 and -0 keep their sign bit
    np.testing.assert_array_equal(again, codes)


def test_quantise_rows_scale_rule_and_error_bound() -> None:
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(2, 6, 64, generator=g) * 0.02).to(torch.bfloat16)
    w[0, 1] = 0
    w[1, 2, 5] = 1.5
    q, scale = fp8_oracle.quantize_rows(w)
    assert q.shape == (2, 6, 64) and q.dtype == np.uint8 and scale.shape == (2, 6)
    amax = w.float().abs().amax(dim=-1).numpy()
    np.testing.assert_array_equal(scale[amax > 0], (amax[amax > 0] / np.float32(448.0)))
    assert scale[0, 1] == 1.0 and not q[0, 1].any()
    deq = fp8_oracle.dequantize_rows(q, scale).numpy()
    # the row maximum is reproduced exactly; every element within half an E4M3 step (2^-4
    # relative) of its value or half a subnormal step of the row scale
    err = np.abs(deq - w.float().numpy())
    bound = np.maximum(np.abs(w.float().numpy()) * 2.0 ** -4, scale[..., None] * 2.0 ** -10)
    assert (err <= bound * 1.0001).all()
    assert np.allclose(np.abs(deq).max(axis=-1)[amax > 0], amax[amax > 0], rtol=1e-6)


def test_three_plane_split_reconstructs_to_twelve_bits() -> None:
    g = torch.Generator().manual_seed(4)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).float().numpy()
    x[3] = 0.0
    x[5, 7] = 40.0  # an outlier sets the row scale
    codes, scale = fp8_oracle.split_planes(x)
    assert codes.shape == (3, 8, 512) and scale.shape == (8,)
    assert scale[3] == 1.0 and not codes[:, 3].any()
    back = fp8_oracle.join_planes(codes, scale)
    amax = np.abs(x).max(axis=-1, keepdims=True)
    err = np.abs(back - x)
    # relative 2^-12 for values in the normal range of the planes, else an absolute floor
    # far below one BF16 step of the row maximum
    bound = np.maximum(np.abs(x) * 2.0 ** -11, amax * 2.0 ** -20)
    assert (err <= bound).all(), float((err / np.maximum(bound, 1e-30)).max())
    # no plane ever needs the NaN code or saturation after the first
    assert not ((codes & 0x7F) == 0x7F).any()


def test_two_plane_split_of_bf16_rows_is_exact() -> None:
    g = torch.Generator().manual_seed(6)
    x = torch.randn(16, 1024, generator=g).to(torch.bfloat16)
    x[2] = 0.0
    x[4, 9] = 300.0
    x[5] *= 1e-3
    x[6, :8] = torch.tensor([1.0, -1.0, 0.5, 255.0, 1.0078125, 3.984375, 2.0 ** -7, -(2.0 ** -9)])
    codes, scale = fp8_oracle.split_planes_pow2(x.float().numpy())
    assert codes.shape == (2, 16, 1024)
    mantissa, _ = np.frexp(scale)
    assert (mantissa == 0.5).all()                      # powers of two
    amax = x.float().abs().amax(dim=-1).numpy()
    ratio = amax[amax > 0] / scale[amax > 0]
    assert (ratio >= 128).all() and (ratio < 256).all()
    planes = fp8_oracle.dequantize_e4m3(codes).astype(np.float64)
    back = (planes[0] + planes[1] / 16.0) * scale.astype(np.float64)[:, None]
    want = x.float().numpy().astype(np.float64)
    err = np.abs(back - want)
    # exact wherever the value is not vanishingly small against its row's maximum
    big = np.abs(want) >= amax[:, None] * 2.0 ** -12
    assert (err[big] == 0).all()
    # below that the second plane runs into its subnormal step: 2^-14 of a scaled maximum >= 2^7
    assert (err <= amax[:, None] * 2.0 ** -21 + 1e-30).all()
