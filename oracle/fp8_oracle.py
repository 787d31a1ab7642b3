"""CPU oracle for the FP8 (E4M3) expert-weight format.  TEST INFRASTRUCTURE.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this
file; the library never does.

The reference has no quantised path to restate: its NVFP4 backend always raises
(fastpath/b300_moe.py:571-596, csrc/quantization_kernels.cu:7-13) and FP8/NVFP4 weights are
listed as future work (docs/goal_1b_report.md:313-314).  What is restated here is the
published OCP 8-bit floating point format "E4M3" (1 sign, 4 exponent bits with bias 7,
3 mantissa bits, no infinities, one NaN mantissa pattern per sign, maximum 448) and this
library's own per-row scaling rule.  **Parity unpinned against the reference** (there is
nothing to pin to); the number format itself is pinned against PyTorch's independent
``torch.float8_e4m3fn`` conversion in ``tests/test_fp8_oracle.py``.

Layer semantics with FP8 weights = the FP32 oracle (``moe_oracle.routed_moe``) run on the
dequantised weights ``E4M3 value * row scale``; the same 2e-2 x RMS bar applies.
"""

from __future__ import annotations

import numpy as np
import torch

E4M3_MAX = 448.0


def e4m3_table() -> np.ndarray:
    """Value of each of the 256 byte codes (float32; codes 0x7F and 0xFF are NaN)."""

    codes = np.arange(256, dtype=np.int64)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exponent = (codes >> 3) & 0xF
    mantissa = codes & 0x7
    normal = (1.0 + mantissa / 8.0) * np.exp2(exponent.astype(np.float64) - 7.0)
    subnormal = (mantissa / 8.0) * 2.0 ** -6
    value = sign * np.where(exponent == 0, subnormal, normal)
    value[(codes & 0x7F) == 0x7F] = np.nan
    return value.astype(np.float32)


_POSITIVE = e4m3_table()[:0x7F].astype(np.float64)  # codes 0x00..0x7E, increasing


def quantize_e4m3(x) -> np.ndarray:
    """float32 array -> E4M3 byte codes: round to nearest, ties to the even code,
    magnitudes above 448 saturate to 448 (no NaN is ever produced for finite input)."""

    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    hi = np.searchsorted(_POSITIVE, mag, side="left")      # first code with value >= mag
    hi = np.clip(hi, 0, len(_POSITIVE) - 1)
    lo = np.clip(hi - 1, 0, len(_POSITIVE) - 1)
    d_lo = np.abs(mag - _POSITIVE[lo])
    d_hi = np.abs(_POSITIVE[hi] - mag)
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((hi & 1) == 0))
    code = np.where(pick_hi, hi, lo)
    code = np.where(mag >= E4M3_MAX, 0x7E, code)
    code = np.where(np.isnan(x), 0x7F, code)
    sign = np.signbit(x).astype(np.int64) << 7
    return (code | sign).astype(np.uint8)


def dequantize_e4m3(codes) -> np.ndarray:
    return e4m3_table()[np.asarray(codes, dtype=np.uint8)]


def quantize_rows(weights: torch.Tensor) -> tuple[np.ndarray, np.ndarray]:
    """Per-row scaling rule of ``b200moe_fp8_quantize_rows``.

    ``weights`` [..., rows, cols] (any float dtype; BF16 in practice): for every row
    ``scale = max|w| / 448`` in float32 (1 for an all-zero row) and
    ``q = E4M3(float32(w) / scale)`` with float32 division.  Returns ``(q uint8, scale
    float32)`` with shapes ``[..., rows, cols]`` and ``[..., rows]``.
    """

    w = weights.detach().to(torch.float32).cpu().numpy()
    amax = np.max(np.abs(w), axis=-1)
    scale = np.where(amax > 0, (amax / np.float32(E4M3_MAX)).astype(np.float32), np.float32(1.0))
    scale = scale.astype(np.float32)
    q = quantize_e4m3((w / scale[..., None]).astype(np.float32))
    return q, scale


def dequantize_rows(q, scale) -> torch.Tensor:
    """FP32 weights ``E4M3 value * scale`` (what the FP8 kernels compute with)."""

    values = dequantize_e4m3(q).astype(np.float32) * np.asarray(scale, np.float32)[..., None]
    return torch.from_numpy(values)


def split_planes(rows) -> tuple[np.ndarray, np.ndarray]:
    """Token rows as three E4M3 planes and one scale per row (float32 arithmetic throughout).

    Restates this library's own rule for the token operand of the FP8-weight GEMMs:
    ``s = max|row| / 448`` (1 for an all-zero row), ``r = x / s``, then
    ``p0 = e4m3(r)``, ``p1 = e4m3((r - p0) * 16)``, ``p2 = e4m3(((r - p0) * 16 - p1) * 16)``
    so that ``x ~= s * (p0 + p1 / 16 + p2 / 256)``.  Returns ``(codes uint8 [3, R, C],
    scale float32 [R])``.
    """

    x = np.asarray(rows, dtype=np.float32)
    amax = np.max(np.abs(x), axis=-1)
    scale = np.where(amax > 0, (amax / np.float32(E4M3_MAX)).astype(np.float32), np.float32(1.0))
    scale = scale.astype(np.float32)
    r0 = (x / scale[:, None]).astype(np.float32)
    c0 = quantize_e4m3(r0)
    r1 = ((r0 - dequantize_e4m3(c0)) * np.float32(16.0)).astype(np.float32)
    c1 = quantize_e4m3(r1)
    r2 = ((r1 - dequantize_e4m3(c1)) * np.float32(16.0)).astype(np.float32)
    c2 = quantize_e4m3(r2)
    return np.stack([c0, c1, c2]), scale


def join_planes(codes, scale) -> np.ndarray:
    """Inverse of :func:`split_planes` in float64: ``s * (p0 + p1/16 + p2/256)``."""

    p = dequantize_e4m3(codes).astype(np.float64)
    return (p[0] + p[1] / 16.0 + p[2] / 256.0) * np.asarray(scale, np.float64)[:, None]


def split_planes_pow2(rows) -> tuple[np.ndarray, np.ndarray]:
    """BF16-valued rows as two E4M3 planes and a power-of-two scale per row.

    This library's rule for the hidden rows of the FP8-weight gate+up GEMM: ``s`` is the power
    of two with ``max|row| / s`` in ``[128, 256)`` (1 for an all-zero row), so ``r = x / s`` is
    exact; ``p0 = e4m3(r)``, ``p1 = e4m3((r - p0) * 16)``.  A BF16 value has eight significant
    bits and each plane holds four, so ``s * (p0 + p1 / 16)`` reproduces it exactly, down to
    values below 2^-12 of the row maximum, whose error stays under 2^-21 of it.  Returns ``(codes uint8 [2, R, C], scale float32 [R])``.
    """

    x = np.asarray(rows, dtype=np.float32)
    amax = np.max(np.abs(x), axis=-1)
    _, exponent = np.frexp(amax)          # amax = f * 2**exponent, f in [0.5, 1)
    scale = np.where(amax > 0, np.ldexp(np.float32(1.0), exponent - 8), np.float32(1.0))
    scale = scale.astype(np.float32)
    r0 = (x / scale[:, None]).astype(np.float32)
    c0 = quantize_e4m3(r0)
    r1 = ((r0 - dequantize_e4m3(c0)) * np.float32(16.0)).astype(np.float32)
    c1 = quantize_e4m3(r1)
    return np.stack([c0, c1]), scale
