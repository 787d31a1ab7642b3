"""CPU oracle for the NVFP4 expert-weight format.  TEST INFRASTRUCTURE.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this
file; the library never does.

The reference has no NVFP4 arithmetic to restate: its ``cutlass_nvfp4`` backend always
raises (fastpath/b300_moe.py:571-596) and csrc/quantization_kernels.cu:3-6 only says what a
real implementation must have -- a 4-bit E2M1 payload and two levels of scales.  What is
restated here is the published format:

* element: E2M1, 1 sign bit, 2 exponent bits (bias 1), 1 mantissa bit; the eight magnitudes
  are 0, 0.5, 1, 1.5, 2, 3, 4, 6; no infinities, no NaN; two elements per byte, the element
  with the even index in the low four bits;
* first scale level: one unsigned E4M3 value (the OCP 8-bit format of ``fp8_oracle``, sign bit
  never set) per block of 16 consecutive elements along the reduction dimension;
* second scale level: one float32 per tensor (here: per expert matrix).

``value = float32_scale * e4m3_block_scale * e2m1_element``.  **Parity unpinned against the
reference** (there is nothing to pin to).  The E4M3 half is pinned to ``torch.float8_e4m3fn``
by ``tests/test_fp8_oracle.py``; the E2M1 half is small enough to be pinned by enumeration
(``tests/test_nvfp4_oracle.py``: all 16 codes, every midpoint, saturation) and against
``torch.float4_e2m1fn_x2`` storage where this PyTorch can view it.

Layer semantics with NVFP4 weights = the FP32 oracle (``moe_oracle.routed_moe``) run on the
dequantised weights; the same 2e-2 x RMS bar applies.

The token operand of the block-scaled tensor-core instruction must be E2M1 as well, so the
kernels hold each token row as several E2M1 *planes* in fixed point (``split_planes``):
plane p rounds what planes 0..p-1 left over, in a unit eight times finer than the one before.
"""

from __future__ import annotations

import numpy as np
import torch

from . import fp8_oracle

BLOCK = 16                                  # elements per block scale
E2M1_MAX = 6.0
E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e2m1_table() -> np.ndarray:
    """Value of each of the 16 codes: bit 3 is the sign, bits 0..2 index the magnitudes."""

    return np.concatenate([E2M1_MAGNITUDES, -E2M1_MAGNITUDES]).astype(np.float32)


def quantize_e2m1(x) -> np.ndarray:
    """float32 array -> E2M1 codes (uint8, one per element): round to nearest, ties to the
    code with an even mantissa bit (even index), magnitudes above 6 saturate to 6."""

    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    grid = E2M1_MAGNITUDES.astype(np.float64)
    hi = np.clip(np.searchsorted(grid, mag, side="left"), 0, 7)
    lo = np.clip(hi - 1, 0, 7)
    d_lo = np.abs(mag - grid[lo])
    d_hi = np.abs(grid[hi] - mag)
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((hi & 1) == 0))
    code = np.where(pick_hi, hi, lo)
    code = np.where(mag >= E2M1_MAX, 7, code)
    sign = np.signbit(x).astype(np.int64) << 3
    return (code | sign).astype(np.uint8)


def _quantize_e2m1_f64(x) -> np.ndarray:
    """:func:`quantize_e2m1` on float64 input (no rounding to float32 first)."""

    x = np.asarray(x, dtype=np.float64)
    mag = np.abs(x)
    grid = E2M1_MAGNITUDES.astype(np.float64)
    hi = np.clip(np.searchsorted(grid, mag, side="left"), 0, 7)
    lo = np.clip(hi - 1, 0, 7)
    d_lo = np.abs(mag - grid[lo])
    d_hi = np.abs(grid[hi] - mag)
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((hi & 1) == 0))
    code = np.where(pick_hi, hi, lo)
    code = np.where(mag >= E2M1_MAX, 7, code)
    return (code | (np.signbit(x).astype(np.int64) << 3)).astype(np.uint8)


def dequantize_e2m1(codes) -> np.ndarray:
    return e2m1_table()[np.asarray(codes, dtype=np.uint8) & 0xF]


def pack_nibbles(codes) -> np.ndarray:
    """[..., C] codes -> [..., C/2] bytes, even element in the low nibble."""

    c = np.asarray(codes, dtype=np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out


def quantize_weights(weights: torch.Tensor) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """``[E, rows, cols]`` weights -> ``(packed uint8 [E, rows, cols/2], block_scale uint8
    [E, rows, cols/16], tensor_scale float32 [E])``.

    Rule of ``b200moe_nvfp4_quantize``: per expert matrix ``g = max|w| / (6 * 448)`` (1 when
    the matrix is all zero); per block ``s = e4m3(max|block| / 6 / g)`` rounded to nearest
    even; element ``q = e2m1(w / (g * value(s)))`` rounded to nearest even and saturated;
    a block whose scale code is 0 stores zeros.  All arithmetic in float32.
    """

    w = weights.detach().to(torch.float32).cpu().numpy()
    experts, rows, cols = w.shape
    if cols % BLOCK:
        raise ValueError("the reduction dimension must be a multiple of 16")
    amax = np.max(np.abs(w).reshape(experts, -1), axis=1)
    g = np.where(amax > 0, (amax / np.float32(E2M1_MAX * fp8_oracle.E4M3_MAX)).astype(np.float32),
                 np.float32(1.0)).astype(np.float32)
    blocks = w.reshape(experts, rows, cols // BLOCK, BLOCK)
    block_amax = np.max(np.abs(blocks), axis=-1)
    target = (block_amax / np.float32(E2M1_MAX)).astype(np.float32) / g[:, None, None]
    sf = fp8_oracle.quantize_e4m3(target.astype(np.float32))
    sf_value = fp8_oracle.dequantize_e4m3(sf).astype(np.float32)
    denom = (g[:, None, None] * sf_value).astype(np.float32)
    safe = np.where(denom > 0, denom, np.float32(1.0))
    ratio = (blocks / safe[..., None]).astype(np.float32)
    codes = quantize_e2m1(ratio)
    codes = np.where(denom[..., None] > 0, codes, 0).astype(np.uint8)
    return pack_nibbles(codes.reshape(experts, rows, cols)), sf, g


def dequantize_weights(packed, block_scale, tensor_scale) -> torch.Tensor:
    """FP32 weights ``g * e4m3(s) * e2m1(q)`` (what the NVFP4 kernels multiply by)."""

    codes = unpack_nibbles(packed)
    values = dequantize_e2m1(codes).astype(np.float32)
    sf = fp8_oracle.dequantize_e4m3(block_scale).astype(np.float32)
    experts, rows, cols = values.shape
    scaled = values.reshape(experts, rows, cols // BLOCK, BLOCK) * sf[..., None]
    scaled = scaled.reshape(experts, rows, cols) * np.asarray(tensor_scale, np.float32)[:, None, None]
    return torch.from_numpy(scaled.astype(np.float32))


def swizzle_block_scales(block_scale) -> np.ndarray:
    """``[..., rows, cols/16]`` scale codes -> the byte order the tensor core's scale-factor
    copy expects: tiles of 128 rows x 4 scales (64 elements of the reduction dimension), 512
    bytes each, byte ``(r % 32) * 16 + (r // 32) * 4 + k`` for row ``r`` and scale ``k`` of
    the tile; tiles ordered row tile first, then along the reduction dimension.  Rows and
    scales beyond the matrix are zero.  Returns ``[..., row_tiles, k_tiles, 512]`` uint8."""

    sf = np.asarray(block_scale, dtype=np.uint8)
    rows, nsf = sf.shape[-2:]
    row_tiles, k_tiles = (rows + 127) // 128, (nsf + 3) // 4
    padded = np.zeros(sf.shape[:-2] + (row_tiles * 128, k_tiles * 4), dtype=np.uint8)
    padded[..., :rows, :nsf] = sf
    tiles = padded.reshape(sf.shape[:-2] + (row_tiles, 4, 32, k_tiles, 4))
    # axes: row_tile, r // 32, r % 32, k_tile, k  ->  row_tile, k_tile, r % 32, r // 32, k
    lead = len(sf.shape) - 2
    order = tuple(range(lead)) + (lead, lead + 3, lead + 2, lead + 1, lead + 4)
    return np.ascontiguousarray(tiles.transpose(order)).reshape(
        sf.shape[:-2] + (row_tiles, k_tiles, 512))


PLANE_STEP = 0.125   # every plane's unit is an eighth of the one before


def row_scale_pow2(rows) -> np.ndarray:
    """Per-row float32 scale of the token planes: the power of two ``t`` with
    ``max|row| / t`` in ``[2, 4)`` (1 for an all-zero row, never below 2**-100)."""

    x = np.asarray(rows, dtype=np.float32)
    amax = np.max(np.abs(x), axis=-1)
    _, exponent = np.frexp(amax)
    exponent = np.maximum(exponent - 2, -100)
    return np.where(amax > 0, np.ldexp(np.float32(1.0), exponent), np.float32(1.0)).astype(np.float32)


def split_planes(rows, planes: int) -> tuple[np.ndarray, np.ndarray]:
    """Token rows ``[R, C]`` as ``planes`` E2M1 planes in fixed point.

    ``t = row_scale_pow2(rows)``; the residual starts as ``x``; plane ``p`` is
    ``q_p = e2m1(residual / (t * 8**-p))`` (nearest, ties to the even mantissa bit) and
    ``residual -= t * 8**-p * q_p``.  Every step is exact in float32: the units are powers of
    two and the residual is a multiple of a much smaller one.  ``|x| / t < 4`` lies where the
    E2M1 grid is at most 1 apart, so the first residual is at most ``t / 2 = 4 * t / 8`` and,
    in turn, every plane removes three bits: ``|x - t * sum_p 8**-p q_p| <= t * 8**-(planes-1) / 2``.
    Returns ``(codes uint8 [planes, R, C], t float32 [R])``.
    """

    x = np.asarray(rows, dtype=np.float32)
    t = row_scale_pow2(x)
    residual = x.copy()
    all_codes = []
    step = t[:, None].astype(np.float32)
    for _ in range(planes):
        # a power-of-two divisor: the float64 quotient is exact
        codes = _quantize_e2m1_f64(residual.astype(np.float64) / step.astype(np.float64)).astype(np.uint8)
        residual = (residual - dequantize_e2m1(codes) * step).astype(np.float32)
        all_codes.append(codes)
        step = (step * np.float32(PLANE_STEP)).astype(np.float32)
    return np.stack(all_codes), t


def join_planes(codes, t) -> np.ndarray:
    """Inverse of :func:`split_planes` in float64."""

    values = dequantize_e2m1(codes).astype(np.float64)
    weights = PLANE_STEP ** np.arange(values.shape[0], dtype=np.float64)
    return (values * weights[:, None, None]).sum(axis=0) * np.asarray(t, np.float64)[:, None]
