"""CPU restatement of the per-token asymmetric INT8 quantizer (test infrastructure only).

Follows the reference kernel `_asymmetric_quant_kernel` (asymmetric_quant.py:32-106):

* row min / max over the head dimension, in fp32                (asymmetric_quant.py:72-81)
* scale = (max - min) / 255, a zero scale becomes 1             (asymmetric_quant.py:84-87)
* zp    = clamp(round(-128 - min / scale), -128, 127)           (asymmetric_quant.py:89-91)
* scale is STORED as fp16, zp as int8                           (asymmetric_quant.py:93-94)
* code  = clamp(round(x / scale + zp), -128, 127), with the
  fp32 (un-rounded) scale                                       (asymmetric_quant.py:103-106)

`round` is libdevice's round-half-away-from-zero.  The GPU kernels divide with
PTX `div.full.f32` (<= 2 ulp, not IEEE), this file divides with IEEE fp32.  The two
differ where x/scale+zp lands within an ulp or two of k+0.5 -- and with 8- or
11-bit-mantissa inputs EXACT .5 ties are common (the quotient of two short
mantissas), so on a B200 the reference's own Triton kernel disagrees with IEEE
division on about 0.4 % (bf16) / 0.15 % (fp16) of the codes, always by one code
(two when the zero-point also moved).  The tests therefore (a) allow that band
between this oracle and the GPU and (b) gate exact equality on fixtures written by
the reference kernel running on a B200 (tests/golden/gpuref_q_*.npz).

The extra output `rowsum` (sum of the codes of a row, int32) has no counterpart
in the reference; the int8 x int8 attention path needs it for the zero-point
correction.
"""
from __future__ import annotations

import numpy as np

QMIN = np.float32(-128.0)
QMAX = np.float32(127.0)


def round_half_away(x: np.ndarray) -> np.ndarray:
    """libdevice `roundf` for |x| < 2**23: trunc(x + copysign(0.5, x)) with the add
    rounded toward zero.  Done in float64 where the add is exact, which gives the same
    integer because integers below 2**23 are fp32-representable."""
    x64 = x.astype(np.float64)
    r = np.trunc(x64 + np.copysign(0.5, x64))
    # libdevice returns x unchanged once |x| >= 2**23 (already an integer)
    r = np.where(np.abs(x64) >= 8388608.0, x64, r)
    return r.astype(np.float32)


def _clamp(x: np.ndarray) -> np.ndarray:
    # max(qmin, min(qmax, x)) with PTX min/max semantics: a NaN operand is dropped
    return np.fmax(QMIN, np.fmin(QMAX, x))


def quantize_per_token(x: np.ndarray):
    """x: float array (..., D) holding values exactly representable in the kernel's
    input dtype (fp16 or bf16), any float dtype.

    Returns (codes int8 (..., D), scale_f32 (...,), scale_f16 (...,) float16,
             zp int8 (...,), rowsum int32 (...,)).
    """
    xf = np.asarray(x, dtype=np.float32)
    with np.errstate(all="ignore"):
        mn = np.fmin.reduce(xf, axis=-1)
        mx = np.fmax.reduce(xf, axis=-1)
        scale = ((mx - mn) / np.float32(255.0)).astype(np.float32)
        scale = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
        zpf = (QMIN - (mn / scale).astype(np.float32)).astype(np.float32)
        zp = _clamp(round_half_away(zpf)).astype(np.float32)
        t = ((xf / scale[..., None]).astype(np.float32) + zp[..., None]).astype(np.float32)
        codes_f = _clamp(round_half_away(t))
    codes = np.nan_to_num(codes_f, nan=0.0).astype(np.int32).astype(np.int8)
    zp_i8 = np.nan_to_num(zp, nan=0.0).astype(np.int32).astype(np.int8)
    rowsum = codes.astype(np.int32).sum(axis=-1, dtype=np.int32)
    with np.errstate(over="ignore"):
        scale_f16 = scale.astype(np.float16)
    return codes, scale, scale_f16, zp_i8, rowsum


def dequantize_per_token(codes: np.ndarray, scale_f16: np.ndarray, zp: np.ndarray) -> np.ndarray:
    """(code - zp) * scale with the STORED fp16 scale, in fp32
    (asymmetric_quant.py:158-160, quant_flash_attn.py:65)."""
    return (codes.astype(np.float32) - zp.astype(np.float32)[..., None]) * \
        scale_f16.astype(np.float32)[..., None]
