"""Oracle for the floating-point fake-cast (CPU, PyTorch tensor ops).

Restates quantization/float/quantizer.py of the reference: ``_float_quantize_dequantize`` /
``_float_quantize`` (:619-705) with its two fake-cast flavours, ``_cast_decast`` (:704-705) and
``fake_cast_to_ieee_float`` (fp_quantization.py:157-214), and the scale of the float quantizers
(``_get_log2_scale`` / ``get_scale`` :333-340, MXFP4 :558-560).  Test infrastructure only.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

from .affine import _interleave, concrete_blocks

TORCH_DTYPES = {
    (5, 10, False, False): torch.float16,
    (8, 7, False, False): torch.bfloat16,
    (4, 3, True, False): torch.float8_e4m3fn,
    (4, 3, True, True): torch.float8_e4m3fnuz,
    (5, 2, False, False): torch.float8_e5m2,
    (5, 2, True, True): torch.float8_e5m2fnuz,
}


def format_max(exponent_bits, mantissa_bits, finite=False, unsigned_zero=False) -> float:
    """float/_finfo.py:62-82"""
    key = (exponent_bits, mantissa_bits, finite, unsigned_zero)
    if key in TORCH_DTYPES:
        return torch.finfo(TORCH_DTYPES[key]).max
    if key == (2, 1, True, False):
        return 6.0
    emax = 2**exponent_bits - 1
    return (2 - 2**-mantissa_bits) * 2 ** (emax - emax // 2 - 1)


def scale_from_maxval(maxval: torch.Tensor, fmt_max: float, power_of_two=False) -> torch.Tensor:
    log2_scale = torch.log2(maxval.abs()) - math.log2(fmt_max)
    if power_of_two:
        log2_scale = torch.round(log2_scale)
    return 2**log2_scale


def _blockwise(op, x, other, block_size):
    if not block_size:
        return op(x, other)
    shape = x.shape
    blocks = concrete_blocks(x.shape, other.shape, block_size)
    x = x.reshape(-1, *_interleave(other.shape, blocks))
    return op(x, other.view(_interleave(other.shape, 1))).reshape(shape)


def fake_cast_to_ieee_float(x, maxval: float, exponent_bits: int, mantissa_bits: int, finite: bool):
    """fp_quantization.py:157-214"""
    maxval = torch.tensor(maxval, dtype=torch.float64)
    bias = 2**exponent_bits - torch.log2(maxval) + np.log2(2 - 2 ** (-mantissa_bits)) - 1
    xc = x.clamp(-maxval, maxval)
    log_scales = torch.clamp(torch.floor(torch.log2(torch.abs(xc)) + bias), 1.0)
    scales = 2.0 ** (log_scales - mantissa_bits - bias)
    out = torch.round(xc / scales) * scales
    if not finite:
        out = torch.where(x.isinf(), x, out)
    return out.to(x.dtype)


def float_quantize_dequantize(x, scale, exponent_bits, mantissa_bits, finite=False, unsigned_zero=False,
                              block_size: Optional[Tuple[int, ...]] = None):
    """_float_quantize_dequantize (:619-642) on top of _float_quantize (:686-702)"""
    key = (exponent_bits, mantissa_bits, finite, unsigned_zero)
    fmax = format_max(*key)
    xs = _blockwise(torch.div, x, scale, block_size)
    xs = xs.clamp(-fmax, fmax)
    if key in TORCH_DTYPES:
        q = xs.to(TORCH_DTYPES[key]).to(xs.dtype)
    elif not unsigned_zero:
        q = fake_cast_to_ieee_float(xs, fmax, exponent_bits, mantissa_bits, finite)
    else:
        raise NotImplementedError
    return _blockwise(torch.mul, q, scale, block_size)
