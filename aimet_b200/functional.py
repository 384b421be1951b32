"""Stand-alone functional API with the reference's call forms.

``quantize`` / ``quantize_dequantize`` accept the grid in any of the three ways the reference's
public functions do (quantization/affine/backends/__init__.py:50-369, parsed there by
``_parse_args`` :408-431):

* ``f(x, scale, offset, qmin, qmax, block_size=None, zero_point_shift=0.0)``
* ``f(x, scale, offset, bitwidth, signed=False, block_size=None, zero_point_shift=0.0)``
* ``f(x, scale, offset, *, num_steps, signed, block_size=None, zero_point_shift=0.0)``

and hand ``qmin, qmax`` to :mod:`aimet_b200.backend` (the protocol form a registered backend gets).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import backend

__all__ = ["quantize", "quantize_dequantize", "dequantize", "derive_qmin_qmax", "parse_grid_arguments"]


def derive_qmin_qmax(*, bitwidth: Optional[int] = None, num_steps: Optional[int] = None, signed: bool) -> Tuple[int, int]:
    """Signed grids are ``[-ceil(steps / 2), floor(steps / 2)]``, unsigned ones ``[0, steps]``, with
    ``steps = 2^bitwidth - 1`` (backends/__init__.py:434-445)."""
    if bitwidth is not None:
        num_steps = 2 ** bitwidth - 1
    if signed:
        return -math.ceil(num_steps / 2), math.floor(num_steps / 2)
    return 0, num_steps


def parse_grid_arguments(args: tuple, kwargs: dict):
    """``(qmin, qmax, block_size, zero_point_shift)`` from the positional and keyword arguments that
    follow ``(tensor, scale, offset)``.  A second grid argument that is missing or a ``bool`` marks
    the ``(bitwidth, signed)`` form; no first grid argument at all marks ``num_steps=, signed=``."""
    if len(args) > 4:
        raise TypeError(f"expected at most 4 positional arguments after (tensor, scale, offset), got {len(args)}")
    first, second, block_pos, shift_pos = tuple(args) + (None,) * (4 - len(args))
    first = kwargs.get("qmin", kwargs.get("bitwidth", first))
    second = kwargs.get("qmax", kwargs.get("signed", second))
    block_size = kwargs.get("block_size", None) or block_pos
    zero_point_shift = shift_pos or kwargs.get("zero_point_shift", 0.0)
    if first is None:
        qmin, qmax = derive_qmin_qmax(num_steps=kwargs["num_steps"], signed=kwargs["signed"])
    elif second is None or isinstance(second, bool):
        qmin, qmax = derive_qmin_qmax(bitwidth=first, signed=bool(second))
    else:
        qmin, qmax = first, second
    return qmin, qmax, block_size, zero_point_shift


def quantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, *args, **kwargs) -> torch.Tensor:
    """``clamp(round(tensor / scale) - offset, qmin, qmax)`` (backends/__init__.py:50-175)."""
    qmin, qmax, block_size, zero_point_shift = parse_grid_arguments(args, kwargs)
    if zero_point_shift != 0.0:
        raise RuntimeError("Nonzero zero_point_shift not supported for quantize()")
    return backend.quantize(tensor, scale, offset, qmin, qmax, block_size)


def quantize_dequantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, *args, **kwargs) -> torch.Tensor:
    """``(clamp(round(tensor / scale - zps) - offset, qmin, qmax) + offset + zps) * scale``
    (backends/__init__.py:215-369)."""
    qmin, qmax, block_size, zero_point_shift = parse_grid_arguments(args, kwargs)
    return backend.quantize_dequantize(tensor, scale, offset, qmin, qmax, block_size, zero_point_shift)


def dequantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, block_size=None) -> torch.Tensor:
    """``(tensor + offset) * scale`` (backends/__init__.py:372-405)."""
    return backend.dequantize(tensor, scale, offset, block_size)
