"""Affine quantizer modules with learnable ranges, on the ``b200`` backend.

Host-side mirror of aimet_torch's ``quantization/affine/quantizer.py``: ``Quantize``,
``QuantizeDequantize``, ``Dequantize`` and ``GroupedBlockQuantizeDequantize`` with the same
constructor overloads, ``min``/``max`` parameters, ``compute_encodings()`` calibration context and
range accessors (``AffineQuantizerBase`` :71-838, ``Quantize`` :903-1069, ``QuantizeDequantize``
:1072-1224, ``Dequantize`` :1227-1267, ``GroupedBlockQuantizeDequantize`` :1270-1440).  The
parameter arithmetic (min/max -> scale/offset) stays ordinary differentiable PyTorch, so gradients
reach ``min`` and ``max`` through autograd; the elementwise passes over the input run in the CUDA
kernels of :mod:`aimet_b200.backend`.
"""

from __future__ import annotations

import contextlib
import math
import warnings
import weakref
from collections import OrderedDict
from itertools import chain, repeat
from typing import Optional, Tuple

import torch
from torch import nn

from . import backend
from .encoding_analyzer import (
    EncodingAnalyzer,
    MinMaxEncodingAnalyzer,
    StatisticsNotFoundError,
    _get_minimum_scale,
    _scalar,
)

__all__ = [
    "finish_calibration",
    "derive_encodings",
    "AffineEncoding",
    "AffineQuantizerBase",
    "Quantize",
    "QuantizeDequantize",
    "Dequantize",
    "GroupedBlockQuantizeDequantize",
]


class _SteRound(torch.autograd.Function):
    """Round half to even with a straight-through gradient (aimet_torch/utils.py:1250-1254)."""

    @staticmethod
    def forward(ctx, x):  # pylint: disable=arguments-differ
        return torch.round(x)

    @staticmethod
    def backward(ctx, grad):  # pylint: disable=arguments-differ
        return grad


def ste_round(x: torch.Tensor) -> torch.Tensor:
    return _SteRound.apply(x)


def _derive_qmin_qmax(*, bitwidth: int = None, num_steps: int = None, signed: bool):
    """(backends/__init__.py:433-445)"""
    if bitwidth is not None:
        num_steps = 2**bitwidth - 1
    if signed:
        return -math.ceil(num_steps / 2), math.floor(num_steps / 2)
    return 0, num_steps


def _is_expandable(src, dst) -> bool:
    if len(src) > len(dst):
        return False
    return all(s in (1, d) for s, d in zip(reversed(src), reversed(dst)))


def _concretize_block_size(in_shape, p_shape, block_size):
    in_shape = tuple(in_shape)[len(in_shape) - len(p_shape):]
    k = len(p_shape) - len(block_size)
    block_size = [*(1 if d > 1 else -1 for d in p_shape[:k]), *block_size]
    return tuple(b if b != -1 else in_shape[i] // p_shape[i] for i, b in enumerate(block_size))


def _interleave(a, b):
    if isinstance(b, int):
        b = [b] * len(a)
    return tuple(chain.from_iterable(zip(a, b)))


class AffineEncoding:
    """Value object describing an affine grid: ``x_q = clamp(round(x / scale) - offset, qmin, qmax)``
    (subset of quantization/affine/encoding.py:25-331 that the quantizers use)."""

    def __init__(self, scale, offset, qmin, qmax, symmetry=False, block_size=None, zero_point_shift=None,
                 producer=None):
        self.scale, self.offset = scale, offset
        self.qmin, self.qmax = qmin, qmax
        self.symmetry = symmetry
        self.block_size = block_size
        self.zero_point_shift = zero_point_shift or 0.0
        self.producer = producer

    @property
    def num_steps(self) -> int:
        return self.qmax - self.qmin

    @property
    def min(self) -> torch.Tensor:
        """(offset + qmin) * scale, without the zero-point shift (quantization/affine/encoding.py:140-152)."""
        return (self.offset + self.qmin) * self.scale

    @property
    def max(self) -> torch.Tensor:
        return (self.offset + self.qmax) * self.scale

    @property
    def bitwidth(self) -> int:
        return int(math.log2(self.qmax - self.qmin + 1))

    @property
    def signed(self) -> bool:
        return self.qmin < 0

    @property
    def mapping(self) -> str:
        return "affine"

    def to(self, *args, **kwargs):
        return type(self)(self.scale.to(*args, **kwargs), self.offset.to(*args, **kwargs), self.qmin, self.qmax,
                          self.symmetry, self.block_size, self.zero_point_shift, self.producer)

    # ---- the encodings wire format (quantization/affine/encoding.py:332-454) --------------
    @property
    def granularity(self) -> str:
        """(quantization/base/encoding.py:116-128)"""
        if self.scale.dim() == 0:
            return "pertensor"
        if self.block_size is not None:
            return "blockwise"
        return "perchannel" if sum(1 for d in self.scale.shape if d > 1) <= 1 else "unknown"

    def _hint_input_shape(self, input_shape) -> "AffineEncoding":
        """The shape of the tensor this encoding quantizes: needed to name channel and block axes."""
        self._input_shape_hint = tuple(input_shape)
        return self

    def _safe_get_channel_and_block_axis(self):
        """(channel axis, block axis) as negative axes of the scale (quantization/base/encoding.py:142-213)."""
        hint = getattr(self, "_input_shape_hint", None)
        if hint is None:
            raise RuntimeError("Could not safely infer channel and block axes because input shape hint is not provided. "
                               "Call `_hint_input_shape` before calling this function.")
        blocks = _concretize_block_size(hint, tuple(self.scale.shape), tuple(self.block_size or ()))
        chan = [a for a, (n, b) in enumerate(zip(self.scale.shape, blocks)) if n > 1 and b <= 1]
        blk = [a for a, (n, b) in enumerate(zip(self.scale.shape, blocks)) if n > 1 and b > 1]
        if len(blk) > 1:
            raise RuntimeError(f"Multiple non-trivial block axes found: {blk}. Cannot determine a unique block axis.")
        block_axis = blk[0] if blk else None
        if not chan and block_axis is not None:  # a singleton dimension can be the channel axis if its block size is 1
            chan = [a for a, b in enumerate(blocks) if b == 1]
        if len(chan) > 1:
            raise RuntimeError(f"Multiple non-trivial channel axes found: {chan}. Cannot determine a unique channel axis.")
        channel_axis = chan[0] if chan else None
        if channel_axis is None and block_axis is not None:
            raise RuntimeError(f"Block axis {block_axis} found without a corresponding channel axis. "
                               "Cannot determine a unique channel axis.")
        nd = self.scale.dim()
        return (None if channel_axis is None else channel_axis - nd, None if block_axis is None else block_axis - nd)

    def _get_export_dtype(self) -> str:
        nbits = math.ceil(math.log2(self.qmax - self.qmin + 1))
        return f"int{nbits}" if self.qmin < 0 <= self.qmax else f"uint{nbits}"

    def _to_legacy_format(self):
        mn, mx, scale = self.min.flatten(), self.max.flatten(), self.scale.flatten()
        offset = self.offset.flatten() + self.qmin  # the legacy format shifts the offset by qmin
        encs = [{"min": float(a), "max": float(b), "scale": float(c), "offset": int(d), "bitwidth": self.bitwidth,
                 "dtype": "int", "is_symmetric": str(self.symmetry)}
                for a, b, c, d in zip(mn.tolist(), mx.tolist(), scale.tolist(), offset.tolist())]
        if self.zero_point_shift:
            encs = [{**e, "zero_point_shift": self.zero_point_shift} for e in encs]
        return encs

    def to_qnn_encoding_dict(self, encoding_version=None):
        """The encoding as the reference's exported dictionary, versions "0.6.1", "1.0.0", "2.0.0" and
        "2.1.0" (quantization/affine/encoding.py:362-454)."""
        if encoding_version == "0.6.1":
            return self._to_legacy_format()
        if encoding_version == "1.0.0":
            out = {"dtype": "INT", "bw": self.bitwidth, "is_sym": self.symmetry, "scale": self.scale.flatten().tolist()}
            offset = self.offset - 2 ** (self.bitwidth - 1) if self.signed else self.offset
            out["offset"] = offset.to(torch.int).flatten().tolist()
            if self.zero_point_shift != 0.0:
                assert self.zero_point_shift == 0.5 and self.symmetry
                out["zero_point_shift"] = [self.zero_point_shift] * len(out["offset"])
            assert self.granularity != "unknown"
            if self.granularity == "pertensor":
                out["enc_type"] = "PER_TENSOR"
            elif self.granularity == "perchannel":
                out["enc_type"] = "PER_CHANNEL"
            else:
                _, block_axis = self._safe_get_channel_and_block_axis()
                out["enc_type"] = "PER_BLOCK"
                out["block_size"] = self.block_size[block_axis]
                if out["block_size"] == -1:
                    raise NotImplementedError("Exporting encodings to 1.0.0 format with block size -1 is not "
                                              "supported yet. Export using sim.export() instead.")
            return out
        if encoding_version in ("2.0.0", "2.1.0"):
            y_scale = self.scale
            if self.symmetry:
                zp = torch.full_like(y_scale, math.ceil((self.qmax + self.qmin) / 2), dtype=torch.int32)
            else:
                zp = -self.offset.to(torch.int32)
            if self.zero_point_shift:
                zp = zp - self.zero_point_shift
            channel_axis = block_axis = block_size = None
            if self.granularity != "pertensor":
                channel_axis, block_axis = self._safe_get_channel_and_block_axis()
            if block_axis is not None:
                axis, block_size = block_axis, self.block_size[block_axis]
            elif channel_axis is not None:
                axis, y_scale, zp = channel_axis, y_scale.flatten(), zp.flatten()
            else:
                axis, y_scale, zp = None, y_scale.squeeze(), zp.squeeze()
            ret = {"output_dtype": self._get_export_dtype(), "y_scale": y_scale.tolist()}
            if not bool(torch.all(zp == 0)):
                ret["y_zero_point"] = zp.tolist()
            if axis is not None:
                ret["axis"] = axis
            if block_size is not None:
                ret["block_size"] = block_size
            return ret
        raise AssertionError(f"Export encoding version {encoding_version} not supported."
                             "Expected one of: ['0.6.1', '1.0.0', '2.0.0', '2.1.0']")

    @classmethod
    def _from_qnn_encoding_dict(cls, encoding_dict, version=None) -> "AffineEncoding":
        """Per-tensor encodings of the 2.x format back into an encoding object (:457-498)."""
        if version is None:
            version = "2.0.0" if "y_scale" in encoding_dict or "per_block_int_scale" in encoding_dict else "unknown"
        if version not in ("2.0.0", "2.1.0"):
            raise NotImplementedError(f"Only 2.0.0 and 2.1.0 encodings are supported; got {version}")
        if "per_block_int_scale" in encoding_dict or "axis" in encoding_dict:
            raise NotImplementedError("Only per-tensor encodings are supported")
        unsigned, bw = encoding_dict["output_dtype"].split("int")
        bw = int(bw)
        qmin, qmax = (0, 2**bw - 1) if unsigned else (-(2 ** (bw - 1)), 2 ** (bw - 1) - 1)
        offset = -encoding_dict.get("y_zero_point", 0)
        return cls(torch.tensor(encoding_dict["y_scale"], dtype=torch.float32), torch.tensor(offset, dtype=torch.float32),
                   qmin, qmax, symmetry=(not unsigned) and offset == 0)

    def quantize(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        return backend.quantize(input, self.scale.to(input.dtype), self.offset.to(input.dtype), self.qmin, self.qmax,
                                self.block_size)

    def dequantize(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        return backend.dequantize(input, self.scale.to(input.dtype), self.offset.to(input.dtype), self.block_size)

    def quantize_dequantize(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        return backend.quantize_dequantize(input, self.scale.to(input.dtype), self.offset.to(input.dtype), self.qmin,
                                           self.qmax, self.block_size, self.zero_point_shift)


class GroupedBlockEncoding(AffineEncoding):
    """Blockwise grid whose block scales are integer multiples of a per-channel scale (LPBQ)."""

    def __init__(self, scale, offset, bitwidth, signed, symmetry, block_size, block_grouping, decompressed_bw,
                 per_channel_scale, zero_point_shift=None, producer=None):
        qmin, qmax = _derive_qmin_qmax(bitwidth=bitwidth, signed=signed)
        super().__init__(scale, offset, qmin, qmax, symmetry, block_size, zero_point_shift, producer)
        self.block_grouping = block_grouping
        self.decompressed_bw = decompressed_bw
        self.per_channel_scale = per_channel_scale

    @property
    def per_block_int_scale(self) -> torch.Tensor:
        """The integer factor of every block scale: ``scale = per_block_int_scale * per_channel_scale``
        (quantization/affine/encoding.py:605-620)."""
        return backend.quantize(self.scale, self.per_channel_scale, torch.zeros_like(self.per_channel_scale), 1,
                                2 ** (self.decompressed_bw - self.bitwidth), self.block_grouping)

    def to_qnn_encoding_dict(self, encoding_version=None):
        """(quantization/affine/encoding.py:622-686)"""
        out = super().to_qnn_encoding_dict(encoding_version)
        if all(g == 1 for g in self.block_grouping) or encoding_version == "0.6.1":
            return out  # equivalent to a plain blockwise encoding
        if encoding_version == "1.0.0":
            out["bw"] = self.decompressed_bw
            out["compressed_bw"] = self.bitwidth
            out["scale"] = self.per_channel_scale.flatten().tolist()
            out["offset"] = [-(2 ** (self.decompressed_bw - 1)) for _ in out["scale"]]
            out["enc_type"] = "LPBQ"
            out["per_block_int_scale"] = self.per_block_int_scale.to(torch.int32).flatten().tolist()
        elif encoding_version in ("2.0.0", "2.1.0"):
            zp = out.pop("y_zero_point", None)
            if zp is not None and bool(torch.any(torch.tensor(zp) != 0)):
                raise RuntimeError(f"LPBQ only supports symmetric quantization; got non-zero y_zero_point {zp}")
            output_dtype = f"int{self.bitwidth}" if self.signed else f"uint{self.bitwidth}"
            int_scale = self.per_block_int_scale.to(torch.int32).tolist()
            if encoding_version == "2.0.0":
                del out["y_scale"], out["output_dtype"]
                out.update({"per_block_int_scale": int_scale, "per_channel_float_scale": self.per_channel_scale.tolist(),
                            "output_dtype": output_dtype})
            else:
                channel_axis, _ = self._safe_get_channel_and_block_axis()
                out.update({"y_scale": {"x": int_scale, "x_scale": self.per_channel_scale.flatten().tolist(),
                                        "axis": channel_axis}, "output_dtype": output_dtype})
        return out


def _get_symmetric_offset(qmin, qmax, shape, dtype, device):
    value = -round((qmin + qmax) / 2)
    offset = torch.full(shape, fill_value=value, requires_grad=False, dtype=dtype, device=device)
    offset._b200_constant = float(value)  # pylint: disable=protected-access  (every element is this host-known value)
    return offset


def _scale_of_range(min, max, num_steps, dtype):  # pylint: disable=redefined-builtin
    """``|max - min| / num_steps``, never below the minimum scale (quantizer.py:319-342).  Elementwise,
    so the ranges of many quantizers laid end to end give each quantizer's own values."""
    scale = (max.to(dtype) - min.to(dtype)) / _scalar(num_steps, dtype, min.device)
    return scale.abs().clamp_min(_get_minimum_scale(num_steps)).to(dtype)


def _offset_of_range(min, scale, qmin, qmax, dtype):  # pylint: disable=redefined-builtin
    """Offset of an asymmetric grid (quantizer.py:357-376); elementwise like :func:`_scale_of_range`."""
    return torch.clamp(ste_round(min / scale) - qmin, -qmax, -qmin).to(dtype)


def _get_scale_offset(min, max, qmin, qmax, symmetric):  # pylint: disable=redefined-builtin
    """float32 (scale, offset) of a range (quantizer.py:869-900)."""
    num_steps = qmax - qmin
    if not isinstance(min, torch.Tensor):
        min = torch.tensor(min, dtype=torch.float32)
    if not isinstance(max, torch.Tensor):
        max = torch.tensor(max, dtype=torch.float32)
    out_dtype = min.dtype
    min, max = min.to(torch.float32), max.to(torch.float32)
    scale = (max - min) / _scalar(num_steps, torch.float32, min.device)
    if symmetric:
        offset = torch.full_like(min, fill_value=-round((qmin + qmax) / 2), requires_grad=False)
    else:
        offset = ste_round(min / scale) - qmin
    return scale.to(out_dtype), offset.to(out_dtype)


def _flag_extreme_min_max(curr_min, curr_max):
    """(encoding_analyzer.py:484-498)"""
    extreme = torch.full_like(curr_min, torch.finfo(curr_min.dtype).max)
    if not (torch.all(torch.isfinite(curr_min)) and torch.all(torch.isfinite(curr_max))):
        warnings.warn("Infinite or NaN values detected within input! This may skew the associated encodings")
    if torch.any(torch.isclose(torch.abs(curr_min), extreme, rtol=0.05)) or torch.any(
        torch.isclose(torch.abs(curr_max), extreme, rtol=0.05)
    ):
        warnings.warn("Extreme values detected within input! This may skew the associated encodings")


class QuantizerBase(nn.Module):
    """Bookkeeping shared by all quantizers: which parameters have been initialised since
    construction and which may be overwritten by calibration (quantization/base/quantizer.py:30-306)."""

    encoding_analyzer: EncodingAnalyzer

    def __init__(self):
        super().__init__()
        self._initial_parameters = OrderedDict()
        self._is_overwrite_allowed = OrderedDict()

    def register_quantization_parameter(self, name: str, param: Optional[nn.Parameter]):
        self.register_parameter(name, param)
        if param is not None:
            self._initial_parameters[name] = (weakref.ref(param), param._version)  # pylint: disable=protected-access

    def is_initialized(self, name: Optional[str] = None) -> bool:
        params = [(n, p) for n, p in self.named_parameters() if name is None or n == name]
        return all(self._is_initialized(n, p) for n, p in params)

    def _is_initialized(self, name, current) -> bool:
        ref, version = self._initial_parameters.get(name, (None, None))
        if ref is None:
            return True
        initial = ref()
        if initial is None or current is not initial:
            return True
        return current._version != version  # pylint: disable=protected-access

    def allow_overwrite(self, *args, **kwargs):
        mode = kwargs.get("mode", args[0] if args else None)
        flags = {n: mode for n in self._is_overwrite_allowed} if mode is not None else dict(kwargs)
        unexpected = sorted(flags.keys() - self._is_overwrite_allowed.keys())
        if unexpected:
            raise RuntimeError(
                f"'allow_overwrite' expected param names {sorted(self._is_overwrite_allowed)};"
                f" got unexpected parameter names {unexpected}"
            )
        self._is_overwrite_allowed.update(flags)

    def is_overwrite_allowed(self, name: Optional[str] = None) -> bool:
        if name is None:
            return any(self._is_overwrite_allowed.values())
        return self._is_overwrite_allowed[name]

    def get_extra_state(self):
        return {
            "is_initialized": {n: torch.tensor(self.is_initialized(n)) for n, _ in self.named_parameters()},
        }

    def set_extra_state(self, state):
        for name, flag in state.get("is_initialized", {}).items():
            if bool(flag) and name in self._initial_parameters:
                self._initial_parameters.pop(name)


class AffineQuantizerBase(QuantizerBase):
    """Base of the affine quantizers.

    ``AffineQuantizerBase(shape, bitwidth, symmetric, encoding_analyzer=None, block_size=None,
    zero_point_shift=None)`` or ``AffineQuantizerBase(shape, qmin, qmax, symmetric, ...)``.
    """

    def __init__(self, shape, *args, **kwargs):
        super().__init__()
        if isinstance(shape, int):
            shape = (shape,)
        self.shape = tuple(shape)
        full_args = (shape, *args)
        args = tuple(chain(args, repeat(None, 6 - len(args))))
        arg0 = kwargs.pop("qmin", kwargs.pop("bitwidth", args[0]))
        arg1 = kwargs.pop("qmax", args[1])
        if arg1 is not None and not isinstance(arg1, bool):
            qmin, qmax = arg0, arg1
            symmetric = kwargs.pop("symmetric", args[2])
            if qmin is None or qmax is None or symmetric is None:
                raise self._arg_parsing_error(full_args, kwargs)
            encoding_analyzer = kwargs.pop("encoding_analyzer", args[3])
            block_size = kwargs.pop("block_size", args[4])
            zero_point_shift = kwargs.pop("zero_point_shift", args[5])
        else:
            bitwidth = arg0
            symmetric = kwargs.pop("symmetric", args[1])
            if bitwidth is None or symmetric is None:
                raise self._arg_parsing_error(full_args, kwargs)
            qmin, qmax = _derive_qmin_qmax(bitwidth=bitwidth, signed=symmetric)
            encoding_analyzer = kwargs.pop("encoding_analyzer", args[2])
            block_size = kwargs.pop("block_size", args[3])
            zero_point_shift = kwargs.pop("zero_point_shift", args[4])
        if kwargs:
            raise TypeError(
                f"{type(self).__qualname__}.__init__ got unexpected keyword argument: {', '.join(kwargs)}"
            )
        if qmin >= qmax:
            raise ValueError(f"qmax should be strictly larger than qmin. Got qmax={qmax}, qmin={qmin}")
        self.qmin, self.qmax = qmin, qmax
        self._symmetric = symmetric
        self.block_size = tuple(block_size) if block_size is not None else None
        self.zero_point_shift = zero_point_shift or 0.0
        if self.zero_point_shift not in (0.0, 0.5):
            raise ValueError(f"zero_point_shift should be 0.0 or 0.5. Got {self.zero_point_shift}")
        self.encoding_analyzer = encoding_analyzer or MinMaxEncodingAnalyzer(shape=self.shape, block_size=self.block_size)
        if not _is_expandable(self.encoding_analyzer.observer.shape, self.shape):
            raise RuntimeError(
                f"Encoding analyzer of shape {self.encoding_analyzer.observer.shape} "
                f"is incompatible with quantizer of shape {self.shape}."
            )
        self.register_quantization_parameter("min", nn.Parameter(-torch.ones(self.shape)))
        self.register_quantization_parameter("max", nn.Parameter(torch.ones(self.shape)))
        self._is_overwrite_allowed.update({"min": True, "max": True})
        self._observer_hook = None  # set while compute_encodings() is active
        self._pinned_encoding = None

    def _arg_parsing_error(self, args, kwargs):
        cls = type(self).__qualname__
        given = ", ".join([*(type(a).__name__ for a in args), *(f"{k}={type(v).__name__}" for k, v in kwargs.items())])
        return TypeError(
            f"{cls}.__init__() takes (shape, bitwidth, symmetric, ...) or (shape, qmin, qmax, symmetric, ...); got ({given})"
        )

    # ---- grid properties -----------------------------------------------------------------
    @property
    def symmetric(self) -> bool:
        return self._symmetric

    @symmetric.setter
    def symmetric(self, symmetric: bool):
        self._symmetric = symmetric

    @property
    def bitwidth(self) -> int:
        return int(math.log2(self.qmax - self.qmin + 1))

    @bitwidth.setter
    def bitwidth(self, bitwidth: int):
        self.qmin, self.qmax = _derive_qmin_qmax(bitwidth=bitwidth, signed=self.signed)

    @property
    def signed(self) -> bool:
        return self.qmin < 0

    @signed.setter
    def signed(self, signed: bool):
        self.qmin, self.qmax = _derive_qmin_qmax(bitwidth=self.bitwidth, signed=signed)

    # ---- range accessors (quantizer.py:287-376) ------------------------------------------
    def get_scale(self, dtype=None) -> Optional[torch.Tensor]:
        """``|max - min| / (qmax - qmin)``, never below the minimum scale; ``None`` before initialisation."""
        if self._pinned_encoding is not None:
            return self._pinned_encoding.scale.to(dtype or torch.float32)
        if not self.is_initialized():
            return None
        return _scale_of_range(self.min, self.max, self.qmax - self.qmin, dtype or torch.float32)

    def get_offset(self, dtype=None) -> Optional[torch.Tensor]:
        return self._get_offset(dtype=dtype)

    def _get_offset(self, scale=None, dtype=None) -> Optional[torch.Tensor]:
        if self._pinned_encoding is not None:
            return self._pinned_encoding.offset.to(dtype or torch.float32)
        if not self.is_initialized():
            return None
        dtype = dtype or torch.float32
        if self.symmetric:
            return _get_symmetric_offset(self.qmin, self.qmax, self.shape, dtype, self.min.device)
        scale = scale if scale is not None else self.get_scale(dtype)
        return _offset_of_range(self.min, scale, self.qmin, self.qmax, dtype)

    def get_min(self, dtype=None) -> Optional[torch.Tensor]:
        scale = self.get_scale(dtype)  # derived once: the offset below is formed from the same values
        if scale is None:
            return None
        return scale * (self._scale_and_offset(scale, dtype) + self.qmin + self.zero_point_shift)

    def get_max(self, dtype=None) -> Optional[torch.Tensor]:
        scale = self.get_scale(dtype)
        if scale is None:
            return None
        return scale * (self._scale_and_offset(scale, dtype) + self.qmax + self.zero_point_shift)

    def _scale_and_offset(self, scale, dtype):
        """``get_offset(dtype)`` given the already derived ``get_scale(dtype)`` (a subclass with its own
        ``get_offset`` is asked directly)."""
        if type(self).get_offset is not AffineQuantizerBase.get_offset:
            return self.get_offset(dtype)
        return self._get_offset(scale=scale, dtype=dtype)

    @torch.no_grad()
    def set_range(self, min, max):  # pylint: disable=redefined-builtin
        """Overwrite ``min`` / ``max`` (either may be ``None`` to keep it)."""
        if min is not None:
            self.min.copy_(min if isinstance(min, torch.Tensor) else torch.tensor(min))
        if max is not None:
            self.max.copy_(max if isinstance(max, torch.Tensor) else torch.tensor(max))

    def get_encodings(self) -> Optional[AffineEncoding]:
        if self._pinned_encoding is not None:
            return self._pinned_encoding
        scale = self.get_scale(dtype=torch.float32)
        if scale is None:
            return None
        offset = self._get_offset(scale=scale, dtype=torch.float32)
        return AffineEncoding(scale, offset, self.qmin, self.qmax, self._symmetric, self.block_size,
                              self.zero_point_shift, producer=self)

    @contextlib.contextmanager
    def _precompute_encodings(self, dtype: Optional[torch.dtype] = None):
        """Derive scale / offset once and use them for every forward inside the context
        (quantizer.py:790-804 of the reference).  Opt-in on purpose: outside it the encoding is
        re-derived from ``min`` / ``max`` on every forward, like the reference does, so that any
        way of editing the parameters (``.data`` included, which leaves no trace in the tensor's
        version counter) takes effect."""
        with torch.no_grad():
            enc = self.get_encodings()
            if enc is not None:
                enc = enc.to(dtype=dtype or torch.float32)
                enc.scale, enc.offset = enc.scale.detach().contiguous(), enc.offset.detach().contiguous()
                if self._symmetric:  # every zero point is this constant: known without reading the device
                    enc.offset._b200_constant = float(-round((self.qmin + self.qmax) / 2))  # pylint: disable=protected-access
        with self._set_encodings(enc):
            yield

    def _get_dummy_encoding(self) -> AffineEncoding:
        device = self.min.device
        return AffineEncoding(torch.ones((), device=device), torch.zeros((), device=device), self.qmin, self.qmax,
                              self._symmetric, None, self.zero_point_shift, producer=self)

    @contextlib.contextmanager
    def _set_encodings(self, enc: Optional[AffineEncoding]):
        prev, self._pinned_encoding = self._pinned_encoding, enc
        try:
            yield
        finally:
            self._pinned_encoding = prev

    # ---- calibration (quantizer.py:591-698) ----------------------------------------------
    @contextlib.contextmanager
    def compute_encodings(self):
        """Observe every input passed through the quantizer, quantizing each batch with the encodings
        of its own statistics; on exit set ``min`` / ``max`` from the accumulated statistics."""
        with self._compute_encodings(passthrough=False):
            yield

    @contextlib.contextmanager
    def _compute_encodings(self, passthrough: bool = False, clone: bool = True, finish: bool = True):
        """``passthrough``: observe without quantizing, returning a copy of the input like the
        reference does (quantizer.py:628-667) or, with ``clone=False``, the input itself (for callers
        that know nothing downstream needs a private copy).  ``finish=False`` leaves the statistics
        in the analyzer on exit: the caller turns them into ranges itself, for many quantizers at
        once (:func:`finish_calibration`)."""
        if not any(self._is_overwrite_allowed.values()):
            yield
            return
        shape = self.shape
        dtype, device = self.min.dtype, self.min.device

        def observe(input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
            run = (torch.Tensor.clone if clone else (lambda t: t)) if passthrough else self._forward
            if input.numel() == 0:
                return run(input)
            if passthrough:  # nothing is quantized while observing: no per-batch statistics or encoding needed
                watch = getattr(self.encoding_analyzer, "observe", None)
                if watch is not None:
                    watch(input)
                else:
                    self.encoding_analyzer.update_stats(input)
                return run(input)
            batch_stats = self.encoding_analyzer.update_stats(input)
            dyn_min, dyn_max = self.encoding_analyzer.compute_encodings_from_stats(
                batch_stats, self._calibration_steps(), self.symmetric
            )
            if self.block_size is not None:
                dyn_min, dyn_max = dyn_min.view(shape), dyn_max.view(shape)
            dyn_min = dyn_min.to(dtype=dtype, device=device).expand(shape)
            dyn_max = dyn_max.to(dtype=dtype, device=device).expand(shape)
            scale, offset = _get_scale_offset(dyn_min.to(torch.float32), dyn_max.to(torch.float32), qmin=self.qmin,
                                              qmax=self.qmax, symmetric=self.symmetric)
            enc = AffineEncoding(scale, offset, self.qmin, self.qmax, self.symmetric, self.block_size,
                                 self.zero_point_shift, producer=self)
            with self._set_encodings(enc):
                ret = run(input)
            if not hasattr(ret, "encoding"):
                ret.encoding = enc
            return ret

        self.encoding_analyzer.reset_stats()
        prev_hook, self._observer_hook = self._observer_hook, observe
        try:
            yield
        finally:
            self._observer_hook = prev_hook
        if finish:
            self._finish_calibration()

    def _finish_calibration(self):
        """Set ``min`` / ``max`` from the statistics gathered so far (quantizer.py:669-698)."""
        shape = self.shape
        try:
            enc_min, enc_max = self.encoding_analyzer.compute_encodings(self._calibration_steps(), self.symmetric)
        except StatisticsNotFoundError:
            return
        if self.block_size is not None:
            enc_min, enc_max = enc_min.view(shape), enc_max.view(shape)
        _flag_extreme_min_max(enc_min, enc_max)
        self.set_range(enc_min if self._is_overwrite_allowed["min"] else None,
                       enc_max if self._is_overwrite_allowed["max"] else None)

    def _calibration_steps(self) -> int:
        steps = self.qmax - self.qmin
        return steps - 1 if self.zero_point_shift == 0.5 else steps

    # ---- forward -------------------------------------------------------------------------
    def forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        if self._observer_hook is not None:
            return self._observer_hook(input.as_subclass(torch.Tensor) if type(input) is not torch.Tensor else input)
        return self._forward(input)

    def _forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        raise NotImplementedError

    def _encoding_for(self, input: torch.Tensor, what: str) -> AffineEncoding:  # pylint: disable=redefined-builtin
        enc = self.get_encodings()
        if enc is None:
            if input.numel() == 0:
                return self._get_dummy_encoding()
            raise RuntimeError(
                f"Failed to run {what} since quantization parameters are not initialized."
                " Please initialize the quantization parameters using `compute_encodings()`."
            )
        return enc

    def extra_repr(self) -> str:
        parts = [f"shape={self.shape}"]
        if self.block_size:
            parts.append(f"block_size={self.block_size}")
        parts += [f"qmin={self.qmin}", f"qmax={self.qmax}", f"symmetric={self.symmetric}"]
        if self.zero_point_shift:
            parts.append(f"zero_point_shift={self.zero_point_shift}")
        return ", ".join(parts)

    def get_extra_state(self):
        state = super().get_extra_state()
        state.update(qmin=torch.tensor(self.qmin), qmax=torch.tensor(self.qmax), symmetric=torch.tensor(self.symmetric),
                     block_size=torch.tensor(self.block_size or ()), zero_point_shift=torch.tensor(self.zero_point_shift))
        return state

    def set_extra_state(self, state):
        super().set_extra_state(state)
        if "qmin" in state:
            self.qmin = int(state["qmin"])
        if "qmax" in state:
            self.qmax = int(state["qmax"])
        if "symmetric" in state:
            self.symmetric = bool(state["symmetric"])
        if "block_size" in state:
            self.block_size = tuple(int(b) for b in state["block_size"]) or None
        if "zero_point_shift" in state:
            self.zero_point_shift = float(state["zero_point_shift"])
        self.shape = tuple(self.min.shape)


def finish_calibration(quantizers) -> None:
    """``_finish_calibration`` of many quantizers with a handful of launches: the statistics of all
    min-max calibrated quantizers that share a grid (steps, symmetry, dtype) are laid end to end,
    turned into ranges by one evaluation of the analyzer's rule (elementwise over the statistics, so
    the values are those of per-quantizer evaluation) and copied back.  A model has a hundred
    quantizers; one by one their few small tensor operations each dominate a calibration."""
    from .encoding_analyzer import _MinMaxRange

    groups = {}
    for q in quantizers:
        an = q.encoding_analyzer
        st = an.observer.get_stats() if isinstance(an, MinMaxEncodingAnalyzer) and type(q)._finish_calibration is \
            AffineQuantizerBase._finish_calibration else None
        if st is None or st.min is None:
            q._finish_calibration()  # pylint: disable=protected-access  (another analyzer, or nothing observed)
            continue
        key = (q._calibration_steps(), q.symmetric, st.min.dtype, st.min.device)  # pylint: disable=protected-access
        groups.setdefault(key, []).append((q, st))
    for (steps, symmetric, _, _), members in groups.items():
        if len(members) == 1:
            members[0][0]._finish_calibration()  # pylint: disable=protected-access
            continue
        mins = torch.cat([st.min.reshape(-1) for _, st in members])
        maxs = torch.cat([st.max.reshape(-1) for _, st in members])
        lo, hi = MinMaxEncodingAnalyzer(()).compute_encodings_from_stats(_MinMaxRange(mins, maxs), steps, symmetric)
        sizes = [st.min.numel() for _, st in members]
        dst, src = [], []
        for (q, _), a, b in zip(members, lo.split(sizes), hi.split(sizes)):
            if q._is_overwrite_allowed["min"]:  # pylint: disable=protected-access
                dst.append(q.min)
                src.append(a.view(q.shape))
            if q._is_overwrite_allowed["max"]:  # pylint: disable=protected-access
                dst.append(q.max)
                src.append(b.view(q.shape))
        with torch.no_grad():
            if all(d.dtype == s.dtype for d, s in zip(dst, src)):
                torch._foreach_copy_(dst, src)  # pylint: disable=protected-access  (all the copies in a launch or two)
            else:
                for d, s in zip(dst, src):
                    d.copy_(s)
        _flag_extreme_min_max(lo, hi)  # reads the device: last, so that the copies are queued behind the forward passes


def derive_encodings(quantizers):
    """``get_encodings()`` of many quantizers with a handful of launches: the ranges of all quantizers
    that share a grid (qmin, qmax, symmetry, dtype) are laid end to end and the scale / offset
    rules, which are elementwise, are evaluated once over all of them; each quantizer gets views of
    the result, with the values its own ``get_encodings()`` would have computed.  Quantizers that
    define their own rules, hold a pinned encoding or are not initialised are asked one by one.
    Returns the encodings in the order of ``quantizers``, detached from the ranges."""
    out, groups = {}, {}
    plain = (AffineQuantizerBase.get_scale, AffineQuantizerBase._get_offset, AffineQuantizerBase.get_encodings)  # pylint: disable=protected-access
    for i, q in enumerate(quantizers):
        cls = type(q)
        if (cls.get_scale, cls._get_offset, cls.get_encodings) != plain or q._pinned_encoding is not None \
                or not q.is_initialized() or q.min.shape != q.max.shape:  # pylint: disable=protected-access
            with torch.no_grad():
                out[i] = q.get_encodings()
            continue
        key = (q.qmin, q.qmax, q._symmetric, q.min.dtype, q.max.dtype, q.min.device)  # pylint: disable=protected-access
        groups.setdefault(key, []).append(i)
    with torch.no_grad():
        for (qmin, qmax, symmetric, _, _, device), members in groups.items():
            qs = [quantizers[i] for i in members]
            mins = torch.cat([q.min.reshape(-1) for q in qs])
            maxs = torch.cat([q.max.reshape(-1) for q in qs])
            scales = _scale_of_range(mins, maxs, qmax - qmin, torch.float32)
            if symmetric:
                offsets = _get_symmetric_offset(qmin, qmax, scales.shape, torch.float32, device)
                constant = offsets._b200_constant  # pylint: disable=protected-access
            else:
                offsets, constant = _offset_of_range(mins, scales, qmin, qmax, torch.float32), None
            sizes = [q.min.numel() for q in qs]
            for i, q, s, o in zip(members, qs, scales.split(sizes), offsets.split(sizes)):
                o = o.view(q.shape)
                if constant is not None:
                    o._b200_constant = constant  # pylint: disable=protected-access
                out[i] = AffineEncoding(s.view(q.shape), o, q.qmin, q.qmax, q._symmetric, q.block_size,  # pylint: disable=protected-access
                                        q.zero_point_shift, producer=q)
    return [out[i] for i in range(len(quantizers))]


class Quantize(AffineQuantizerBase):
    """``out = clamp(round(input / scale) - offset, qmin, qmax)`` with scale / offset derived from the
    learnable ``min`` / ``max``; the output carries its encoding as ``out.encoding``."""

    def __init__(self, shape, *args, **kwargs):
        super().__init__(shape, *args, **kwargs)
        if self.zero_point_shift != 0.0:
            raise RuntimeError("Nonzero quant shift not supported for Quantize")

    def _forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        enc = self._encoding_for(input, "Quantize")
        out = backend.quantize(input, enc.scale, enc.offset, enc.qmin, enc.qmax, block_size=enc.block_size)
        out.encoding = enc
        return out


class QuantizeDequantize(AffineQuantizerBase):
    """Fake-quantization ``out = (clamp(round(input / scale) - offset, qmin, qmax) + offset) * scale``."""

    def _forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        enc = self._encoding_for(input, "QuantizeDequantize")
        out = backend.quantize_dequantize(input, enc.scale, enc.offset, enc.qmin, enc.qmax, block_size=enc.block_size,
                                          zero_point_shift=enc.zero_point_shift)
        out.encoding = enc
        return out


class Dequantize(AffineQuantizerBase):
    """``out = (input + offset) * scale``"""

    def _forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        if self.zero_point_shift != 0.0:
            raise RuntimeError("Nonzero quant shift not supported for Dequantize")
        enc = self._encoding_for(input, "Dequantize")
        out = backend.dequantize(input, enc.scale, enc.offset, block_size=enc.block_size)
        out.encoding = enc
        return out


class GroupedBlockQuantizeDequantize(QuantizeDequantize):
    """Low-power blockwise quantization: every block scale is ``k * per_channel_scale`` with an integer
    ``k`` in ``[1, 2^(decompressed_bw - bitwidth)]``, the per-channel scale being the largest block
    scale of the group divided by that power of two (quantizer.py:1270-1440)."""

    def __init__(self, shape, bitwidth: int, symmetric: bool, decompressed_bw: int,
                 encoding_analyzer: EncodingAnalyzer = None, block_size: Optional[Tuple[int, ...]] = None,
                 block_grouping: Optional[Tuple[int, ...]] = None):
        super().__init__(shape, bitwidth, symmetric, encoding_analyzer, block_size)
        self.decompressed_bw = decompressed_bw
        self.block_grouping = tuple(block_grouping) if block_grouping is not None else tuple(1 for _ in self.shape)
        if block_grouping is not None:
            if len(block_grouping) != len(self.shape):
                raise RuntimeError(f"Length of block grouping {block_grouping} must equal length of shape {shape}.")
            for dim, group in zip(self.shape, block_grouping):
                if group != -1 and dim % group != 0:
                    raise RuntimeError(
                        f"Quantizer shape dimensions must divide evenly with corresponding block "
                        f"grouping values for shapes {shape} and block grouping {block_grouping}."
                    )
        if self.decompressed_bw < self.bitwidth:
            raise RuntimeError(f"Decompressed bitwidth {decompressed_bw} cannot be smaller than self.bitwidth {bitwidth}")
        if not symmetric:
            raise RuntimeError("GroupedBlockQuantizeDequantize only supports symmetric quantization.")

    def get_scale(self, dtype=None) -> Optional[torch.Tensor]:
        return self._get_scale(dtype)[0]

    def get_per_channel_scale(self, dtype=None) -> Optional[torch.Tensor]:
        raw = super().get_scale(dtype)
        return None if raw is None else self._get_per_channel_scale(raw)

    def _get_scale(self, dtype=None):
        raw = super().get_scale(dtype)
        if raw is None:
            return None, None
        per_channel = self._get_per_channel_scale(raw)
        lpbq = backend.quantize_dequantize(raw, per_channel, torch.zeros_like(per_channel), 1,
                                           2 ** (self.decompressed_bw - self.bitwidth), self.block_grouping)
        return lpbq, per_channel

    def _get_per_channel_scale(self, raw: torch.Tensor) -> torch.Tensor:
        pc_shape = [d // g if g != -1 else 1 for d, g in zip(raw.shape, self.block_grouping)]
        grouping = _concretize_block_size(raw.shape, pc_shape, self.block_grouping)
        grouped = raw.reshape(*raw.shape[: raw.dim() - len(pc_shape)], *_interleave(pc_shape, grouping))
        group_max = torch.amax(grouped, dim=tuple(range(1, grouped.dim(), 2)))
        return group_max / 2 ** (self.decompressed_bw - self.bitwidth)

    def get_encodings(self) -> Optional[GroupedBlockEncoding]:
        if self._pinned_encoding is not None:
            return self._pinned_encoding
        if not self.is_initialized():
            return None
        lpbq, per_channel = self._get_scale(dtype=torch.float32)
        return GroupedBlockEncoding(lpbq, self.get_offset(dtype=torch.float32), self.bitwidth, self.signed,
                                    self.symmetric, self.block_size, self.block_grouping, self.decompressed_bw,
                                    per_channel, self.zero_point_shift, producer=self)
