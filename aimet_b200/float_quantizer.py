"""Floating-point fake-cast quantizers on the ``aimet_b200_float_fake_cast`` kernel.

Host-side mirror of aimet_torch's ``quantization/float/quantizer.py``: ``FloatQuantizeDequantize``
(:44-540; alias ``QuantizeDequantize``), ``_MXFP4QuantizeDequantize`` (:546-584),
``_NVFP4QuantizeDequantize`` (:587-630), ``FloatEncoding`` (float/encoding.py:24-250) and the format
descriptor ``_finfo`` (float/_finfo.py).  A quantizer simulates a narrow float format on a wider
tensor: ``out = fake_cast(clamp(x / scale, -max, max)) * scale`` with
``scale = |maxval| / format_max`` calibrated from the observed range (sub-16-bit formats) or fixed
at one.  The elementwise pass is one kernel; calibration uses the B200 encoding analyzers.
"""

from __future__ import annotations

import contextlib
import math
from collections import namedtuple
from typing import Optional

import torch

from . import _lib
from ._lib import lib
from .backend import _dense_perm, _param_blocks
from .encoding_analyzer import EncodingAnalyzer, MinMaxEncodingAnalyzer, StatisticsNotFoundError
from .quantizer import QuantizerBase, _flag_extreme_min_max, _is_expandable

__all__ = ["FloatQuantizeDequantize", "QuantizeDequantize", "FloatEncoding"]


class _finfo(namedtuple("_finfo", ("exponent_bits", "mantissa_bits", "finite", "unsigned_zero"))):
    """Exponent / mantissa split of a float format, whether it lacks infinities (``finite``) and
    whether its zero is unsigned (float/_finfo.py:13-82)."""

    def to_torch_dtype(self) -> Optional[torch.dtype]:
        return _FINFO_TO_TORCH.get(self)

    @classmethod
    def from_torch_dtype(cls, dtype: torch.dtype) -> "_finfo":
        try:
            return _TORCH_TO_FINFO[dtype]
        except KeyError as e:
            raise ValueError(f"Expected dtype to be one of {list(_TORCH_TO_FINFO)}; got {dtype}") from e

    def to_str(self) -> str:
        dt = self.to_torch_dtype()
        if dt:
            return str(dt).split(".")[1]
        e, m, fn, uz = self
        return f"float{e + m + 1}_e{e}m{m}{'fn' if fn else ''}{'uz' if uz else ''}"

    def is_float16(self) -> bool:
        return self == _float16

    def is_bfloat16(self) -> bool:
        return self == _bfloat16

    @property
    def max(self) -> float:
        dt = self.to_torch_dtype()
        if dt:
            return torch.finfo(dt).max
        if self == _float4_e2m1fn:
            return 6.0
        if not self.finite and not self.unsigned_zero:
            e, m, _, _ = self
            emax = 2**e - 1
            return (2 - 2**-m) * 2 ** (emax - emax // 2 - 1)
        raise RuntimeError(f"Maximum representable value of {self.to_str()} is unkown")

    @property
    def exponent_bias(self) -> int:
        """Bias of the exponent field: the smallest normal number is 2^(1 - bias)."""
        e = self.exponent_bits
        if self.unsigned_zero:  # the "fnuz" formats give the code of -0 to NaN and shift the bias by one
            return 2 ** (e - 1)
        return 2 ** (e - 1) - 1


_float16 = _finfo(5, 10, False, False)
_bfloat16 = _finfo(8, 7, False, False)
_float8_e4m3fn = _finfo(4, 3, True, False)
_float8_e4m3fnuz = _finfo(4, 3, True, True)
_float8_e5m2 = _finfo(5, 2, False, False)
_float8_e5m2fnuz = _finfo(5, 2, True, True)
_float4_e2m1fn = _finfo(2, 1, True, False)
_FINFO_TO_TORCH = {_float16: torch.float16, _bfloat16: torch.bfloat16}
for _fi, _name in ((_float8_e4m3fn, "float8_e4m3fn"), (_float8_e4m3fnuz, "float8_e4m3fnuz"), (_float8_e5m2, "float8_e5m2"),
                   (_float8_e5m2fnuz, "float8_e5m2fnuz")):
    if hasattr(torch, _name):
        _FINFO_TO_TORCH[_fi] = getattr(torch, _name)
_TORCH_TO_FINFO = {dt: fi for fi, dt in _FINFO_TO_TORCH.items()}


class FloatEncoding:
    """Value object of a float grid with a scale (float/encoding.py:24-250, the part the quantizers use)."""

    def __init__(self, mantissa_bits: int, exponent_bits: int, finite: bool, unsigned_zero: bool, scale: torch.Tensor,
                 block_size=None, *, producer=None):
        if scale is None:
            raise ValueError("scale cannot be None for FloatEncoding")
        self._finfo = _finfo(exponent_bits, mantissa_bits, finite, unsigned_zero)
        self.scale = scale
        self.block_size = tuple(block_size) if block_size else None
        self.producer = producer

    mapping = "float"

    @property
    def mantissa_bits(self) -> int:
        return self._finfo.mantissa_bits

    @property
    def exponent_bits(self) -> int:
        return self._finfo.exponent_bits

    @property
    def bitwidth(self) -> int:
        return self._finfo.exponent_bits + self._finfo.mantissa_bits + 1

    @property
    def maxval(self) -> torch.Tensor:
        return self.scale * self._finfo.max

    def to(self, *args, **kwargs):
        return type(self)(self.mantissa_bits, self.exponent_bits, self._finfo.finite, self._finfo.unsigned_zero,
                          self.scale.to(*args, **kwargs), self.block_size, producer=self.producer)

    def quantize_dequantize(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        return float_quantize_dequantize(input, self._finfo, self.scale, self.block_size)


def float_quantize_dequantize(input: torch.Tensor, finfo: _finfo, scale: torch.Tensor,  # pylint: disable=redefined-builtin
                              block_size=None) -> torch.Tensor:
    """``fake_cast(clamp(input / scale, -max, max)) * scale`` (float/quantizer.py:619-705).  The result
    has the dtype PyTorch's type promotion gives ``input / scale`` (a scale with dimensions
    promotes a 16-bit input to float32, a 0-d one does not), like the reference's."""
    if not input.is_cuda:
        raise RuntimeError(f"aimet_b200 runs on CUDA tensors only (got a tensor on '{input.device}'); there is no CPU "
                           "fallback in this backend.")
    if finfo.to_torch_dtype() is None and finfo.unsigned_zero:
        raise NotImplementedError(f"Fake-casting to {finfo.to_str()} is not implemented")
    out_dtype = torch.result_type(input, scale)
    if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"the float fake-cast supports float16, bfloat16 and float32 tensors; got {out_dtype}")
    block_size = tuple(block_size) if block_size else None
    pshape = tuple(scale.shape)
    if block_size is not None and len(block_size) < len(pshape):  # leading scale dims broadcast numpy-style
        k = len(pshape) - len(block_size)
        block_size = tuple(1 if d > 1 else -1 for d in pshape[:k]) + block_size
    if block_size is None and not _is_expandable(pshape, input.shape):
        raise RuntimeError(f"Scale of shape {pshape} cannot be expanded like input tensor of shape {tuple(input.shape)}.")
    x = input.detach()
    if x.dtype not in (torch.float16, torch.bfloat16) or out_dtype != torch.float32:
        x = x.to(out_dtype)  # (a 16-bit tensor under a float32 result is widened inside the kernel)
    perm = None if block_size else _dense_perm(x)
    blocks = _param_blocks(x.shape, pshape, block_size)
    if perm is not None and list(perm) != list(range(x.dim())):
        pdims = [k for k in perm if x.shape[k] // blocks[k] > 1]
        if pdims != sorted(pdims):
            perm = None
    if perm is None:
        x = x.contiguous()
        perm = tuple(range(x.dim()))
    xd = x.permute(perm)
    y = torch.empty_like(xd, dtype=out_dtype, memory_format=torch.contiguous_format)
    if x.numel():
        lay = _lib.make_layout([x.shape[k] for k in perm], [blocks[k] for k in perm])
        s = scale.detach().to(torch.float32).contiguous()
        io = _lib.DTYPE_CODE[out_dtype]
        flags = (0 if finfo.to_torch_dtype() is not None else 1) | (0 if finfo.finite else 2) | (4 if finfo.unsigned_zero else 0)
        with _lib.on_device(x.device):
            rc = lib.aimet_b200_float_fake_cast(xd.data_ptr(), y.data_ptr(), s.data_ptr(), lay, _lib.DTYPE_CODE[x.dtype], io, io,
                                                finfo.exponent_bits,
                                                finfo.mantissa_bits, finfo.exponent_bias, float(finfo.max), flags,
                                                _lib.stream_ptr(x.device))
        _lib.check(rc)
    inv = [0] * len(perm)
    for i, k in enumerate(perm):
        inv[k] = i
    return y.permute(inv) if list(inv) != sorted(inv) else y


class FloatQuantizeDequantize(QuantizerBase):
    """Simulates quantization by fake-casting the input to a float format given either as a torch
    dtype or as exponent / mantissa bits (float/quantizer.py:44-540)."""

    maxval: torch.Tensor

    def __init__(self, exponent_bits: Optional[int] = None, mantissa_bits: Optional[int] = None,
                 finite: Optional[bool] = None, unsigned_zero: Optional[bool] = None, dtype: Optional[torch.dtype] = None,
                 shape=None, block_size=None, encoding_analyzer: Optional[EncodingAnalyzer] = None):
        super().__init__()
        if dtype is None:
            if exponent_bits is None or mantissa_bits is None:
                raise ValueError('Neither "dtype" nor "exponent/mantissa_bits" was specified.')
            finite = False if finite is None else finite
            unsigned_zero = False if unsigned_zero is None else unsigned_zero
        else:
            if exponent_bits is not None or mantissa_bits is not None or finite is not None or unsigned_zero is not None:
                raise ValueError('Argument "dtype" is mutually exclusive with "exponent/mantissa_bits/finite/unsigned_zero".')
            exponent_bits, mantissa_bits, finite, unsigned_zero = _finfo.from_torch_dtype(dtype)
        self._finfo = _finfo(exponent_bits, mantissa_bits, finite, unsigned_zero)
        if shape is None:
            self.shape = tuple(encoding_analyzer.observer.shape) if encoding_analyzer else ()
        else:
            self.shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        self.block_size = tuple(block_size) if block_size is not None else None
        if self.bitwidth < 16 and encoding_analyzer is None:
            encoding_analyzer = MinMaxEncodingAnalyzer(self.shape, self.block_size)
        self.encoding_analyzer = encoding_analyzer
        if encoding_analyzer and not _is_expandable(encoding_analyzer.observer.shape, self.shape):
            raise RuntimeError(f"Encoding analyzer of shape {encoding_analyzer.observer.shape} "
                               f"is incompatible with quantizer of shape {self.shape}.")
        self.register_buffer("maxval", torch.full(self.shape, self._finfo.max))
        self._is_overwrite_allowed.update({"maxval": True})
        self._observer_hook = None
        self._assert_supported_dtype()

    def _assert_supported_dtype(self):
        fi = self._finfo
        if fi != _float4_e2m1fn and (fi.finite or fi.unsigned_zero) and fi.to_torch_dtype() is None:
            special = [dt for dt in _TORCH_TO_FINFO if dt not in (torch.float16, torch.bfloat16)]
            raise RuntimeError("finite/unsigned_zero floating point has limited support. "
                               f"Expected PyTorch built-in data types, such as {special}; got '{fi.to_str()}'")

    # ---- format properties ---------------------------------------------------------------
    @property
    def exponent_bits(self) -> int:
        return self._finfo.exponent_bits

    @exponent_bits.setter
    def exponent_bits(self, value: int):
        self._finfo = self._finfo._replace(exponent_bits=value)

    @property
    def mantissa_bits(self) -> int:
        return self._finfo.mantissa_bits

    @mantissa_bits.setter
    def mantissa_bits(self, value: int):
        self._finfo = self._finfo._replace(mantissa_bits=value)

    @property
    def bitwidth(self) -> int:
        return self.exponent_bits + self.mantissa_bits + 1

    def is_float16(self) -> bool:
        return self._finfo.is_float16()

    def is_bfloat16(self) -> bool:
        return self._finfo.is_bfloat16()

    def is_initialized(self, name: Optional[str] = None) -> bool:  # the scale is a buffer, set at construction
        return self.maxval is not None

    # ---- encodings -----------------------------------------------------------------------
    def _get_log2_scale(self) -> torch.Tensor:
        return torch.log2(self.maxval.abs()) - math.log2(self._finfo.max)

    def get_scale(self) -> torch.Tensor:
        return 2 ** self._get_log2_scale()

    def get_encodings(self) -> Optional[FloatEncoding]:
        if not self.is_initialized():
            return None
        fi = self._finfo
        return FloatEncoding(fi.mantissa_bits, fi.exponent_bits, fi.finite, fi.unsigned_zero, self.get_scale(),
                             block_size=self.block_size, producer=self)

    @classmethod
    def from_encodings(cls, encodings: FloatEncoding) -> "FloatQuantizeDequantize":
        if not isinstance(encodings, FloatEncoding):
            raise TypeError(f"Expected {FloatEncoding}; got {type(encodings)}")
        q = cls(*encodings._finfo, shape=encodings.scale.shape, block_size=encodings.block_size)  # pylint: disable=protected-access
        if not (encodings.scale.numel() == 1 and float(encodings.scale) == 1):
            q.maxval = encodings.maxval.clone().detach()
        return q

    # ---- calibration (float/quantizer.py:380-454) ----------------------------------------
    @contextlib.contextmanager
    def compute_encodings(self):
        """Observe every input passed through the quantizer, quantizing each batch with the range of
        its own statistics; on exit set ``maxval`` from the accumulated statistics."""
        with self._compute_encodings(passthrough=False):
            yield

    @contextlib.contextmanager
    def _compute_encodings(self, passthrough: bool = False):
        if not self.encoding_analyzer or not any(self._is_overwrite_allowed.values()):
            yield
            return
        num_steps = math.pow(2, self.bitwidth) - 1

        def observe(input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
            run = torch.Tensor.clone if passthrough else self._forward
            if input.numel() == 0:
                return run(input)
            stats = self.encoding_analyzer.update_stats(input)
            if passthrough:
                return run(input)
            dmin, dmax = self.encoding_analyzer.compute_encodings_from_stats(stats, num_steps, is_symmetric=False)
            absmax = torch.maximum(dmin.abs(), dmax.abs()).to(dtype=self.maxval.dtype, device=self.maxval.device)
            prev, self.maxval = self.maxval, absmax.expand_as(self.maxval)
            try:
                return run(input)
            finally:
                self.maxval = prev

        self.encoding_analyzer.reset_stats()
        prev_hook, self._observer_hook = self._observer_hook, observe
        try:
            yield
        finally:
            self._observer_hook = prev_hook
        try:
            emin, emax = self.encoding_analyzer.compute_encodings(num_steps, is_symmetric=False)
            _flag_extreme_min_max(emin, emax)
        except StatisticsNotFoundError:
            return
        absmax = torch.maximum(emin.abs(), emax.abs()).expand_as(self.maxval)
        with torch.no_grad():
            self.maxval.copy_(absmax.to(dtype=self.maxval.dtype, device=self.maxval.device))

    # ---- forward -------------------------------------------------------------------------
    def forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        if self._observer_hook is not None:
            return self._observer_hook(input.as_subclass(torch.Tensor) if type(input) is not torch.Tensor else input)
        return self._forward(input)

    def _forward(self, input: torch.Tensor) -> torch.Tensor:  # pylint: disable=redefined-builtin
        if not input.is_floating_point():
            return input
        self._assert_supported_dtype()
        enc = self.get_encodings()
        if enc is None:
            if input.numel():
                raise RuntimeError("Failed to run FloatQuantizeDequantize since quantization parameters are not initialized."
                                   " Please initialize the quantization parameters using `compute_encodings()`.")
            enc = FloatEncoding(self.mantissa_bits, self.exponent_bits, self._finfo.finite, self._finfo.unsigned_zero,
                                torch.ones((), device=input.device), producer=self)
        out = float_quantize_dequantize(input, self._finfo, enc.scale, enc.block_size)
        out.encoding = enc
        return out

    def extra_repr(self) -> str:
        dt = self._finfo.to_torch_dtype()
        parts = [f"dtype={dt}"] if dt is not None else [f"exponent_bits={self.exponent_bits}", f"mantissa_bits={self.mantissa_bits}",
                                                        f"finite={self._finfo.finite}", f"unsigned_zero={self._finfo.unsigned_zero}"]
        if self.shape:
            parts.append(f"shape={self.shape}")
        if self.block_size:
            parts.append(f"block_size={self.block_size}")
        return ", ".join(parts)


class QuantizeDequantize(FloatQuantizeDequantize):
    """Alias of FloatQuantizeDequantize."""


class _MXFP4Encoding(FloatEncoding):
    def __init__(self, scale, block_size=None, *, producer=None):
        super().__init__(_float4_e2m1fn.mantissa_bits, _float4_e2m1fn.exponent_bits, _float4_e2m1fn.finite,
                         _float4_e2m1fn.unsigned_zero, scale, block_size, producer=producer)


class _NVFP4Encoding(FloatEncoding):
    def __init__(self, scale, meta_scale, block_size=None, *, producer=None):
        super().__init__(_float4_e2m1fn.mantissa_bits, _float4_e2m1fn.exponent_bits, _float4_e2m1fn.finite,
                         _float4_e2m1fn.unsigned_zero, scale, block_size, producer=producer)
        self.meta_scale = meta_scale


class _MXFP4QuantizeDequantize(FloatQuantizeDequantize):
    """fp4 (e2m1) blocks under power-of-two scales: the logarithm of the scale is rounded to an integer
    (float/quantizer.py:546-584)."""

    def __init__(self, shape, block_size):
        super().__init__(*_float4_e2m1fn, shape=shape, block_size=block_size)

    def _get_log2_scale(self) -> torch.Tensor:
        return torch.round(super()._get_log2_scale())

    def get_encodings(self) -> Optional[_MXFP4Encoding]:
        if not self.is_initialized():
            return None
        return _MXFP4Encoding(self.get_scale(), block_size=self.block_size, producer=self)


class _NVFP4QuantizeDequantize(FloatQuantizeDequantize):
    """fp4 (e2m1) blocks whose scales carry a further per-tensor ``meta_scale`` for export; the
    simulation itself is that of the plain fp4 quantizer (float/quantizer.py:587-630)."""

    def __init__(self, shape, block_size):
        super().__init__(*_float4_e2m1fn, shape=shape, block_size=block_size)
        self.register_buffer("meta_scale", torch.ones(()))

    def get_encodings(self) -> Optional[_NVFP4Encoding]:
        if not self.is_initialized():
            return None
        return _NVFP4Encoding(self.get_scale(), self.meta_scale, self.block_size, producer=self)
