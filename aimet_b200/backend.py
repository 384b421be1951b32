"""The ``b200`` quantization backend.

This module satisfies aimet_torch's ``_QuantizationBackendProtocol``
(quantization/affine/backends/utils.py:16-44): three callables ``quantize``,
``dequantize`` and ``quantize_dequantize`` with the reference's argument meaning, validation
errors and dtype rules (quantization/affine/backends/torch_builtins.py:119-302, 537-571),
executed by the sm_100a kernels behind the C ABI.  Register it with
``aimet_b200.register_backend()`` and select it with
``aimet_torch.quantization.set_backend("b200")``.

CUDA tensors only: a CPU tensor raises ``RuntimeError`` (there is no fallback path).
"""

from __future__ import annotations

import functools
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib, pgs
from ._lib import lib

__all__ = ["quantize", "dequantize", "quantize_dequantize"]

_MANTISSA_BITS = {
    torch.float32: 23,
    torch.float16: 10,
    torch.bfloat16: 7,
    torch.float64: 52,
}


# ---------------------------------------------------------------------------
# dtype rules (torch_builtins.py:49-116)
# ---------------------------------------------------------------------------
def _is_value_representable(dtype: torch.dtype, value: int) -> bool:
    """An integer is exact in ``dtype`` iff the span between its highest and lowest set bit
    fits in the mantissa (and it is within range)."""
    if dtype not in _MANTISSA_BITS:
        raise ValueError(f"Expected dtype to be one of float32, float16, bfloat16, or float64; got {dtype}")
    finfo = torch.finfo(dtype)
    if not finfo.min <= value <= finfo.max:
        return False
    mag = abs(int(value))
    if mag == 0:
        return True
    msb = mag.bit_length() - 1
    lsb = (mag & -mag).bit_length() - 1
    return msb - lsb <= _MANTISSA_BITS[dtype]


@functools.lru_cache(None)
def _is_grid_representable(dtype: torch.dtype, qmin: int, qmax: int) -> bool:
    return all(_is_value_representable(dtype, v) for v in (qmax, qmax - 1, qmin + 1, qmin))


def _is_numerically_stable(dtype: torch.dtype, qmin: int, qmax: int) -> bool:
    if not _is_grid_representable(dtype, qmin, qmax):
        return False
    if qmin == qmax:
        return True
    return not torch.finfo(dtype).eps > 0.25 / (qmax - qmin)


def _internal_dtype(dtype: torch.dtype, qmin: int, qmax: int) -> torch.dtype:
    if _is_numerically_stable(dtype, qmin, qmax):
        return dtype
    if _is_numerically_stable(torch.float32, qmin, qmax):
        return torch.float32
    return torch.float64


# ---------------------------------------------------------------------------
# validation (torch_builtins.py:119-162)
# ---------------------------------------------------------------------------
def _is_expandable(src: Sequence[int], dst: Sequence[int]) -> bool:
    if len(src) > len(dst):
        return False
    return all(s in (1, d) for s, d in zip(reversed(src), reversed(dst)))


def _validate(tensor, scale, offset, qmin=None, qmax=None, block_size=None):
    for name, t in (("input", tensor), ("scale", scale), ("offset", offset)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor, got {type(t)}")
    if not tensor.is_cuda:
        raise RuntimeError(
            "aimet_b200 runs on CUDA tensors only (got a tensor on "
            f"'{tensor.device}'); there is no CPU fallback in this backend."
        )
    if scale.device != tensor.device or offset.device != tensor.device:
        raise RuntimeError(
            "Expected all tensors to be on the same device, but found input on "
            f"{tensor.device}, scale on {scale.device} and offset on {offset.device}"
        )
    if block_size is not None:
        if len(scale.shape) != len(block_size):
            raise RuntimeError(
                f"Length of scale shape {scale.shape} must equal length of block size {block_size}"
            )
        if len(tensor.shape) < len(scale.shape):
            raise RuntimeError(
                f"Input shape {tuple(tensor.shape)} must have at least as many dimensions as "
                f"scale shape {tuple(scale.shape)}."
            )
        for i in range(1, len(block_size) + 1):
            if block_size[-i] == -1:
                if scale.shape[-i] == 0 or tensor.shape[-i] % scale.shape[-i] != 0:
                    raise RuntimeError(
                        f"Each tensor dimension size for tensor shape {tensor.shape} must divide "
                        f"evenly with corresponding scale dimension value for scale shape {scale.shape}"
                    )
            elif block_size[-i] * scale.shape[-i] != tensor.shape[-i]:
                raise RuntimeError(
                    f"Each tensor dimension size for tensor shape {tensor.shape} must equal the "
                    f"corresponding scale dimension size * block size for scale shape {scale.shape} "
                    f"and block size {block_size}"
                )
    elif not _is_expandable(scale.shape, tensor.shape):
        msg = f"Scale of shape {scale.shape} cannot be expanded like input tensor of shape {tensor.shape}. "
        if tensor.numel() == 0:
            msg += "Detected that the tensor is empty; check that the input tensor is the intended one."
        raise RuntimeError(msg)
    if qmin is not None and qmax is not None and qmin > qmax:
        raise RuntimeError(f"qmin ({qmin}) must be smaller than or equal to qmax ({qmax})")


# ---------------------------------------------------------------------------
# layout: which run of coordinates along each dim shares one parameter
# ---------------------------------------------------------------------------
def _param_blocks(shape: Sequence[int], pshape: Sequence[int], block_size) -> Tuple[int, ...]:
    """Elements per parameter along each tensor dim (parameter shape right-aligned)."""
    nd = len(shape)
    pad = nd - len(pshape)
    blocks = []
    for k in range(nd):
        if k < pad:
            blocks.append(shape[k])
            continue
        p = pshape[k - pad]
        if block_size is None:
            blocks.append(shape[k] if p == 1 else 1)
        else:
            b = block_size[k - pad]
            blocks.append(shape[k] // p if b == -1 else b)
    return tuple(int(max(b, 1)) for b in blocks)


def _dense_perm(t: torch.Tensor) -> Optional[Tuple[int, ...]]:
    """Permutation of dims under which ``t`` is row-major contiguous, else None."""
    if t.is_contiguous():
        return tuple(range(t.dim()))
    perm = tuple(sorted(range(t.dim()), key=lambda k: (-t.stride(k), k)))
    if t.permute(perm).is_contiguous():
        return perm
    return None


class _Plan:
    """Everything the C ABI needs to know about one call, derived once in forward."""

    __slots__ = ("perm", "layout", "io", "ct", "pt", "pshape", "upcast")

    def __init__(self, perm, layout, io, ct, pt, pshape, upcast):
        self.perm, self.layout, self.io, self.ct, self.pt = perm, layout, io, ct, pt
        self.pshape, self.upcast = pshape, upcast


def _prepare(tensor, scale, offset, block_size, internal_dtype):
    """Returns (x_dense_view, plan).  ``x_dense_view`` is a contiguous permuted view (or copy)."""
    # (torch.broadcast_shapes costs as much as the rest of this function; the shapes are nearly always equal)
    pshape = scale.shape if scale.shape == offset.shape else torch.broadcast_shapes(scale.shape, offset.shape)
    perm = None if block_size else _dense_perm(tensor)
    if perm is None:
        x = tensor.contiguous()
        perm = tuple(range(tensor.dim()))
    else:
        x = tensor.permute(perm)
    blocks = _param_blocks(tensor.shape, pshape, block_size)
    if list(perm) != list(range(tensor.dim())):
        # parameters follow the logical dim order; only a permutation that keeps the parameter
        # array row-major can be described to the kernels, otherwise densify the input
        pdims = [k for k in perm if tensor.shape[k] // blocks[k] > 1]
        if pdims != sorted(pdims):
            x = tensor.contiguous()
            perm = tuple(range(tensor.dim()))
    size_p = [tensor.shape[k] for k in perm]
    block_p = [blocks[k] for k in perm]

    io_dtype = x.dtype
    upcast = False
    if io_dtype not in _lib.DTYPE_CODE:
        raise RuntimeError(f"aimet_b200 supports float16, bfloat16, float32 and float64 inputs; got {io_dtype}")
    if internal_dtype == torch.float64 and io_dtype in (torch.float16, torch.bfloat16):
        x = x.to(torch.float32)
        io_dtype = torch.float32
        upcast = True
    elif internal_dtype == torch.float32 and io_dtype == torch.float64:
        internal_dtype = torch.float64
    pt = torch.float64 if internal_dtype == torch.float64 else torch.float32
    plan = _Plan(
        perm,
        _lib.make_layout(size_p, block_p),
        _lib.DTYPE_CODE[io_dtype],
        _lib.DTYPE_CODE[internal_dtype],
        pt,
        tuple(pshape),
        upcast,
    )
    return x, plan


def _param(t, plan: _Plan):
    t = t.detach()
    if t.dtype == plan.pt and tuple(t.shape) == plan.pshape and t.is_contiguous():
        return t  # the common case: float32 parameters of the parameter shape
    return t.expand(plan.pshape).to(plan.pt).contiguous()


def _params(scale, offset, plan: _Plan):
    return _param(scale, plan), _param(offset, plan)


def _restore(y_dense: torch.Tensor, plan: _Plan, like: torch.Tensor) -> torch.Tensor:
    """Undo the dense permutation and the optional upcast."""
    if plan.upcast:
        y_dense = y_dense.to(like.dtype)
    inv = [0] * len(plan.perm)
    for i, k in enumerate(plan.perm):
        inv[k] = i
    return y_dense.permute(inv) if list(inv) != sorted(inv) else y_dense


_OPS_FWD = {
    "q": lib.aimet_b200_quantize,
    "dq": lib.aimet_b200_dequantize,
    "qdq": lib.aimet_b200_quantize_dequantize,
}


def _run_forward(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype):
    """Launch one forward kernel.  Returns (output, dense input view, scale, offset, plan)."""
    x, plan = _prepare(tensor, scale, offset, block_size, internal_dtype)
    s, o = _params(scale, offset, plan)
    y = torch.empty_like(x, memory_format=torch.contiguous_format)
    if x.numel() > 0:
        pt = _lib.DTYPE_CODE[plan.pt]
        with _lib.on_device(x.device):
            st = _lib.stream_ptr(x.device)
            if op == "q":
                rc = lib.aimet_b200_quantize(x.data_ptr(), y.data_ptr(), s.data_ptr(), o.data_ptr(), plan.layout,
                                             plan.io, plan.ct, pt, qmin, qmax, st)
            elif op == "dq":
                rc = lib.aimet_b200_dequantize(x.data_ptr(), y.data_ptr(), s.data_ptr(), o.data_ptr(), plan.layout,
                                               plan.io, plan.ct, pt, st)
            elif op == "fq":
                rc = lib.aimet_b200_fake_quantize(x.data_ptr(), y.data_ptr(), s.data_ptr(), o.data_ptr(), plan.layout,
                                                  plan.io, qmin, qmax, st)
            else:
                rc = lib.aimet_b200_quantize_dequantize(x.data_ptr(), y.data_ptr(), s.data_ptr(), o.data_ptr(),
                                                        plan.layout, plan.io, plan.ct, pt, qmin, qmax, float(zps), st)
        _lib.check(rc)
    return _restore(y, plan, tensor), x, s, o, plan


@torch.compiler.disable
def _apply(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype):
    """Through autograd only when a gradient can flow; otherwise straight to the kernel.

    Opaque to ``torch.compile``: the kernels are reached through ctypes, which a tracing compiler
    cannot follow, so a compiled region breaks its graph here and runs this call eagerly (the
    reference registers ``torch.library`` operators with meta kernels for its Triton backend,
    triton.py:685-881; an opaque eager call gives the same results without a second code path)."""
    if torch.is_grad_enabled() and (tensor.requires_grad or scale.requires_grad or offset.requires_grad):
        return _AffineFunction.apply(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype)
    return _run_forward(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype)[0]


class _AffineFunction(torch.autograd.Function):
    """Forward and backward of the three affine functionals through the C ABI.

    Gradients follow QuantizeFunc / DequantizeFunc / QuantDequantFunc.backward
    (torch_builtins.py:637-659, 689-701, 772-831); scale and offset gradients come back already
    reduced to the parameter shape.
    """

    @staticmethod
    def forward(ctx, tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype):
        y, x, s, o, plan = _run_forward(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype)
        ctx.plan = plan
        ctx.op, ctx.qmin, ctx.qmax, ctx.zps = op, qmin, qmax, float(zps)
        ctx.pgs = (pgs.get_pgs_eps(), pgs.get_pgs_multiplier())  # as set when the forward ran, like the reference
        ctx.in_dtype = tensor.dtype
        ctx.scale_meta = (scale.shape, scale.dtype)
        ctx.offset_meta = (offset.shape, offset.dtype)
        if any(ctx.needs_input_grad[:3]):
            ctx.save_for_backward(x, s, o)
        return y

    @staticmethod
    def backward(ctx, grad):
        x, s, o = ctx.saved_tensors
        plan: _Plan = ctx.plan
        need_x, need_s, need_o = ctx.needs_input_grad[:3]
        g = grad.permute(plan.perm).to(x.dtype).contiguous()
        gx = torch.empty_like(x) if need_x else None
        gs = torch.empty(plan.pshape, dtype=plan.pt, device=x.device) if need_s else None
        go = torch.empty(plan.pshape, dtype=plan.pt, device=x.device) if need_o else None
        if x.numel() == 0:
            if gs is not None:
                gs.zero_()
            if go is not None:
                go.zero_()
        else:
            with _lib.on_device(x.device):
                nbytes = lib.aimet_b200_backward_scratch_bytes(plan.layout, plan.io)
                _lib.check(nbytes)
                scratch = _lib.scratch.get(x.device, nbytes) if (need_s or need_o) else None
                st = _lib.stream_ptr(x.device)
                common = (x.data_ptr(), g.data_ptr(), s.data_ptr(), o.data_ptr(), plan.layout, plan.io,
                          plan.ct, _lib.DTYPE_CODE[plan.pt])
                tail = (_lib.ptr(gx), _lib.ptr(gs), _lib.ptr(go), _lib.ptr(scratch),
                        0 if scratch is None else scratch.numel(), st)
                if ctx.op == "fq":
                    rc = lib.aimet_b200_fake_quantize_backward(x.data_ptr(), g.data_ptr(), s.data_ptr(), o.data_ptr(),
                                                               plan.layout, plan.io, ctx.qmin, ctx.qmax,
                                                               _lib.ptr(gx), st)
                elif ctx.op == "q":
                    rc = lib.aimet_b200_quantize_backward(*common, ctx.qmin, ctx.qmax, *tail)
                elif ctx.op == "dq":
                    rc = lib.aimet_b200_dequantize_backward(*common, *tail)
                else:
                    rc = lib.aimet_b200_quantize_dequantize_backward_ex(*common, ctx.qmin, ctx.qmax, ctx.zps, ctx.pgs[0],
                                                                        ctx.pgs[1], *tail)
            _lib.check(rc)
        if gx is not None:
            gx = _restore(gx, plan, grad).to(ctx.in_dtype)
        if gs is not None:
            gs = gs.sum_to_size(ctx.scale_meta[0]).to(ctx.scale_meta[1])
        if go is not None:
            go = go.sum_to_size(ctx.offset_meta[0]).to(ctx.offset_meta[1])
        return gx, gs, go, None, None, None, None, None, None


def _normalize_block_size(block_size) -> Optional[Tuple[int, ...]]:
    if block_size is None:
        return None
    block_size = tuple(int(b) for b in block_size)
    return block_size or None


def quantize(
    input: torch.Tensor,  # pylint: disable=redefined-builtin
    scale: torch.Tensor,
    offset: torch.Tensor,
    qmin: int,
    qmax: int,
    block_size: Optional[List] = None,
) -> torch.Tensor:
    """``clamp(round(input / scale) - offset, qmin, qmax)`` as float-valued integer codes in
    ``input.dtype`` (torch_builtins.py:166-212)."""
    block_size = _normalize_block_size(block_size)
    _validate(input, scale, offset, qmin, qmax, block_size)
    qmin, qmax = int(qmin), int(qmax)
    if not _is_grid_representable(input.dtype, qmin, qmax):
        raise RuntimeError(f"{input.dtype} is unable to represent quantized output of range [{qmin}, {qmax}].")
    internal = _internal_dtype(input.dtype, qmin, qmax)
    return _apply(input, scale, offset, "q", qmin, qmax, 0.0, block_size, internal)


def dequantize(
    input: torch.Tensor,  # pylint: disable=redefined-builtin
    scale: torch.Tensor,
    offset: torch.Tensor,
    block_size: Optional[List] = None,
) -> torch.Tensor:
    """``(input + offset) * scale`` evaluated in ``input.dtype`` (torch_builtins.py:537-571)."""
    block_size = _normalize_block_size(block_size)
    _validate(input, scale, offset, block_size=block_size)
    return _apply(input, scale, offset, "dq", 0, 0, 0.0, block_size, input.dtype)


def quantize_dequantize(
    input: torch.Tensor,  # pylint: disable=redefined-builtin
    scale: torch.Tensor,
    offset: torch.Tensor,
    qmin: int,
    qmax: int,
    block_size: Optional[List] = None,
    zero_point_shift: float = 0.0,
) -> torch.Tensor:
    """Fake-quantization ``(clamp(round(input / scale - zps) - offset, qmin, qmax) + offset + zps) * scale``
    with straight-through gradients (torch_builtins.py:216-302).

    Like the reference, two arithmetics exist.  When a gradient for ``scale`` or ``offset`` may be
    needed (or for blockwise encodings, a non-zero ``zero_point_shift``, several channel axes) the
    ``QuantDequantFunc`` chain runs: true division, round-half-to-even, every step in the internal
    dtype.  Otherwise the reference calls ``torch.fake_quantize_per_tensor_affine`` /
    ``..._per_channel_affine`` (torch_builtins.py:243-266): float32, multiplication by ``1 / scale``,
    integer zero point -- and so does this backend, so results agree with the reference in both
    modes.
    """
    if torch.onnx.is_in_onnx_export():
        return input
    block_size = _normalize_block_size(block_size)
    _validate(input, scale, offset, qmin, qmax, block_size)
    qmin, qmax = int(qmin), int(qmax)
    zero_point_shift = zero_point_shift or 0.0
    if _takes_fake_quantize_path(input, scale, offset, block_size, zero_point_shift, qmin, qmax):
        return _apply(input, scale.detach(), offset.detach(), "fq", qmin, qmax, 0.0, None, torch.float32)
    internal = _internal_dtype(input.dtype, qmin, qmax)
    if not _is_grid_representable(internal, qmin, qmax):
        raise RuntimeError(f"{internal} is unable to represent quantized output of range [{qmin}, {qmax}].")
    return _apply(input, scale, offset, "qdq", qmin, qmax, zero_point_shift, block_size, internal)


def _zero_points_in_grid(offset: torch.Tensor, qmin: int, qmax: int) -> bool:
    """Whether every zero point (-offset) lies in [qmin, qmax].  torch.fake_quantize_per_channel_affine
    refuses anything else, and the reference then falls back to the QuantDequantFunc arithmetic
    (torch_builtins.py:418-425).  Offsets that a quantizer module built from a constant carry that
    constant, so the usual case (symmetric per-channel weights) is decided on the host; otherwise
    the device is asked, as ATen's own check does."""
    const = getattr(offset, "_b200_constant", None)
    if const is not None:
        return qmin <= -const <= qmax
    lo, hi = torch.aminmax(offset.detach())
    return bool((-hi >= qmin) & (-lo <= qmax))


def _takes_fake_quantize_path(tensor, scale, offset, block_size, zero_point_shift, qmin=None, qmax=None) -> bool:
    """The reference's ``_fast_forward`` test plus the tests of ``_torch_fake_quantize``
    (torch_builtins.py:243-266, 352-431): no parameter gradient wanted, not blockwise, no shift, not
    being traced by ``torch.compile``, and the parameters are per-tensor or vary along exactly one
    axis with every zero point inside the grid."""
    if block_size is not None or zero_point_shift != 0.0 or torch.jit.is_tracing():
        return False
    if torch.compiler.is_compiling():
        return False
    if torch.is_grad_enabled() and (scale.requires_grad or offset.requires_grad):
        return False
    if tensor.requires_grad and pgs.is_pgs_enabled():  # the fake-quantize arithmetic has no such gradient
        return False
    if tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return False
    if scale.numel() == 1 and offset.numel() == 1:
        return True
    if scale.dim() > tensor.dim() or offset.dim() > tensor.dim():
        return False
    sshape = (1,) * (tensor.dim() - scale.dim()) + tuple(scale.shape)
    oshape = (1,) * (tensor.dim() - offset.dim()) + tuple(offset.shape)
    if sshape != oshape or any(d not in (1, t) for d, t in zip(sshape, tensor.shape)):
        return False
    if sum(1 for d in sshape if d != 1) != 1:
        return False
    return qmin is None or _zero_points_in_grid(offset, qmin, qmax)


def quantize_dequantize_stack(input: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, qmin: int, qmax: int,  # pylint: disable=redefined-builtin
                              block_size: Optional[List] = None, zero_point_shift: float = 0.0,
                              parameter_gradients: bool = False) -> torch.Tensor:
    """``out[c] = quantize_dequantize(input, scale[c], offset[c], ...)`` for every leading index ``c``
    of the parameters, without autograd: one allocation and one launch per ``c`` on the same input
    (SeqMSE's candidate weights, seq_mse.py:544-553 of the reference, which quantizes the weight
    once per candidate).  Each slice takes the arithmetic :func:`quantize_dequantize` would take for
    it: the fake-quantize fast path unless ``parameter_gradients`` says that the caller's quantizer
    would have asked for scale / offset gradients."""
    block_size = _normalize_block_size(block_size)
    count = scale.shape[0]
    s0, o0 = scale[0].detach(), offset[0].detach()
    _validate(input, s0, o0, qmin, qmax, block_size)
    qmin, qmax = int(qmin), int(qmax)
    zero_point_shift = zero_point_shift or 0.0
    fast = (not parameter_gradients and _takes_fake_quantize_path(input, s0, o0, block_size, zero_point_shift)
            and _zero_points_in_grid(offset, qmin, qmax))
    internal = torch.float32 if fast else _internal_dtype(input.dtype, qmin, qmax)
    if not fast and not _is_grid_representable(internal, qmin, qmax):
        raise RuntimeError(f"{internal} is unable to represent quantized output of range [{qmin}, {qmax}].")
    x, plan = _prepare(input.detach(), s0, o0, None if fast else block_size, internal)
    if plan.upcast or list(plan.perm) != list(range(input.dim())):
        # rare layouts: one ordinary call per slice
        return torch.stack([quantize_dequantize(input.detach(), scale[c].detach(), offset[c].detach(), qmin, qmax,
                                                block_size, zero_point_shift) for c in range(count)])
    s_all = scale.detach().expand((count,) + plan.pshape).to(plan.pt).contiguous()
    o_all = offset.detach().expand((count,) + plan.pshape).to(plan.pt).contiguous()
    out = torch.empty((count,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    if x.numel() == 0:
        return out
    pt = _lib.DTYPE_CODE[plan.pt]
    step_y, step_p = x.numel() * x.element_size(), s_all[0].numel() * s_all.element_size()
    with _lib.on_device(x.device):
        st = _lib.stream_ptr(x.device)
        for c in range(count):
            if fast:
                rc = lib.aimet_b200_fake_quantize(x.data_ptr(), out.data_ptr() + c * step_y, s_all.data_ptr() + c * step_p,
                                                  o_all.data_ptr() + c * step_p, plan.layout, plan.io, qmin, qmax, st)
            else:
                rc = lib.aimet_b200_quantize_dequantize(x.data_ptr(), out.data_ptr() + c * step_y,
                                                        s_all.data_ptr() + c * step_p, o_all.data_ptr() + c * step_p,
                                                        plan.layout, plan.io, plan.ct, pt, qmin, qmax,
                                                        float(zero_point_shift), st)
            _lib.check(rc)
    return out
