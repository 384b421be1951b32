"""Oracle for the affine functionals: forward values and hand-derived gradients.

Restates quantization/affine/backends/torch_builtins.py: dtype rules (:49-116), blockwise
reshape (:283-289), QuantizeFunc (:588-659), DequantizeFunc (:662-701), QuantDequantFunc
(:705-831).  Gradients are written out explicitly and summed down to the parameter shape in the
internal dtype, which is what autograd's sum-to-size does to the full-size tensors the reference
returns.  Test infrastructure only.
"""

from __future__ import annotations

import itertools
from typing import Optional, Sequence, Tuple

import torch

_MANTISSA = {torch.float32: 23, torch.float16: 10, torch.bfloat16: 7, torch.float64: 52}


def value_representable(dtype: torch.dtype, value: int) -> bool:
    """torch_builtins.py:49-84"""
    fi = torch.finfo(dtype)
    if not fi.min <= value <= fi.max:
        return False
    msb = max(0, value.bit_length() - 1)
    lsb = max(0, (value & -value).bit_length() - 1)
    return msb - lsb <= _MANTISSA[dtype]


def grid_representable(dtype, qmin, qmax) -> bool:
    """torch_builtins.py:87-97"""
    return all(value_representable(dtype, v) for v in (qmax, qmax - 1, qmin + 1, qmin))


def numerically_stable(dtype, qmin, qmax) -> bool:
    """torch_builtins.py:99-116"""
    if not grid_representable(dtype, qmin, qmax):
        return False
    if qmin == qmax:
        return True
    return not torch.finfo(dtype).eps > 0.25 / (qmax - qmin)


def internal_dtype(dtype, qmin, qmax) -> torch.dtype:
    """torch_builtins.py:268-277"""
    for cand in (dtype, torch.float32):
        if numerically_stable(cand, qmin, qmax):
            return cand
    return torch.float64


def _interleave(a: Sequence[int], b) -> Tuple[int, ...]:
    if isinstance(b, int):
        b = [b] * len(a)
    return tuple(itertools.chain.from_iterable(zip(a, b)))


def concrete_blocks(in_shape, p_shape, block_size) -> Tuple[int, ...]:
    """quantization/_utils.py:30-63"""
    in_shape = tuple(in_shape)[-len(p_shape):] if len(p_shape) else ()
    k = len(p_shape) - len(block_size)
    block_size = [*(1 if d > 1 else -1 for d in p_shape[:k]), *block_size]
    return tuple(b if b != -1 else in_shape[i] // p_shape[i] for i, b in enumerate(block_size))


def _blocked(x, scale, offset, block_size):
    """Bring (x, scale, offset) to broadcastable shapes (torch_builtins.py:283-289)."""
    if block_size:
        blocks = concrete_blocks(x.shape, scale.shape, block_size)
        x = x.reshape(-1, *_interleave(scale.shape, blocks))
        scale = scale.reshape(_interleave(scale.shape, 1))
        offset = offset.reshape(_interleave(offset.shape, 1))
    return x, scale, offset


def _sum_to(t: torch.Tensor, shape) -> torch.Tensor:
    return t.sum_to_size(shape) if tuple(t.shape) != tuple(shape) else t


def quantize(x, scale, offset, qmin, qmax, block_size=None):
    """QuantizeFunc.forward (torch_builtins.py:604-633)"""
    idt = internal_dtype(x.dtype, qmin, qmax)
    shape = x.shape
    xb, s, o = _blocked(x, scale, offset, block_size)
    s, o = s.to(idt), o.to(idt)
    r = torch.round(xb.to(idt) / s) - o
    return r.clamp(qmin, qmax).to(x.dtype).view(shape)


def dequantize(x, scale, offset, block_size=None):
    """DequantizeFunc.forward (torch_builtins.py:675-685)"""
    shape = x.shape
    xb, s, o = _blocked(x, scale, offset, block_size)
    s, o = s.to(x.dtype), o.to(x.dtype)
    return ((xb + o) * s).to(x.dtype).view(shape)


def quantize_dequantize(x, scale, offset, qmin, qmax, block_size=None, zero_point_shift=0.0):
    """QuantDequantFunc.forward (torch_builtins.py:722-746): the path taken whenever gradients of
    scale/offset are needed, and the one the CUDA kernels follow in every mode."""
    idt = internal_dtype(x.dtype, qmin, qmax)
    shape = x.shape
    xb, s, o = _blocked(x, scale, offset, block_size)
    s, o = s.to(idt), o.to(idt)
    t = xb.to(idt) / s
    if zero_point_shift != 0:
        t = t - zero_point_shift
    t = torch.round(t) - o
    t = t.clamp(qmin, qmax)
    t = t + (o if zero_point_shift == 0 else o + zero_point_shift)
    return (t * s).to(x.dtype).view(shape)


def quantize_dequantize_backward(x, grad, scale, offset, qmin, qmax, block_size=None, zero_point_shift=0.0,
                                 pgs_eps=0.0, pgs_multiplier=1.0):
    """QuantDequantFunc.backward (torch_builtins.py:772-831) followed by the sum-to-size autograd
    applies.  Returns (grad_x in x.dtype, grad_scale, grad_offset in the parameters' dtypes).
    ``pgs_eps`` / ``pgs_multiplier``: the experimental gradient multiplier near rounding boundaries
    (:790-821), applied in the gradient's own dtype."""
    idt = internal_dtype(x.dtype, qmin, qmax)
    shape = x.shape
    xb, s0, o0 = _blocked(x, scale, offset, block_size)
    gb = grad.reshape(xb.shape).to(idt)
    s, o = s0.to(idt), o0.to(idt)
    xs = xb.to(idt) / s
    fwd = xs - zero_point_shift if zero_point_shift != 0 else xs
    mask = ((torch.round(fwd) - o) >= qmin) & ((torch.round(fwd) - o) <= qmax)
    xs = xs - zero_point_shift
    xr = torch.round(xs)
    err = xr - xs
    xc = torch.clamp(xr, o + qmin, o + qmax)
    if zero_point_shift != 0.0:
        xc = xc + zero_point_shift
    gs_full = gb * torch.where(mask, err, xc)
    go_full = torch.where(mask, torch.zeros((), dtype=idt), gb * s)
    if pgs_eps > 0.0 and pgs_multiplier != 1.0:
        g_in = grad.reshape(xb.shape)
        near = err.abs() > (1 - pgs_eps) / 2
        g_in = torch.where(near, g_in * pgs_multiplier, g_in)
        gx = torch.where(mask, g_in, torch.zeros((), dtype=g_in.dtype)).to(x.dtype).view(shape)
    else:
        gx = torch.where(mask, gb, torch.zeros((), dtype=idt)).to(x.dtype).view(shape)
    gs = _sum_to(gs_full, s.shape).to(scale.dtype).view(scale.shape)
    go = _sum_to(go_full, o.shape).to(offset.dtype).view(offset.shape)
    return gx, gs, go


def quantize_backward(x, grad, scale, offset, qmin, qmax, block_size=None):
    """QuantizeFunc.backward (torch_builtins.py:637-659)"""
    idt = internal_dtype(x.dtype, qmin, qmax)
    shape = x.shape
    xb, s0, o0 = _blocked(x, scale, offset, block_size)
    gb = grad.reshape(xb.shape).to(idt)
    s, o = s0.to(idt), o0.to(idt)
    xs = xb.to(idt) / s
    r = torch.round(xs) - o
    mask = (r >= qmin) & (r <= qmax)
    mg = gb * mask
    gx_full = mg / s
    gs_full = -(mg / s) * xs
    go_full = -mg
    gx = gx_full.to(x.dtype).view(shape)
    gs = _sum_to(gs_full, s.shape).to(scale.dtype).view(scale.shape)
    go = _sum_to(go_full.expand(xb.shape), o.shape).to(offset.dtype).view(offset.shape)
    return gx, gs, go


def dequantize_backward(x, grad, scale, offset, block_size=None):
    """DequantizeFunc.backward (torch_builtins.py:689-701)"""
    shape = x.shape
    xb, s0, o0 = _blocked(x, scale, offset, block_size)
    gb = grad.reshape(xb.shape).to(x.dtype)
    s, o = s0.to(x.dtype), o0.to(x.dtype)
    gx_full = gb * s
    gs_full = gb * (xb + o)
    gx = gx_full.to(x.dtype).view(shape)
    gs = _sum_to(gs_full, s.shape).to(scale.dtype).view(scale.shape)
    go = _sum_to(gx_full, o.shape).to(offset.dtype).view(offset.shape)
    return gx, gs, go


def takes_fake_quantize_path(x, scale, offset, block_size=None, zero_point_shift=0.0, param_grads=False) -> bool:
    """The reference's fast-path test (torch_builtins.py:243-266 and the shape tests of
    _torch_fake_quantize :352-431)."""
    if block_size is not None or zero_point_shift != 0.0 or param_grads:
        return False
    if scale.numel() == 1 and offset.numel() == 1:
        return True
    if scale.dim() > x.dim():
        return False
    sshape = (1,) * (x.dim() - scale.dim()) + tuple(scale.shape)
    oshape = (1,) * (x.dim() - offset.dim()) + tuple(offset.shape)
    if sshape != oshape or any(d not in (1, t) for d, t in zip(sshape, x.shape)):
        return False
    return sum(1 for d in sshape if d != 1) == 1


def fake_quantize(x, scale, offset, qmin, qmax):
    """_torch_fake_quantize (torch_builtins.py:335-431): the reference hands the work to
    torch.fake_quantize_per_tensor_affine / torch.fake_quantize_per_channel_affine with a float32
    scale and the int32 zero point -offset.  Those ATen kernels evaluate, in float32,
        out = (clamp(nearbyint(x * (1 / scale)) + zp, qmin, qmax) - zp) * scale
    which is the formula the CUDA kernel implements; the oracle calls the same ATen function."""
    s = scale.to(torch.float32)
    zp = -offset.to(torch.int32)
    if scale.numel() == 1:
        return torch.fake_quantize_per_tensor_affine(x, s.reshape(()), zp.reshape(()), qmin, qmax)
    sshape = (1,) * (x.dim() - scale.dim()) + tuple(scale.shape)
    axis = [a for a, d in enumerate(sshape) if d != 1][0]
    return torch.fake_quantize_per_channel_affine(x, s.flatten(), zp.flatten(), axis, qmin, qmax)


def fake_quantize_formula(x, scale, offset, qmin, qmax):
    """The same arithmetic written out (float32, parameters broadcast against x)."""
    s = scale.to(torch.float32)
    zp = (-offset.to(torch.int32)).to(torch.float32)
    inv = 1.0 / s
    q = torch.round(x.to(torch.float32) * inv) + zp
    q = torch.where(q.isnan(), torch.zeros_like(q), q)
    return ((q.clamp(qmin, qmax) - zp) * s).to(x.dtype)


def fake_quantize_backward(x, grad, scale, offset, qmin, qmax):
    """Backward of the ATen fake-quantize ops: grad where the integer code is inside the grid."""
    s = scale.to(torch.float32)
    zp = (-offset.to(torch.int32)).to(torch.float32)
    q = torch.round(x.to(torch.float32) * (1.0 / s)) + zp
    q = torch.where(q.isnan(), torch.zeros_like(q), q)
    return torch.where((q >= qmin) & (q <= qmax), grad, torch.zeros_like(grad))
