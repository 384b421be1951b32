"""SeqMSE candidate search for Linear and Conv2d layers on the tcgen05 reconstruction-loss kernel.

Host-side mirror of aimet_torch's ``seq_mse.py`` / ``_base/seq_mse.py``:
``SeqMseParams`` (_base/seq_mse.py:50-82), ``SequentialMse.optimize_module`` (seq_mse.py:523-578),
``_get_candidate`` (:360-372), ``compute_param_encodings`` (:263-294), ``_compute_loss`` (:375-401),
``_compute_linear_loss`` (:403-482), ``_compute_conv_loss`` (:485-520) and
``_freeze_quantizer_encoding`` (:301-305).  The reference evaluates one candidate at a time with
two matmuls (or convolutions, one pair per block) and three elementwise passes each; here the
weight is quantized under all candidates first and one kernel launch per calibration batch returns
the loss of every candidate, output channel and input-channel block
(``aimet_b200_seqmse_linear_loss_blocks``), computing ``x @ w.T`` once per tile.  A convolution is
handed to the same kernel as a matrix product over its unfolded input.

bfloat16 / float16 operands go to the tensor cores as they are.  float32 operands are rewritten as
differences and split into three bfloat16 terms each (see :func:`block_losses_all_candidates`),
which keeps float32-level accuracy on the same kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
from torch import nn

from . import _lib, backend
from ._lib import lib
from .encoding_analyzer import _div
from .quantizer import AffineQuantizerBase, QuantizeDequantize

__all__ = ["SeqMseParams", "SequentialMse", "QuantizedLinear", "QuantizedConv2d", "optimize_module"]

_LOSS_KIND = {"mse": 0, "l1": 1, "sqnr": 2}


def default_forward_fn(model, inputs):
    if isinstance(inputs, torch.Tensor):
        return model(inputs)
    return model(*inputs)


@dataclass
class SeqMseParams:
    """Search parameters (_base/seq_mse.py:50-82).  ``precise_loss`` is specific to this backend:
    True accumulates the loss in float32; False re-rounds products and loss terms to the operand
    dtype the way the reference's half-precision aten chain does."""

    num_batches: Optional[int]
    num_candidates: int = 20
    inp_symmetry: str = "symqt"
    loss_fn: str = "mse"
    forward_fn: Callable = default_forward_fn
    precise_loss: bool = True

    def __post_init__(self):
        if self.loss_fn not in _LOSS_KIND:
            raise ValueError(f"Invalid loss function: {self.loss_fn}")

    def get_loss_fn(self) -> str:
        return self.loss_fn


class QuantizedLinear(nn.Linear):
    """A Linear layer carrying a weight quantizer in ``param_quantizers["weight"]`` -- the part of the
    reference's quantized-module interface (nn/base.py) the candidate search touches."""

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.param_quantizers = nn.ModuleDict({"weight": None})

    def forward(self, input):  # pylint: disable=redefined-builtin
        q = self.param_quantizers["weight"]
        w = self.weight if q is None else q(self.weight)
        return nn.functional.linear(input, w, self.bias)


class QuantizedConv2d(nn.Conv2d):
    """A Conv2d layer carrying a weight quantizer in ``param_quantizers["weight"]``."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.param_quantizers = nn.ModuleDict({"weight": None})

    def forward(self, input):  # pylint: disable=redefined-builtin
        q = self.param_quantizers["weight"]
        w = self.weight if q is None else q(self.weight)
        return self._conv_forward(input, w, self.bias)


def _split_bf16x3(t: torch.Tensor):
    """float32 -> three bfloat16 terms whose sum is the input (to 24 significant bits)."""
    t1 = t.to(torch.bfloat16)
    r1 = t - t1.float()
    t2 = r1.to(torch.bfloat16)
    t3 = (r1 - t2.float()).to(torch.bfloat16)
    return t1, t2, t3


def _expand_fp32(t: torch.Tensor, num_blocks: int, lhs: bool) -> torch.Tensor:
    """[.., K] float32 -> [.., 6K] bfloat16, block by block.  A left operand expanded with
    ``lhs=True`` against a right operand expanded with ``lhs=False`` makes the bfloat16 contraction
    equal the float32 one up to the third-order terms of the split:
    sum_{i+j<=4} a_i . b_j = [a1 a1 a2 a1 a2 a3] . [b1 b2 b1 b3 b2 b1].
    The six terms of a block stay inside the block, so a blockwise contraction sees its own terms."""
    t1, t2, t3 = _split_bf16x3(t)
    terms = (t1, t1, t2, t1, t2, t3) if lhs else (t1, t2, t1, t3, t2, t1)
    k = t.shape[-1]
    kb = k // num_blocks
    parts = [u.reshape(*u.shape[:-1], num_blocks, 1, kb) for u in terms]
    return torch.cat(parts, dim=-2).reshape(*t.shape[:-1], num_blocks * 6 * kb)


def _interleave_blocks(a: torch.Tensor, b: torch.Tensor, num_blocks: int) -> torch.Tensor:
    """Concatenate two operands along K block by block: [.., nb, Ka] + [.., nb, Kb] -> [.., nb*(Ka+Kb)]."""
    ka, kb = a.shape[-1] // num_blocks, b.shape[-1] // num_blocks
    a = a.reshape(*a.shape[:-1], num_blocks, ka)
    b = b.reshape(*b.shape[:-1], num_blocks, kb)
    return torch.cat([a, b], dim=-1).reshape(*a.shape[:-2], num_blocks * (ka + kb))


def _pad_blocks(t: torch.Tensor, num_blocks: int, multiple: int) -> torch.Tensor:
    """Zero-pad the columns of every block up to a multiple of ``multiple``."""
    kb = t.shape[-1] // num_blocks
    pad = (-kb) % multiple
    if pad == 0:
        return t
    t = nn.functional.pad(t.reshape(*t.shape[:-1], num_blocks, kb), (0, pad))
    return t.reshape(*t.shape[:-2], num_blocks * (kb + pad))


def _raise_on_status(status: torch.Tensor):
    code = int(status.max().item())
    if code != 0:
        raise RuntimeError(f"aimet_b200: the SeqMSE kernel gave up waiting (device status {code})")


def _launch(x, xq, w, wq_all, num_blocks, kind, lowp, has_ref, status_sink):
    """One kernel launch: float32 [C, N, num_blocks, nvals]."""
    c, n, k = wq_all.shape
    m = xq.shape[0]
    multiple = 16 if num_blocks > 1 else 8
    if (k // num_blocks) % multiple:
        xq, wq_all = _pad_blocks(xq, num_blocks, multiple), _pad_blocks(wq_all, num_blocks, multiple)
        if has_ref:
            x, w = _pad_blocks(x, num_blocks, multiple), _pad_blocks(w, num_blocks, multiple)
        k = xq.shape[1]
    xq, wq_all = xq.contiguous(), wq_all.contiguous()
    if has_ref:
        x, w = (xq if x is xq else x.contiguous()), w.contiguous()
    dev = xq.device
    nvals = 2 if kind >= 2 else 1
    out = torch.empty((c, n, num_blocks, nvals), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    with _lib.on_device(dev):
        nbytes = lib.aimet_b200_seqmse_blocks_scratch_bytes(m, n, k, num_blocks, c)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(dev, nbytes)
        rc = lib.aimet_b200_seqmse_linear_loss_blocks(
            x.data_ptr() if has_ref else None, xq.data_ptr(), w.data_ptr() if has_ref else None, wq_all.data_ptr(),
            m, n, k, num_blocks, c, _lib.DTYPE_CODE[xq.dtype], kind, int(lowp), int(has_ref), out.data_ptr(),
            status.data_ptr(), scratch.data_ptr(), scratch.numel(), _lib.stream_ptr(dev))
    _lib.check(rc)
    if status_sink is None:
        _raise_on_status(status)  # reads the kernel's status word: synchronises with the device
    else:
        status_sink.append(status)  # the caller checks all its launches at once
    return out


def block_losses_all_candidates(x, xq, w, wq_all, num_blocks: int = 1, loss_fn: str = "mse", lowp: bool = False,
                                status_sink: Optional[list] = None, signal: str = "quantized") -> torch.Tensor:
    """Loss of every candidate, output channel and input-channel block for one batch of tokens.

    x, xq: [tokens, K]; w: [N, K]; wq_all: [C, N, K]; block b covers columns
    [b * K / num_blocks, (b + 1) * K / num_blocks).  Returns float32 [C, N, num_blocks]:
    ``mse``: sum_m (x.w - xq.wq_c)^2, ``l1``: sum_m |x.w - xq.wq_c|, ``sqnr``: the reference's negative
    SQNR in dB whose signal is ``xq.wq_c`` (``signal="quantized"``: the Linear path,
    seq_mse.py:440-454) or ``x.w`` (``signal="original"``: the Conv2d path,
    _base/seq_mse.py:705-720).

    bfloat16 / float16 operands go to the tensor cores as they are.  float32 operands are handed
    over as differences, ``x.w - xq.wq = xq.(w - wq) + (x - xq).w``, every factor split into three
    bfloat16 terms: the two nearly equal products are never formed, so nothing cancels and the loss
    keeps float32 accuracy.
    ``status_sink``: a list that receives the launch's device status word instead of it being read
    back (and the host waiting) here; the caller then checks all its launches with one read.
    """
    if not x.is_cuda:
        raise RuntimeError("aimet_b200 SeqMSE runs on CUDA tensors only; there is no CPU fallback.")
    kind = _LOSS_KIND[loss_fn]
    m = x.shape[0]
    same = xq is x or (xq.data_ptr() == x.data_ptr() and xq.shape == x.shape and xq.stride() == x.stride())
    if x.dtype == torch.float32:
        dw = w.unsqueeze(0) - wq_all
        lhs = _expand_fp32(xq, num_blocks, True)
        rhs = _expand_fp32(dw, num_blocks, False)
        if not same:
            lhs = _interleave_blocks(lhs, _expand_fp32(x - xq, num_blocks, True), num_blocks)
            rhs = _interleave_blocks(rhs, _expand_fp32(w, num_blocks, False).unsqueeze(0).expand(rhs.shape[0], -1, -1),
                                     num_blocks)
        noise = _launch(None, lhs, None, rhs, num_blocks, 1 if kind == 1 else 0, False, False, status_sink)[..., 0]
        if kind != 2:
            return noise
        if signal == "quantized":
            sig = _launch(None, _expand_fp32(xq, num_blocks, True), None, _expand_fp32(wq_all, num_blocks, False),
                          num_blocks, 0, False, False, status_sink)[..., 0]
        else:
            sig = _launch(None, _expand_fp32(x, num_blocks, True), None,
                          _expand_fp32(w, num_blocks, False).unsqueeze(0), num_blocks, 0, False, False,
                          status_sink)[..., 0]
    elif x.dtype in (torch.bfloat16, torch.float16):
        if kind == 2 and signal != "quantized":
            kind = 3
        out = _launch(x, x if same else xq, w, wq_all, num_blocks, kind, lowp, True, status_sink)
        if kind < 2:
            return out[..., 0]
        noise, sig = out[..., 0], out[..., 1]
    else:
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    noise = _div(noise, m) + 1e-10
    return -(10 * torch.log10(_div(sig, m) / noise))


def linear_loss_all_candidates(x, xq, w, wq_all, loss_fn: str = "mse", lowp: bool = False,
                               status_sink: Optional[list] = None) -> torch.Tensor:
    """:func:`block_losses_all_candidates` for a single block: float32 [C, N]."""
    return block_losses_all_candidates(x, xq, w, wq_all, 1, loss_fn, lowp, status_sink)[..., 0]


class SequentialMse:
    """Layer-wise search for the weight encodings that minimise the reconstruction error of the
    layer output (all classmethods, like the reference)."""

    inp_symmetry: str = "symqt"
    loss_fn: str = "mse"

    @classmethod
    def compute_param_encodings(cls, quantizer: AffineQuantizerBase, x_min: torch.Tensor, x_max: torch.Tensor):
        """Re-calibrate ``quantizer`` on the range [x_min, x_max] (seq_mse.py:263-294)."""
        probe = QuantizeDequantize(quantizer.shape, quantizer.bitwidth, quantizer.symmetric,
                                   block_size=quantizer.block_size,
                                   zero_point_shift=quantizer.zero_point_shift).to(x_min.device)
        lo, hi = x_min, x_max
        if quantizer.block_size:
            for axis, blk in enumerate(quantizer.block_size):
                if blk == -1:
                    continue
                lo = lo.repeat_interleave(blk, axis)
                hi = hi.repeat_interleave(blk, axis)
        with probe.compute_encodings():
            probe(torch.stack([lo, hi]))
        quantizer.set_range(probe.min, probe.max)

    @classmethod
    def _candidate_encodings(cls, quantizer: AffineQuantizerBase, x_min: torch.Tensor, x_max: torch.Tensor):
        """The (min, max) that :meth:`compute_param_encodings` would set, computed with a handful of
        tensor ops instead of a throw-away quantizer: the min-max statistics of the stacked pair
        (x_min, x_max) reduced to the quantizer's shape, then the min-max analyzer's range rule."""
        from .encoding_analyzer import MinMaxEncodingAnalyzer, _MinMaxRange

        shape = tuple(quantizer.shape)
        lo, hi = torch.minimum(x_min, x_max), torch.maximum(x_min, x_max)
        lo, hi = torch.broadcast_tensors(lo, hi)
        pad = (1,) * (lo.dim() - len(shape)) + shape
        dims = tuple(d for d, (have, want) in enumerate(zip(lo.shape, pad)) if have != want)
        if dims:
            lo, hi = lo.amin(dims, keepdim=True), hi.amax(dims, keepdim=True)
        lo, hi = lo.reshape(shape), hi.reshape(shape)
        steps = quantizer.qmax - quantizer.qmin - (1 if quantizer.zero_point_shift == 0.5 else 0)
        return MinMaxEncodingAnalyzer(shape).compute_encodings_from_stats(_MinMaxRange(lo, hi), steps, quantizer.symmetric)

    @classmethod
    def _all_candidate_weights(cls, quantizer: AffineQuantizerBase, w: torch.Tensor, min_t, max_t, num_candidates: int):
        """The weight quantize-dequantized under every candidate range, [C, out, in]: the candidates'
        ranges are formed with the same element-wise operations as :meth:`_get_candidate` /
        :meth:`_candidate_encodings` (a leading candidate dimension added), a quantizer of shape
        (C, *shape) turns them into scales and offsets, and one launch per candidate writes its
        slice of the result from the one weight (the reference quantizes the weight once per
        candidate too, seq_mse.py:544-553; nothing is repeated or copied here)."""
        from .encoding_analyzer import MinMaxEncodingAnalyzer, _MinMaxRange

        c = num_candidates
        shape = tuple(quantizer.shape)
        idx = torch.arange(1, c + 1, device=w.device, dtype=min_t.dtype).reshape((c,) + (1,) * min_t.dim())
        cmax = _div(max_t, c).unsqueeze(0) * idx
        cmin = _div(min_t, c).unsqueeze(0) * idx
        lo, hi = torch.minimum(cmin, cmax), torch.maximum(cmin, cmax)
        pad = (1,) * (lo.dim() - 1 - len(shape)) + shape
        dims = tuple(d + 1 for d, (have, want) in enumerate(zip(lo.shape[1:], pad)) if have != want)
        if dims:
            lo, hi = lo.amin(dims, keepdim=True), hi.amax(dims, keepdim=True)
        wide = (c,) + (1,) * (w.dim() - len(shape)) + shape
        lo, hi = lo.reshape(wide), hi.reshape(wide)
        steps = quantizer.qmax - quantizer.qmin - (1 if quantizer.zero_point_shift == 0.5 else 0)
        lo, hi = MinMaxEncodingAnalyzer(wide).compute_encodings_from_stats(_MinMaxRange(lo, hi), steps, quantizer.symmetric)
        # scale and offset as a quantizer of shape (C, *shape) holding these ranges would derive them
        # (float32 parameters, the quantizer's own grid), without building one
        from .quantizer import _get_symmetric_offset, _offset_of_range, _scale_of_range

        with torch.no_grad():
            lo32, hi32 = lo.to(torch.float32), hi.to(torch.float32)
            scale = _scale_of_range(lo32, hi32, quantizer.qmax - quantizer.qmin, torch.float32)
            if quantizer.symmetric:
                offset = _get_symmetric_offset(quantizer.qmin, quantizer.qmax, wide, torch.float32, w.device)
            else:
                offset = _offset_of_range(lo32, scale, quantizer.qmin, quantizer.qmax, torch.float32)
        pshape = (c,) + shape  # per candidate: the quantizer's own parameter shape
        wants_grad = torch.is_grad_enabled() and any(p.requires_grad for p in quantizer.parameters())
        offsets = offset.reshape(pshape)
        const = getattr(offset, "_b200_constant", None)
        if const is not None:  # a symmetric grid: every zero point is this constant (no device round trip)
            offsets._b200_constant = const  # pylint: disable=protected-access
        return backend.quantize_dequantize_stack(w, scale.reshape(pshape), offsets, quantizer.qmin,
                                                 quantizer.qmax, quantizer.block_size, quantizer.zero_point_shift,
                                                 parameter_gradients=wants_grad)

    @classmethod
    def _freeze_quantizer_encoding(cls, quantizer):
        quantizer.requires_grad_(False)
        quantizer.allow_overwrite(False)

    @classmethod
    def _get_quantized_weight(cls, quant_module):
        return quant_module.param_quantizers["weight"].forward(quant_module.weight)

    @staticmethod
    def _get_input_channel_block_size(quant_module) -> int:
        """(seq_mse.py:316-326)"""
        if not isinstance(quant_module, (nn.Linear, nn.Conv2d)):
            raise NotImplementedError("Unsupported module type: ", type(quant_module))
        q = quant_module.param_quantizers["weight"]
        if q.block_size is None:
            return quant_module.weight.shape[1]
        return quant_module.weight.shape[1] // q.shape[1]

    @classmethod
    def get_min_and_max_for_candidate_selection(cls, quant_module) -> Tuple[torch.Tensor, torch.Tensor]:
        q = quant_module.param_quantizers["weight"]
        if type(q).get_min is AffineQuantizerBase.get_min and type(q).get_max is AffineQuantizerBase.get_max:
            # get_min() and get_max() with the scale and offset they share derived once
            scale = q.get_scale()
            if scale is not None:
                offset = q._scale_and_offset(scale, None)  # pylint: disable=protected-access
                return (scale * (offset + q.qmin + q.zero_point_shift),
                        scale * (offset + q.qmax + q.zero_point_shift))
        return q.get_min(), q.get_max()

    @classmethod
    def _get_candidate(cls, candidate_idx, num_candidates: int, min_tensor, max_tensor):
        """Candidate i keeps (i + 1) / num_candidates of the range; the division comes first
        (seq_mse.py:360-372), which matters in the last bit."""
        cand_max = _div(max_tensor, num_candidates) * (candidate_idx + 1)
        cand_min = _div(min_tensor, num_candidates) * (candidate_idx + 1)
        return cand_min, cand_max

    @classmethod
    def _compute_loss(cls, quant_module, x, xq, w, wq, params: SeqMseParams) -> torch.Tensor:
        """Single-candidate loss with the reference's signature (seq_mse.py:375-401)."""
        block_size = cls._get_input_channel_block_size(quant_module)
        if isinstance(quant_module, nn.Linear):
            return cls._compute_linear_loss(x, xq, w, wq, block_size, params)
        if isinstance(quant_module, nn.Conv2d):
            return cls._compute_conv_loss(quant_module, x, xq, w, wq, block_size, params)
        raise TypeError(f"Unsupported module type: {type(quant_module)}")

    @classmethod
    def _compute_linear_loss(cls, x, xq, w, wq, block_size: int, params: SeqMseParams) -> torch.Tensor:
        """Single-candidate form with the reference's signature -> [C_out, num_blocks] in x.dtype
        (seq_mse.py:403-482); all blocks in one launch."""
        in_ch = w.shape[1]
        lowp = not params.precise_loss and x.dtype != torch.float32
        loss = block_losses_all_candidates(x.reshape(-1, in_ch), xq.reshape(-1, in_ch), w, wq[None],
                                           in_ch // block_size, params.loss_fn, lowp)
        return loss[0].to(x.dtype)

    @staticmethod
    def _conv_columns(quant_module: nn.Conv2d, x: torch.Tensor, block_size: int, num_blocks: int, group: int):
        """The input of one group's convolution as a matrix (im2col): rows = output positions, columns =
        (input channel, kernel row, kernel column), the order ``w.reshape(out, -1)`` has.  The
        reference cuts the input channels of ``x`` into pieces of ``block_size * groups`` and lets
        group j of piece b see channels [j * block_size, (j + 1) * block_size) of the piece
        (seq_mse.py:504-520); the columns of the blocks are laid side by side accordingly."""
        groups = quant_module.groups
        if groups > 1:
            ch = (torch.arange(num_blocks, device=x.device)[:, None] * (block_size * groups) + group * block_size
                  + torch.arange(block_size, device=x.device)[None, :]).flatten()
            x = x.index_select(-3, ch)
        cols = nn.functional.unfold(x.reshape(-1, *x.shape[-3:]), quant_module.kernel_size, dilation=quant_module.dilation,
                                    padding=quant_module.padding, stride=quant_module.stride)
        return cols.transpose(1, 2).reshape(-1, cols.shape[1])

    @classmethod
    def _conv_losses_all_candidates(cls, quant_module, x, xq, w, wq_all, block_size: int, params: SeqMseParams,
                                    lowp: bool, pending: Optional[list]) -> torch.Tensor:
        """float32 [C, out, num_blocks] for one batch: the im2col form of the reference's per-block
        convolutions (seq_mse.py:485-520), one launch per group."""
        if isinstance(quant_module.padding, str) or quant_module.padding_mode != "zeros":
            raise NotImplementedError("the B200 SeqMSE path covers Conv2d layers with explicit zero padding")
        nb = w.shape[1] // block_size
        c, out_ch = wq_all.shape[0], w.shape[0]
        per_group = out_ch // quant_module.groups
        same = xq is x or (xq.data_ptr() == x.data_ptr() and xq.shape == x.shape)
        parts = []
        for g in range(quant_module.groups):
            rows = slice(g * per_group, (g + 1) * per_group)
            x2 = cls._conv_columns(quant_module, x, block_size, nb, g)
            xq2 = x2 if same else cls._conv_columns(quant_module, xq, block_size, nb, g)
            parts.append(block_losses_all_candidates(x2, xq2, w[rows].reshape(per_group, -1),
                                                     wq_all[:, rows].reshape(c, per_group, -1), nb, params.loss_fn,
                                                     lowp, pending, signal="original"))
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)

    @classmethod
    def _compute_conv_loss(cls, quant_module, x, xq, w, wq, block_size: int, params: SeqMseParams) -> torch.Tensor:
        """Single-candidate form with the reference's signature -> [C_out, num_blocks] in x.dtype."""
        lowp = not params.precise_loss and x.dtype != torch.float32
        return cls._conv_losses_all_candidates(quant_module, x, xq, w, wq[None], block_size, params, lowp, None)[0].to(x.dtype)

    @classmethod
    def optimize_module(cls, quant_module, x: torch.Tensor, xq: torch.Tensor, params: SeqMseParams):
        """Pick, per output channel (and block), the candidate range with the lowest reconstruction
        loss, set it on the weight quantizer and freeze it (seq_mse.py:523-578).  ``x`` / ``xq`` are
        iterated over their first dimension as calibration batches."""
        if not isinstance(quant_module, (nn.Linear, nn.Conv2d)):
            raise NotImplementedError("the B200 SeqMSE path covers Linear and Conv2d layers")
        qtz = quant_module.param_quantizers["weight"]
        block = cls._get_input_channel_block_size(quant_module)
        min_t, max_t = cls.get_min_and_max_for_candidate_selection(quant_module)
        min_t, max_t = min_t.detach(), max_t.detach()
        w = quant_module.weight.detach()
        in_ch = w.shape[1]
        nb = in_ch // block
        c = params.num_candidates

        if type(qtz) is QuantizeDequantize:  # pylint: disable=unidiomatic-typecheck
            wq_all = cls._all_candidate_weights(qtz, w, min_t, max_t, c)
        else:  # quantizers that derive their scale in their own way (LPBQ): one candidate at a time
            wq_all = torch.empty((c, *w.shape), dtype=w.dtype, device=w.device)
            for i in range(c):
                cmin, cmax = cls._get_candidate(i, c, min_t, max_t)
                qtz.set_range(*cls._candidate_encodings(qtz, cmin, cmax))
                wq_all[i].copy_(cls._get_quantized_weight(quant_module).detach())

        lowp = not params.precise_loss and w.dtype != torch.float32
        total = None
        pending = []  # status words of the launches below, read back once
        with torch.no_grad():
            for b, (bx, bxq) in enumerate(zip(x, xq)):
                if params.num_batches and b >= params.num_batches:
                    break
                if isinstance(quant_module, nn.Conv2d):
                    loss = cls._conv_losses_all_candidates(quant_module, bx, bxq, w, wq_all, block, params, lowp, pending)
                else:
                    bx2, bxq2 = bx.reshape(-1, in_ch), bxq.reshape(-1, in_ch)
                    same = bxq is bx or (bxq.data_ptr() == bx.data_ptr() and bxq.shape == bx.shape)
                    loss = block_losses_all_candidates(bx2, bx2 if same else bxq2, w, wq_all, nb, params.loss_fn, lowp,
                                                       pending)  # [C, out, nb] float32
                if lowp:
                    loss = loss.to(w.dtype)
                total = loss if total is None else total + loss
        if pending:
            _raise_on_status(torch.cat(pending))
        cls.last_losses = total  # kept for inspection by tests and tools
        best = total.min(0)[1]
        while best.dim() < max_t.dim():
            best = best[..., None]
        bmin, bmax = cls._get_candidate(best, c, min_t, max_t)
        qtz.set_range(*cls._candidate_encodings(qtz, bmin, bmax))
        cls._freeze_quantizer_encoding(qtz)
        return best


optimize_module = SequentialMse.optimize_module
