"""SeqMSE candidate search for Linear layers on the tcgen05 reconstruction-loss kernel.

Host-side mirror of aimet_torch's ``seq_mse.py`` / ``_base/seq_mse.py`` for the Linear case:
``SeqMseParams`` (_base/seq_mse.py:50-82), ``SequentialMse.optimize_module`` (seq_mse.py:523-578),
``_get_candidate`` (:360-372), ``compute_param_encodings`` (:263-294), ``_compute_linear_loss``
(:403-482) and ``_freeze_quantizer_encoding`` (:301-305).  The reference evaluates one candidate at
a time with two matmuls and three elementwise passes each; here the weight is quantized under all
candidates first and one kernel launch per calibration batch returns the loss of every candidate
and output channel (``aimet_b200_seqmse_linear_loss``), computing ``x @ w.T`` once per tile.

bfloat16 / float16 operands go to the tensor cores as they are.  float32 operands are split into
three bfloat16 terms each and the six significant cross products are laid side by side along the
contraction dimension, which keeps float32-level accuracy on the same kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
from torch import nn

from . import _lib
from ._lib import lib
from .encoding_analyzer import _div
from .quantizer import AffineQuantizerBase, QuantizeDequantize

__all__ = ["SeqMseParams", "SequentialMse", "QuantizedLinear", "optimize_module"]

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


def _split_bf16x3(t: torch.Tensor):
    """float32 -> three bfloat16 terms whose sum is the input (to 24 significant bits)."""
    t1 = t.to(torch.bfloat16)
    r1 = t - t1.float()
    t2 = r1.to(torch.bfloat16)
    t3 = (r1 - t2.float()).to(torch.bfloat16)
    return t1, t2, t3


def _expand_fp32_lhs(x: torch.Tensor) -> torch.Tensor:
    """[.., K] float32 -> [.., 6K] bfloat16.  Together with :func:`_expand_fp32_rhs` the bfloat16
    contraction equals the float32 one up to the dropped third-order terms:
    sum_{i+j<=4} x_i . w_j = [x1 x1 x2 x1 x2 x3] . [w1 w2 w1 w3 w2 w1]."""
    x1, x2, x3 = _split_bf16x3(x)
    return torch.cat([x1, x1, x2, x1, x2, x3], dim=-1).contiguous()


def _expand_fp32_rhs(w: torch.Tensor) -> torch.Tensor:
    w1, w2, w3 = _split_bf16x3(w)
    return torch.cat([w1, w2, w1, w3, w2, w1], dim=-1).contiguous()


def _raise_on_status(status: torch.Tensor):
    code = int(status.max().item())
    if code != 0:
        raise RuntimeError(f"aimet_b200: the SeqMSE kernel gave up waiting (device status {code})")


def linear_loss_all_candidates(x, xq, w, wq_all, loss_fn: str = "mse", lowp: bool = False,
                               status_sink: Optional[list] = None) -> torch.Tensor:
    """Loss of every candidate and output channel for one batch of tokens.

    x, xq: [tokens, K]; w: [N, K]; wq_all: [C, N, K].  Returns float32 [C, N]:
    ``mse``: sum_m (x.w - xq.wq_c)^2, ``l1``: sum_m |x.w - xq.wq_c|, ``sqnr``: the reference's negative
    SQNR in dB with ``xq.wq_c`` as the signal (seq_mse.py:440-454 passes (xw, xqwq) in that order).
    ``status_sink``: a list that receives the launch's device status word instead of it being read
    back (and the host waiting) here; the caller then checks all its launches with one read.
    """
    if not x.is_cuda:
        raise RuntimeError("aimet_b200 SeqMSE runs on CUDA tensors only; there is no CPU fallback.")
    kind = _LOSS_KIND[loss_fn]
    c, n, k = wq_all.shape
    m = x.shape[0]
    if x.dtype == torch.float32:
        xe = _expand_fp32_lhs(x)
        xqe = xe if xq is x else _expand_fp32_lhs(xq)
        x, xq, w, wq_all, lowp = xe, xqe, _expand_fp32_rhs(w), _expand_fp32_rhs(wq_all), False
        k = x.shape[1]
    elif x.dtype in (torch.bfloat16, torch.float16):
        x, xq, w, wq_all = x.contiguous(), xq.contiguous(), w.contiguous(), wq_all.contiguous()
    else:
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    if k % 8 != 0:
        pad = 8 - k % 8
        x, xq, w = (nn.functional.pad(t, (0, pad)) for t in (x, xq, w))
        wq_all = nn.functional.pad(wq_all, (0, pad))
        k += pad
    dev = x.device
    nvals = 2 if kind == 2 else 1
    out = torch.empty((c, n, nvals), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        nbytes = lib.aimet_b200_seqmse_scratch_bytes(m, n, k, c)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(dev, nbytes)
        rc = lib.aimet_b200_seqmse_linear_loss(x.data_ptr(), xq.data_ptr(), w.data_ptr(), wq_all.data_ptr(), m, n, k,
                                               c, _lib.DTYPE_CODE[x.dtype], kind, int(lowp), out.data_ptr(),
                                               status.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                               _lib.stream_ptr(dev))
    _lib.check(rc)
    if status_sink is None:
        _raise_on_status(status)  # reads the kernel's status word: synchronises with the device
    else:
        status_sink.append(status)  # the caller checks all its launches at once
    if kind == 2:
        noise = _div(out[..., 0], m) + 1e-10
        signal = _div(out[..., 1], m)
        return -(10 * torch.log10(signal / noise))
    return out[..., 0]


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
        """The weight quantize-dequantized under every candidate range, [C, out, in], with one kernel
        launch: the candidates' ranges are formed with the same element-wise operations as
        :meth:`_get_candidate` / :meth:`_candidate_encodings` (a leading candidate dimension added),
        and a quantizer of shape (C, *shape) applies them to the weight repeated along that
        dimension -- the same arithmetic per element as C separate calls."""
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
        block = None
        if quantizer.block_size:
            block = (1,) * (len(wide) - len(quantizer.block_size)) + tuple(quantizer.block_size)
        probe = QuantizeDequantize(wide, quantizer.bitwidth, quantizer.symmetric, block_size=block,
                                   zero_point_shift=quantizer.zero_point_shift).to(w.device)
        probe.signed = quantizer.signed
        probe.set_range(lo, hi)
        return probe(w.unsqueeze(0).expand((c,) + tuple(w.shape))).detach()

    @classmethod
    def _freeze_quantizer_encoding(cls, quantizer):
        quantizer.requires_grad_(False)
        quantizer.allow_overwrite(False)

    @classmethod
    def _get_quantized_weight(cls, quant_module):
        return quant_module.param_quantizers["weight"].forward(quant_module.weight)

    @staticmethod
    def _get_input_channel_block_size(quant_module) -> int:
        if not isinstance(quant_module, nn.Linear):
            raise NotImplementedError("Unsupported module type: ", type(quant_module))
        q = quant_module.param_quantizers["weight"]
        if q.block_size is None:
            return quant_module.weight.shape[1]
        return quant_module.weight.shape[1] // q.shape[1]

    @classmethod
    def get_min_and_max_for_candidate_selection(cls, quant_module) -> Tuple[torch.Tensor, torch.Tensor]:
        q = quant_module.param_quantizers["weight"]
        return q.get_min(), q.get_max()

    @classmethod
    def _get_candidate(cls, candidate_idx, num_candidates: int, min_tensor, max_tensor):
        """Candidate i keeps (i + 1) / num_candidates of the range; the division comes first
        (seq_mse.py:360-372), which matters in the last bit."""
        cand_max = _div(max_tensor, num_candidates) * (candidate_idx + 1)
        cand_min = _div(min_tensor, num_candidates) * (candidate_idx + 1)
        return cand_min, cand_max

    @classmethod
    def _compute_linear_loss(cls, x, xq, w, wq, block_size: int, params: SeqMseParams) -> torch.Tensor:
        """Single-candidate form with the reference's signature -> [C_out, num_blocks] in x.dtype."""
        out_ch, in_ch = w.shape
        nb = in_ch // block_size
        x2, xq2 = x.reshape(-1, in_ch), xq.reshape(-1, in_ch)
        lowp = not params.precise_loss and x.dtype != torch.float32
        cols = []
        for b in range(nb):
            sl = slice(b * block_size, (b + 1) * block_size)
            loss = linear_loss_all_candidates(x2[:, sl].contiguous(), xq2[:, sl].contiguous(), w[:, sl].contiguous(),
                                              wq[None, :, sl].contiguous(), params.loss_fn, lowp)
            cols.append(loss[0])
        return torch.stack(cols, dim=-1).to(x.dtype)

    @classmethod
    def optimize_module(cls, quant_module, x: torch.Tensor, xq: torch.Tensor, params: SeqMseParams):
        """Pick, per output channel (and block), the candidate range with the lowest reconstruction
        loss, set it on the weight quantizer and freeze it (seq_mse.py:523-578).  ``x`` / ``xq`` are
        iterated over their first dimension as calibration batches."""
        if not isinstance(quant_module, nn.Linear):
            raise NotImplementedError("the B200 SeqMSE path covers Linear layers")
        qtz = quant_module.param_quantizers["weight"]
        block = cls._get_input_channel_block_size(quant_module)
        min_t, max_t = cls.get_min_and_max_for_candidate_selection(quant_module)
        min_t, max_t = min_t.detach(), max_t.detach()
        w = quant_module.weight.detach()
        out_ch, in_ch = w.shape
        nb = in_ch // block
        c = params.num_candidates

        if type(qtz) is QuantizeDequantize:  # pylint: disable=unidiomatic-typecheck
            wq_all = cls._all_candidate_weights(qtz, w, min_t, max_t, c)
        else:  # quantizers that derive their scale in their own way (LPBQ): one candidate at a time
            wq_all = torch.empty((c, out_ch, in_ch), dtype=w.dtype, device=w.device)
            for i in range(c):
                cmin, cmax = cls._get_candidate(i, c, min_t, max_t)
                qtz.set_range(*cls._candidate_encodings(qtz, cmin, cmax))
                wq_all[i].copy_(cls._get_quantized_weight(quant_module).detach())

        lowp = not params.precise_loss and w.dtype != torch.float32
        total = None
        pending = []  # status words of the launches below, read back once
        w_blocks = wq_blocks = None
        with torch.no_grad():
            for b, (bx, bxq) in enumerate(zip(x, xq)):
                if params.num_batches and b >= params.num_batches:
                    break
                bx2, bxq2 = bx.reshape(-1, in_ch), bxq.reshape(-1, in_ch)
                same = bxq is bx or (bxq.data_ptr() == bx.data_ptr() and bxq.shape == bx.shape)
                cols = []
                if nb > 1:
                    # block-major copies once per batch: [nb, rows, block], contiguous per block
                    xb = bx2.reshape(-1, nb, block).permute(1, 0, 2).contiguous()
                    xqb = xb if same else bxq2.reshape(-1, nb, block).permute(1, 0, 2).contiguous()
                    if w_blocks is None:
                        w_blocks = w.reshape(out_ch, nb, block).permute(1, 0, 2).contiguous()
                        wq_blocks = wq_all.reshape(c, out_ch, nb, block).permute(2, 0, 1, 3).contiguous()
                    for k in range(nb):
                        xk = xb[k]
                        cols.append(linear_loss_all_candidates(xk, xk if same else xqb[k], w_blocks[k], wq_blocks[k],
                                                               params.loss_fn, lowp, pending))
                else:
                    xs = bx2.contiguous()
                    cols.append(linear_loss_all_candidates(xs, xs if same else bxq2.contiguous(), w, wq_all,
                                                           params.loss_fn, lowp, pending))
                loss = torch.stack(cols, dim=-1)  # [C, out, nb] float32
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
