"""Oracle for the SeqMSE candidate search of a Linear or Conv2d layer (CPU, PyTorch tensor ops).

Restates seq_mse.py of the reference: candidate ranges (_get_candidate :360-372), the
re-calibration of the weight quantizer on a candidate range (compute_param_encodings :263-294),
the block-wise reconstruction loss (_compute_linear_loss :403-454, _compute_conv_loss :485-520 with
compute_outputs / compute_recon_loss of _base/seq_mse.py:705-720, 753-800) and the per-channel
arg-min (optimize_module :523-578); loss functions from _base/seq_mse.py:69-82, 872-888.
Test infrastructure only.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import affine as A
from . import encoding_analyzer as E
from . import quantizer as Q


def neg_sqnr(pred, target, eps=1e-10, reduction="none"):  # pylint: disable=unused-argument
    """_base/seq_mse.py:872-888"""
    err = target - pred
    noise = torch.mean(err**2, 0, keepdim=True) + eps
    signal = torch.mean(target**2, 0, keepdim=True)
    return -(10 * torch.log10(signal / noise))


LOSS_FNS = {"mse": F.mse_loss, "l1": F.l1_loss, "sqnr": neg_sqnr}


def candidate(i, num_candidates, min_t, max_t):
    """_get_candidate (:360-372): note the division comes first."""
    return min_t / num_candidates * (i + 1), max_t / num_candidates * (i + 1)


def encodings_for_candidate(cand_min, cand_max, qshape, qmin, qmax, symmetric, zero_point_shift=0.0):
    """compute_param_encodings (:263-294): a fresh min-max calibration, with the quantizer's shape,
    on the stacked pair (cand_min, cand_max).  (The block expansion the reference does first
    repeats values and so cannot change a per-block minimum or maximum.)"""
    steps = qmax - qmin - (1 if zero_point_shift == 0.5 else 0)
    shape = torch.broadcast_shapes(cand_min.shape, cand_max.shape)
    stacked = torch.stack([cand_min.expand(shape), cand_max.expand(shape)])
    lo, hi = E.minmax_collect(stacked, tuple(qshape))
    return E.minmax_encodings(lo, hi, steps, symmetric)


def quantized_weight(w, enc_min, enc_max, qmin, qmax, symmetric, block_size=None, zero_point_shift=0.0):
    scale, offset = Q.scale_offset_from_min_max(enc_min, enc_max, qmin, qmax, symmetric)
    return A.quantize_dequantize(w, scale, offset, qmin, qmax, block_size, zero_point_shift)


def linear_loss(x, xq, w, wq, block_size, loss_fn="mse"):
    """_compute_linear_loss, vectorised form (:403-454) -> [C_out, num_blocks] in x.dtype"""
    out_ch, in_ch = w.shape
    nb = in_ch // block_size
    xb = x.reshape(-1, nb, block_size).permute(1, 0, 2)
    wb = w.reshape(out_ch, nb, block_size).permute(1, 2, 0)
    xqb = xq.reshape(-1, nb, block_size).permute(1, 0, 2)
    wqb = wq.reshape(out_ch, nb, block_size).permute(1, 2, 0)
    xw = torch.bmm(xb, wb).permute(1, 2, 0)
    xqwq = torch.bmm(xqb, wqb).permute(1, 2, 0)
    return LOSS_FNS[loss_fn](xw, xqwq, reduction="none").sum(0).view(out_ch, nb)


def conv_loss(x, xq, w, wq, block_size, loss_fn="mse", stride=1, padding=0, dilation=1, groups=1):
    """_compute_conv_loss (:485-520): the weight is cut into blocks of ``block_size`` input channels,
    the input into pieces of ``block_size * groups`` channels, one pair of convolutions per block;
    the loss is taken with the quantized output as prediction and summed over all positions
    (_base/seq_mse.py:705-720, 753-800) -> [C_out, num_blocks]"""
    w_blocks, wq_blocks = torch.split(w, block_size, dim=1), torch.split(wq, block_size, dim=1)
    x_blocks, xq_blocks = torch.split(x, block_size * groups, dim=-3), torch.split(xq, block_size * groups, dim=-3)
    cols = []
    for i, xb in enumerate(x_blocks):
        kw = dict(stride=stride, padding=padding, dilation=dilation, groups=groups)
        xqwq = F.conv2d(xq_blocks[i], wq_blocks[i], **kw).permute(0, 2, 3, 1)
        xw = F.conv2d(xb, w_blocks[i], **kw).permute(0, 2, 3, 1)
        ch = xqwq.shape[-1]
        cols.append(LOSS_FNS[loss_fn](xqwq.reshape(-1, ch), xw.reshape(-1, ch), reduction="none").sum(0))
    return torch.stack(cols, dim=-1)


def optimize_linear(w, xs, xqs, min_t, max_t, qmin, qmax, symmetric, block_size=None, num_candidates=20,
                    loss_fn="mse", zero_point_shift=0.0, num_batches=None, conv=None):
    """optimize_module (:523-578) for a Linear weight, or for a Conv2d weight when ``conv`` holds
    its stride / padding / dilation / groups.  ``min_t`` / ``max_t`` are the quantizer's
    get_min() / get_max() before the search.  Returns (losses [C, out, blocks], best indices,
    final encoding min, final encoding max)."""
    in_block = w.shape[1] if block_size is None else w.shape[1] // min_t.shape[1]
    total = []
    for i in range(num_candidates):
        cmin, cmax = candidate(i, num_candidates, min_t, max_t)
        emin, emax = encodings_for_candidate(cmin, cmax, min_t.shape, qmin, qmax, symmetric, zero_point_shift)
        wq = quantized_weight(w, emin, emax, qmin, qmax, symmetric, block_size, zero_point_shift)
        loss = 0
        for b, (x, xq) in enumerate(zip(xs, xqs)):
            if num_batches and b >= num_batches:
                break
            if conv is None:
                loss = loss + linear_loss(x, xq, w, wq, in_block, loss_fn)
            else:
                loss = loss + conv_loss(x, xq, w, wq, in_block, loss_fn, **conv)
        total.append(loss)
    losses = torch.stack(total)
    best = losses.min(0)[1]
    while best.dim() < max_t.dim():
        best = best[..., None]
    cmin, cmax = candidate(best, num_candidates, min_t, max_t)
    emin, emax = encodings_for_candidate(cmin, cmax, min_t.shape, qmin, qmax, symmetric, zero_point_shift)
    return losses, best, emin, emax
