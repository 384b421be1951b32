"""Oracle for the SeqMSE candidate search of a Linear layer (CPU, PyTorch tensor ops).

Restates seq_mse.py of the reference: candidate ranges (_get_candidate :360-372), the
re-calibration of the weight quantizer on a candidate range (compute_param_encodings :263-294),
the block-wise reconstruction loss (_compute_linear_loss :403-454) and the per-channel arg-min
(optimize_module :523-578); loss functions from _base/seq_mse.py:69-82, 872-888.
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


def optimize_linear(w, xs, xqs, min_t, max_t, qmin, qmax, symmetric, block_size=None, num_candidates=20,
                    loss_fn="mse", zero_point_shift=0.0, num_batches=None):
    """optimize_module (:523-578) for a Linear weight.  ``min_t`` / ``max_t`` are the quantizer's
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
            loss = loss + linear_loss(x, xq, w, wq, in_block, loss_fn)
        total.append(loss)
    losses = torch.stack(total)
    best = losses.min(0)[1]
    while best.dim() < max_t.dim():
        best = best[..., None]
    cmin, cmax = candidate(best, num_candidates, min_t, max_t)
    emin, emax = encodings_for_candidate(cmin, cmax, min_t.shape, qmin, qmax, symmetric, zero_point_shift)
    return losses, best, emin, emax
