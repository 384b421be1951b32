"""Oracle for the calibration statistics and encoding analyzers (CPU, PyTorch tensor ops).

Restates quantization/encoding_analyzer.py of the reference in a flat, functional form:
min/max observer (:69-118), histogram observer (:121-338), min-max encodings (:426-481),
percentile (:501-650), SQNR / TF-enhanced sweep (:653-1002).  Statistics are plain dicts.
Histogram slices are visited one by one with 0-d tensors exactly as the reference does, because
its results depend on PyTorch's type-promotion rules for 0-d operands.  Test infrastructure only.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .affine import _interleave, concrete_blocks

FP32_EPS = float(np.finfo(np.float32).eps)


def minimum_scale(num_steps) -> float:
    """_aimet_common/quantsim.py:537-559"""
    return min(FP32_EPS, 0.01 / num_steps)


# --------------------------------------------------------------------------------------------
# reshaping an input so that axis 0 enumerates the statistics and axis 1 what they are taken over
# --------------------------------------------------------------------------------------------
def _stat_matrix(x: torch.Tensor, shape: Sequence[int], block_size=None) -> torch.Tensor:
    """[prod(shape), everything reduced] view/copy of ``x`` (aimet_torch/utils.py:1115-1148 and
    encoding_analyzer.py:148-192 both reduce to this)."""
    shape = tuple(shape)
    if block_size is not None:
        blocks = concrete_blocks(x.shape, shape, block_size)
        x = x.reshape(-1, *_interleave(shape, blocks))
        shape = _interleave(shape, 1)
    if len(shape) > x.dim() or any(s not in (1, d) for s, d in zip(reversed(shape), reversed(x.shape))):
        raise RuntimeError(f"Shape {shape} is incompatible with input of shape {tuple(x.shape)}")
    padded = (1,) * (x.dim() - len(shape)) + shape
    keep = [a for a, d in enumerate(padded) if d > 1]
    drop = [a for a, d in enumerate(padded) if d == 1]
    n = int(np.prod([padded[a] for a in keep])) if keep else 1
    return x.permute(*keep, *drop).reshape(n, -1)


# --------------------------------------------------------------------------------------------
# min / max
# --------------------------------------------------------------------------------------------
def minmax_collect(x, shape, block_size=None) -> Tuple[torch.Tensor, torch.Tensor]:
    m = _stat_matrix(x, shape, block_size)
    return torch.amin(m, dim=1).view(tuple(shape)), torch.amax(m, dim=1).view(tuple(shape))


def minmax_merge(state, new):
    if state is None:
        return new[0].clone(), new[1].clone()
    return torch.minimum(state[0], new[0]), torch.maximum(state[1], new[1])


def minmax_encodings(mn, mx, num_steps, symmetric):
    """MinMaxEncodingAnalyzer.compute_encodings_from_stats (:426-481)"""
    if num_steps <= 0:
        raise ValueError("The number of quantization bins cannot be less than or equal to 0.")
    ms = minimum_scale(num_steps)
    lo = torch.clamp(mn, max=0)
    hi = torch.clamp(mx, min=0)
    step = (hi - lo) / num_steps
    adj = ms * (step < ms)
    if symmetric:
        hi = hi + math.floor(num_steps / 2) * adj
        lo = lo - math.ceil(num_steps / 2) * adj
        pos, neg = math.floor(num_steps / 2), math.ceil(num_steps / 2)
        extra = 1 if num_steps == 3 else 0
        delta = torch.maximum(hi / (pos + extra), -lo / neg)
        lo = -1 * neg * delta
        hi = pos * delta
    else:
        hi = hi + num_steps * adj
    hi = torch.clamp(hi, max=torch.finfo(mn.dtype).max).to(mn.dtype)
    lo = torch.clamp(lo, min=torch.finfo(mx.dtype).min).to(mx.dtype)
    return lo, hi


# --------------------------------------------------------------------------------------------
# histograms
# --------------------------------------------------------------------------------------------
def _finite_min_max(v):
    fin = v.isfinite()
    return torch.where(fin, v, float("inf")).min(), torch.where(fin, v, -float("inf")).max()


def _bin_edges(mn, mx, num_bins):
    """_create_bin_edges (:221-229)"""
    lo = torch.where(mn == mx, mn - 0.5, mn).float()
    hi = torch.where(mn == mx, mx + 0.5, mx).float()
    step = (hi - lo) / num_bins
    return torch.arange(0, num_bins + 1) * step + lo


def hist_collect(x, shape, num_bins, block_size=None) -> List[dict]:
    """_HistogramObserver.collect_stats (:194-211)"""
    out = []
    for row in _stat_matrix(x, shape, block_size):
        mn, mx = _finite_min_max(row)
        edges = _bin_edges(mn, mx, num_bins)
        h = torch.histc(row.to(torch.float), bins=num_bins, min=edges[0], max=edges[-1])
        h[0] += torch.sum(row < edges[0])
        h[-1] += torch.sum(row > edges[-1])
        out.append(dict(histogram=h, bin_edges=edges, min=mn, max=mx))
    return out


def _bin_of(width, base, data, num_bins):
    """_get_bin_num (:231-234)"""
    idx = ((data - base) / width).to(torch.int32)
    return torch.minimum(idx, torch.full(data.shape, num_bins - 1, dtype=torch.int32)).long()


def hist_merge(state: Optional[dict], new: List[dict], x, shape, num_bins, growth_limit=float("inf"), block_size=None):
    """_HistogramObserver.merge_stats (:239-332).  ``state`` = dict(stats=[...], limits=[H,2])."""
    if state is None:
        e0 = torch.tensor([h["bin_edges"][0] for h in new])
        e1 = torch.tensor([h["bin_edges"][-1] for h in new])
        rng = e1 - e0
        limits = torch.stack(((e0 - rng * growth_limit / 2).flatten(), (e1 + rng * growth_limit / 2).flatten()), dim=1)
        return dict(stats=new, limits=limits)
    merged = []
    rows = _stat_matrix(x, shape, block_size)
    for i, (nw, row) in enumerate(zip(new, rows)):
        cur = state["stats"][i]
        lo_lim, hi_lim = state["limits"][i]
        umin = nw["min"].clamp(lo_lim, cur["bin_edges"][0])
        umax = nw["max"].clamp(cur["bin_edges"][-1], hi_lim)
        if umin == cur["min"] and umax == cur["max"]:
            carry = cur["histogram"]
        else:
            dw = (umax - umin) / num_bins
            sw = cur["bin_edges"][1] - cur["bin_edges"][0]
            carry = torch.zeros(num_bins)
            src = cur["bin_edges"][:-1]
            d1 = _bin_of(dw, umin, src, num_bins)
            d1_end = umin + dw * (d1 + 1)
            first = torch.minimum(torch.round(((d1_end - src) / sw) * cur["histogram"]), cur["histogram"])
            carry.index_add_(0, d1, first)
            split = (first < cur["histogram"]).nonzero().flatten()
            d2 = _bin_of(dw, umin, src + dw, num_bins)
            rest = cur["histogram"] - first
            carry.index_add_(0, d2[split], rest[split])
        h = torch.histc(row.to(torch.float), bins=num_bins, min=umin, max=umax)
        h += carry
        h[0] += torch.sum(row < umin)
        h[-1] += torch.sum(row > umax)
        merged.append(dict(histogram=h, bin_edges=_bin_edges(umin, umax, num_bins), min=umin, max=umax))
    return dict(stats=merged, limits=state["limits"])


def adjust_min_max(cmin, cmax, num_steps, symmetric):
    """adjust_min_max (:501-534): 0-d tensors in, 0-d tensors out"""
    ms = minimum_scale(num_steps)
    cmin = torch.minimum(cmin, torch.zeros_like(cmin))
    cmax = torch.maximum(cmax, torch.zeros_like(cmax))
    cmin = cmin.clamp(min=torch.finfo(cmax.dtype).min, max=0)
    cmax = cmax.clamp(min=0, max=torch.finfo(cmax.dtype).max)
    thr = (cmax - cmin) / num_steps
    if symmetric:
        if thr < ms:
            cmin = cmin - ms * math.ceil(num_steps / 2)
            cmax = cmax + ms * math.floor(num_steps / 2)
        pos, neg = math.floor(num_steps / 2), math.ceil(num_steps / 2)
        delta = max(cmax / pos, -cmin / neg)
        cmin = -1 * neg * delta
        cmax = pos * delta
    elif thr < ms:
        cmax = cmax + ms * num_steps
    return cmin, cmax


def percentile_encodings(stats: List[dict], shape, percentile, num_steps, symmetric):
    """PercentileEncodingAnalyzer.compute_encodings_from_stats (:601-650)"""
    if num_steps <= 0:
        raise ValueError("The number of quantization bins cannot be less than or equal to 0.")
    mins, maxs = [], []
    for st in stats:
        cum = torch.cumsum(st["histogram"], dim=0)
        hi_idx = torch.searchsorted(cum, cum[-1] * percentile / 100)
        lo_idx = torch.searchsorted(cum, cum[-1] * (1 - percentile / 100))
        if percentile == 100:
            lo_idx, hi_idx = 0, -1
        lo, hi = adjust_min_max(st["bin_edges"][lo_idx], st["bin_edges"][hi_idx], num_steps, symmetric)
        mins.append(lo)
        maxs.append(hi)
    emin = torch.tensor(mins, dtype=stats[0]["min"].dtype).reshape(tuple(shape))
    emax = torch.tensor(maxs, dtype=stats[0]["max"].dtype).reshape(tuple(shape))
    return emin, emax


# --------------------------------------------------------------------------------------------
# SQNR / TF-enhanced
# --------------------------------------------------------------------------------------------
def sqnr_candidates(stats, num_steps, symmetric, asym_deltas=17, sym_deltas=101, num_offsets=21):
    """_pick_test_candidates* and _clamp_delta_offset_values (:728-820).
    Returns (deltas, offsets) broadcastable to [H, K, O]."""
    ms = minimum_scale(num_steps)
    mn = torch.stack([s["min"] for s in stats])
    mx = torch.stack([s["max"] for s in stats])
    mn = torch.min(mn, torch.zeros_like(mn))
    mx = torch.max(mx, torch.zeros_like(mx))
    mx = torch.max(mx, mn + ms * num_steps)
    f32 = dict(dtype=torch.float32)
    if symmetric:
        max_delta = 2 * torch.max(mx, -mn).to(torch.float32) / num_steps
        offsets = torch.full((1,), (-num_steps) // 2, **f32)
        space = torch.arange(start=1, end=1 + sym_deltas, step=1, **f32)
        deltas = max_delta[:, None] * space[None, :] / (sym_deltas - 1)
        deltas = torch.max(deltas, torch.tensor([ms], **f32))
        return deltas[:, :, None], offsets[:, None, None]
    max_delta = (mx - mn).to(torch.float32) / num_steps
    obs_off = torch.round(mn / max_delta)
    obs_min = max_delta * obs_off
    obs_max = obs_min + max_delta * num_steps
    space = torch.arange(start=1, end=1 + asym_deltas, step=1, **f32)
    deltas = max_delta[:, None] * space[None, :] / (asym_deltas - 1)
    n_off = min(num_steps + 2, num_offsets)
    off_step = num_steps / (n_off - 2)
    offs = torch.round(torch.arange(start=-num_steps, end=off_step, step=off_step, **f32))
    offs = offs[None, :].expand(mn.shape[0], -1)
    offs = torch.concat((offs, obs_off[:, None]), dim=1)
    tmin = deltas[:, :, None] * offs[:, None, :]
    tmax = tmin + deltas[:, :, None] * num_steps
    tmin = torch.max(obs_min[:, None, None], tmin)
    tmax = torch.min(obs_max[:, None, None], tmax)
    deltas = torch.max((tmax - tmin) / num_steps, torch.tensor([ms], **f32))
    return deltas, torch.round(tmin / deltas)


def sqnr_noise(stats, deltas, offsets, num_steps, gamma=3.0, p=2.0):
    """_estimate_clip_and_quant_noise (:822-899) -> [H, K, O]"""
    hists = torch.stack([s["histogram"] for s in stats])
    edges = torch.stack([s["bin_edges"] for s in stats])
    width = edges[:, 1] - edges[:, 0]
    mids = (edges[:, 0] + width / 2)[:, None] + width[:, None] * torch.arange(0, edges.shape[1] - 1, dtype=deltas.dtype)[None, :]
    ob, db = offsets[:, :, :, None], deltas[:, :, :, None]
    q = mids[:, None, None, :].div(db).sub(ob).round()
    clipped = torch.logical_or(q < 0, q > num_steps)
    q = q.clamp(0, num_steps).add(ob).mul(db)
    err = torch.abs(q.sub(mids[:, None, None, :])).pow(p).mul(hists[:, None, None, :])
    if gamma != 1.0:
        err = torch.where(clipped, err * gamma, err)
    return torch.sum(err, dim=-1)


def sqnr_encodings(stats, shape, num_steps, symmetric, gamma=3.0, asym_deltas=17, sym_deltas=101,
                   num_offsets=21, return_details=False, p=2.0):
    """_LpNormEncodingAnalyzer.compute_encodings_from_stats (:685-726) for one chunk of histograms
    (the reference processes at most ``max_parallelism`` histograms per chunk; chunks are
    independent, so one chunk restates all of them)."""
    if num_steps <= 0:
        raise ValueError("The number of quantization bins cannot be less than or equal to 0.")
    deltas, offsets = sqnr_candidates(stats, num_steps, symmetric, asym_deltas, sym_deltas, num_offsets)
    noise = sqnr_noise(stats, deltas, offsets, num_steps, gamma, p)
    _, idx = torch.min(noise.flatten(start_dim=1), dim=1)
    best_delta = torch.gather(deltas.flatten(start_dim=1), 1, idx[:, None])
    best_offset = offsets if offsets.numel() == 1 else torch.gather(offsets.flatten(start_dim=1), 1, idx[:, None])
    emin = best_offset * best_delta
    emax = emin + num_steps * best_delta
    emin = emin.to(stats[0]["min"].dtype).view(tuple(shape))
    emax = emax.to(stats[0]["max"].dtype).view(tuple(shape))
    if return_details:
        return emin, emax, dict(deltas=deltas, offsets=offsets, noise=noise, best=idx)
    return emin, emax
