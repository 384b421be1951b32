"""Encoding analyzers on the B200 statistics kernels.

Host-side mirror of aimet_torch's ``quantization/encoding_analyzer.py``: the same class names,
constructor arguments, statistics containers and error behaviour (``_MinMaxObserver`` :69-118,
``_HistogramObserver`` :121-338, ``EncodingAnalyzer`` :341-394, ``MinMaxEncodingAnalyzer``
:397-481, ``PercentileEncodingAnalyzer`` :537-650, ``SqnrEncodingAnalyzer`` :902-953,
``TfEnhancedEncodingAnalyzer`` :956-1002), so an instance can be passed as ``encoding_analyzer=``
to a quantizer.  Every pass over the observed tensor is a CUDA kernel behind the C ABI
(min/max, histogram, SQNR sweep); what remains in PyTorch is O(bins) bookkeeping on device
tensors.  All histograms of an observer are kept as one batched tensor and handled at once.
"""

from __future__ import annotations

import math
from collections.abc import Sequence as _SequenceABC
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import lib
from .backend import _dense_perm, _param_blocks

__all__ = [
    "StatisticsNotFoundError",
    "EncodingAnalyzer",
    "MinMaxEncodingAnalyzer",
    "PercentileEncodingAnalyzer",
    "SqnrEncodingAnalyzer",
    "TfEnhancedEncodingAnalyzer",
]


class StatisticsNotFoundError(RuntimeError):
    """compute_encodings() was called before any statistics were observed (aimet_torch/utils.py:1257)."""


def _get_minimum_scale(num_steps) -> float:
    """Largest s <= float32 eps whose grid still spans [-0.005, 0.005] (_aimet_common/quantsim.py:537-559)."""
    return min(float(np.finfo(np.float32).eps), 0.01 / num_steps)


_SCALARS = {}


def _scalar(value, dtype, device) -> torch.Tensor:
    """A cached 0-d tensor holding ``value``.  Built with a fill kernel: ``torch.tensor(value,
    device=cuda)`` copies from pageable host memory, which makes the host wait for everything
    queued on the stream -- in the middle of a forward pass."""
    key = (float(value), dtype, str(device))
    t = _SCALARS.get(key)
    if t is None:
        t = torch.full((), float(value), dtype=dtype, device=device)
        _SCALARS[key] = t
    return t


def _div(a: torch.Tensor, b) -> torch.Tensor:
    """``a / b`` for a Python number ``b`` with IEEE division.  PyTorch's CUDA kernels turn a division
    by a Python scalar into a multiplication by its reciprocal, which differs from the CPU result in
    the last bit whenever ``b`` is not a power of two; dividing by a 0-d tensor does not."""
    if a.dtype in (torch.float16, torch.bfloat16):
        return (a.float() / _scalar(b, torch.float32, a.device)).to(a.dtype)
    return a / _scalar(b, a.dtype, a.device)


@dataclass
class _MinMaxRange:
    min: Optional[torch.Tensor] = None
    max: Optional[torch.Tensor] = None


@dataclass
class _Histogram:
    histogram: torch.Tensor = None
    bin_edges: torch.Tensor = None
    min: Optional[torch.Tensor] = None
    max: Optional[torch.Tensor] = None


class _HistogramList(_SequenceABC):
    """``List[_Histogram]`` view over batched tensors ``[H, bins]`` / ``[H, bins+1]`` / ``[H]``."""

    def __init__(self, histogram, bin_edges, min, max):  # pylint: disable=redefined-builtin
        self.histogram, self.bin_edges, self.min, self.max = histogram, bin_edges, min, max

    def __len__(self):
        return self.histogram.shape[0]

    def __getitem__(self, i):
        if isinstance(i, slice):
            return _HistogramList(self.histogram[i], self.bin_edges[i], self.min[i], self.max[i])
        if i < 0:
            i += len(self)
        if not 0 <= i < len(self):
            raise IndexError(i)
        return _Histogram(self.histogram[i], self.bin_edges[i], self.min[i], self.max[i])

    @staticmethod
    def from_stats(stats) -> "_HistogramList":
        if isinstance(stats, _HistogramList):
            return stats
        return _HistogramList(
            torch.stack([s.histogram for s in stats]),
            torch.stack([s.bin_edges for s in stats]),
            torch.stack([s.min for s in stats]),
            torch.stack([s.max for s in stats]),
        )


class _LazyHistogramList(_HistogramList):
    """Statistics of one batch whose histogram (and bin edges) are computed when they are first
    read.  Merging into an accumulated histogram only needs the batch's range (the counts are taken
    again over the merged range), so a caller that does not look at the per-batch histogram saves a
    pass over the tensor.  The observed tensor must not be modified before the histogram is read."""

    def __init__(self, compute, bin_edges, min, max):  # pylint: disable=redefined-builtin,super-init-not-called
        self._compute, self._hist = compute, None
        self._edges = bin_edges  # a tensor, or a callable that makes it
        self.min, self.max = min, max

    @property
    def bin_edges(self):
        if callable(self._edges):
            self._edges = self._edges()
        return self._edges

    @bin_edges.setter
    def bin_edges(self, value):
        self._edges = value

    @property
    def histogram(self):
        if self._hist is None:
            self._hist, self._compute = self._compute(), None
        return self._hist

    @histogram.setter
    def histogram(self, value):
        self._hist, self._compute = value, None

    def __len__(self):
        return self.min.shape[0]


# --------------------------------------------------------------------------------------------
# kernel plumbing
# --------------------------------------------------------------------------------------------
def _check_input(x: torch.Tensor) -> torch.Tensor:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"expected a torch.Tensor, got {type(x)}")
    if not x.is_cuda:
        raise RuntimeError(
            f"aimet_b200 analyzers observe CUDA tensors only (got '{x.device}'); there is no CPU fallback."
        )
    if x.dtype not in _lib.DTYPE_CODE:
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    return x.detach()


def _is_reducible(src_shape, target_shape) -> bool:
    if len(target_shape) > len(src_shape):
        return False
    return all(t in (1, s) for s, t in zip(reversed(src_shape), reversed(target_shape)))


class _StatLayout:
    """Dense view of an observed tensor plus the layout that maps it onto ``shape`` statistics."""

    def __init__(self, x: torch.Tensor, shape: Tuple[int, ...], block_size):
        if block_size is not None:
            if len(block_size) != len(shape) or len(shape) > x.dim():
                raise RuntimeError(f"Shape {shape} / block size {block_size} is incompatible with input of shape {tuple(x.shape)}")
            for k in range(1, len(shape) + 1):
                b, s, d = block_size[-k], shape[-k], x.shape[-k]
                if (b == -1 and (s == 0 or d % s != 0)) or (b != -1 and b * s != d):
                    raise RuntimeError(
                        f"Input of shape {list(x.shape)} can't be reduced to shape {list(shape)} with block size {block_size}"
                    )
        elif not _is_reducible(x.shape, shape):
            raise RuntimeError(f"Input of shape {list(x.shape)} can't be reduced to shape {list(shape)}")
        blocks = _param_blocks(x.shape, shape, block_size)
        perm = _dense_perm(x)
        if perm is not None and list(perm) != list(range(x.dim())):
            pdims = [k for k in perm if x.shape[k] // blocks[k] > 1]
            if pdims != sorted(pdims):
                perm = None
        self._key = (tuple(x.shape), x.stride(), x.dtype, x.device)
        self._copied = perm is None
        if perm is None:
            x = x.contiguous()
            perm = tuple(range(x.dim()))
        self._perm = perm
        self._identity = list(perm) == list(range(x.dim()))
        self.x = x.permute(perm)
        self.size = [x.shape[k] for k in perm]
        self.block = [blocks[k] for k in perm]
        self.layout = _lib.make_layout(self.size, self.block)
        self.count = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        self.io = _lib.DTYPE_CODE[self.x.dtype]

    def like(self, x: torch.Tensor) -> "_StatLayout":
        """The layout of another tensor of the same shape, strides, dtype and device (a list of
        calibration batches): nothing is derived again.  ``None`` if ``x`` differs in any of them."""
        if (tuple(x.shape), x.stride(), x.dtype, x.device) != self._key:
            return None
        other = _StatLayout.__new__(_StatLayout)
        other.__dict__.update(self.__dict__)
        if self._copied:
            x = x.contiguous()
        other.x = x if self._identity else x.permute(self._perm)
        return other

    def densify(self):
        """Fallback for layouts the kernels cannot walk in place: copy to [count, rest]."""
        x, size, block = self.x, self.size, self.block
        view = []
        for s, b in zip(size, block):
            view.extend((s // b, b))
        x = x.reshape(view)
        nd = len(size)
        x = x.permute(*range(0, 2 * nd, 2), *range(1, 2 * nd, 2)).reshape(self.count, -1).contiguous()
        self.x = x
        self.size, self.block = list(x.shape), [1, x.shape[1]]
        self.layout = _lib.make_layout(self.size, self.block)


def _run_minmax(lay: _StatLayout, finite_only: bool):
    x = lay.x
    mn = torch.empty(lay.count, dtype=x.dtype, device=x.device)
    mx = torch.empty(lay.count, dtype=x.dtype, device=x.device)
    with _lib.on_device(x.device):
        nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(x.device, nbytes)
        rc = lib.aimet_b200_minmax(x.data_ptr(), lay.layout, lay.io, int(finite_only), mn.data_ptr(), mx.data_ptr(),
                                   _lib.ptr(scratch), 0 if scratch is None else scratch.numel(),
                                   _lib.stream_ptr(x.device))
    _lib.check(rc)
    return mn, mx


def _minmax(lay: _StatLayout, finite_only: bool):
    try:
        return _run_minmax(lay, finite_only)
    except NotImplementedError:
        lay.densify()
        return _run_minmax(lay, finite_only)


def _run_histogram(lay: _StatLayout, num_bins: int, lo, hi, below, above):
    x = lay.x
    counts = torch.empty((lay.count, num_bins), dtype=torch.int64, device=x.device)
    with _lib.on_device(x.device):
        nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(x.device, nbytes)
        rc = lib.aimet_b200_histogram(x.data_ptr(), lay.layout, lay.io, num_bins, lo.data_ptr(), hi.data_ptr(),
                                      below.data_ptr(), above.data_ptr(), counts.data_ptr(), None, None,
                                      _lib.ptr(scratch), 0 if scratch is None else scratch.numel(),
                                      _lib.stream_ptr(x.device))
    _lib.check(rc)
    return counts


def _histogram_counts(lay: _StatLayout, num_bins: int, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """int64 [count, num_bins] histogram of the observed tensor over [lo, hi] per statistic, values
    below / above the range (including -inf / +inf) added to the first / last bin.  The outlier
    comparison happens in the observed tensor's dtype, like the reference's ``input < edge``."""
    if lay.x.dtype == torch.float64:
        lay.x = lay.x.to(torch.float32)
        lay.io = _lib.AB_F32
    lo = lo.to(torch.float32).contiguous()
    hi = hi.to(torch.float32).contiguous()
    below = lo.to(lay.x.dtype).to(torch.float32)
    above = hi.to(lay.x.dtype).to(torch.float32)
    try:
        return _run_histogram(lay, num_bins, lo, hi, below, above)
    except NotImplementedError:
        lay.densify()
        return _run_histogram(lay, num_bins, lo, hi, below, above)


def _histogram(lay: _StatLayout, num_bins: int, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """The same as float32, the dtype the reference keeps histograms in (exact below 2^24)."""
    return _histogram_counts(lay, num_bins, lo, hi).to(torch.float32)


def _layouts_of(tensors, shape, block_size):
    """A ``_StatLayout`` per tensor of a list; tensors shaped like the first share its derivation."""
    first = _StatLayout(_check_input(tensors[0]), shape, block_size)
    lays = [first]
    for x in tensors[1:]:
        x = _check_input(x)
        lays.append(first.like(x) or _StatLayout(x, shape, block_size))
    return lays


def _same_layout(lays) -> bool:
    first = lays[0]
    return all(l.size == first.size and l.block == first.block and l.io == first.io and l.x.device == first.x.device
               for l in lays[1:])


def _minmax_batches(lays, finite_only: bool):
    """Min / max over a list of observed tensors of one layout, one statistic pair for the whole list;
    tensors of a single contiguous statistic share launches."""
    if not _same_layout(lays):
        raise RuntimeError("the tensors of one calibration phase must share shape, dtype and device")
    lay = lays[0]
    x = lay.x
    mn = torch.empty(lay.count, dtype=x.dtype, device=x.device)
    mx = torch.empty(lay.count, dtype=x.dtype, device=x.device)
    with _lib.on_device(x.device):
        nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(x.device, max(nbytes, 1))
        rc = lib.aimet_b200_minmax_batches(_lib.ptr_array([l.x for l in lays]), len(lays), lay.layout, lay.io,
                                           int(finite_only), 0, mn.data_ptr(), mx.data_ptr(), _lib.ptr(scratch),
                                           scratch.numel(), _lib.stream_ptr(x.device))
    _lib.check(rc)
    return mn, mx


def _stat_dtype_code(dtype) -> int:
    return _lib.DTYPE_CODE[dtype] if dtype in (torch.float16, torch.bfloat16) else _lib.AB_F32


def _range_edges(mn: torch.Tensor, mx: torch.Tensor, num_bins: int, growth_limit: float, want_limit: bool = True):
    """Everything a histogram pass over [mn, mx] needs, in one launch: bin edges [H, bins + 1] (a
    degenerate range widened by 0.5 on each side), first / last edge, the two rounded to the tensor
    dtype (for the outlier comparisons) and the growth limit of the range."""
    dev = mn.device
    h = mn.numel()
    f32 = lambda t: t.detach().reshape(-1).to(torch.float32).contiguous()  # noqa: E731
    edges = torch.empty((h, num_bins + 1), dtype=torch.float32, device=dev)
    lo, hi, below, above = (torch.empty(h, dtype=torch.float32, device=dev) for _ in range(4))
    limit = torch.empty((h, 2), dtype=torch.float32, device=dev) if want_limit else None
    a, b = f32(mn), f32(mx)
    with _lib.on_device(dev):
        rc = lib.aimet_b200_histogram_edges(a.data_ptr(), b.data_ptr(), h, num_bins, _stat_dtype_code(mn.dtype),
                                            float(growth_limit), edges.data_ptr(), lo.data_ptr(), hi.data_ptr(),
                                            below.data_ptr(), above.data_ptr(), _lib.ptr(limit), _lib.stream_ptr(dev))
    _lib.check(rc)
    return edges, lo, hi, below, above, limit


def _histogram_batches(lays, num_bins: int, lo, hi, below, above, counts=None, want_minmax=False, run_if=None):
    """int64 counts [count, num_bins] of a list of tensors of one layout over [lo, hi] (added to
    ``counts`` when given), optionally with the finite min / max of the list from the same pass;
    ``run_if``: a device int32 flag -- the pass is skipped on the device when it is zero."""
    if not _same_layout(lays):
        raise RuntimeError("the tensors of one calibration phase must share shape, dtype and device")
    lay = lays[0]
    x = lay.x
    flags = 0
    if counts is None:
        counts = torch.empty((lay.count, num_bins), dtype=torch.int64, device=x.device)
    else:
        flags |= 1
    mn = mx = None
    if want_minmax:
        mn = torch.empty(lay.count, dtype=x.dtype, device=x.device)
        mx = torch.empty(lay.count, dtype=x.dtype, device=x.device)
    with _lib.on_device(x.device):
        nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
        _lib.check(nbytes)
        scratch = _lib.scratch.get(x.device, max(nbytes, 1))
        rc = lib.aimet_b200_histogram_batches(_lib.ptr_array([l.x for l in lays]), len(lays), lay.layout, lay.io, num_bins,
                                              lo.data_ptr(), hi.data_ptr(), below.data_ptr(), above.data_ptr(),
                                              counts.data_ptr(), _lib.ptr(mn), _lib.ptr(mx), flags, _lib.ptr(run_if),
                                              _lib.ptr(scratch), scratch.numel(), _lib.stream_ptr(x.device))
    _lib.check(rc)
    return (counts, mn, mx) if want_minmax else counts


def _f32c(t: torch.Tensor) -> torch.Tensor:
    """float32 contiguous (exact for 16-bit statistics); the tensor itself when it already is."""
    t = t.detach()
    return t if t.dtype == torch.float32 and t.is_contiguous() else t.to(torch.float32).contiguous()


def _merge_histograms(new: "_HistogramList", cur: "_HistogramList", limit: torch.Tensor, num_bins: int,
                      want_moved: bool = False, stat_dtype=torch.float32):
    """(updated min, updated max, carried counts, updated edges) of ``cur`` widened to cover ``new``;
    with ``want_moved`` also the per-histogram flag "the range no longer ends at the current edges"
    and [H, 4] = (first edge, last edge, both rounded to ``stat_dtype``) of the updated range."""
    dev = cur.histogram.device
    h = cur.histogram.shape[0]
    out_min = torch.empty(h, dtype=torch.float32, device=dev)
    out_max = torch.empty(h, dtype=torch.float32, device=dev)
    carry = torch.empty((h, num_bins), dtype=torch.float32, device=dev)
    edges = torch.empty((h, num_bins + 1), dtype=torch.float32, device=dev)
    args = [_f32c(new.min), _f32c(new.max), _f32c(cur.min), _f32c(cur.max), _f32c(cur.bin_edges), _f32c(cur.histogram),
            _f32c(limit)]
    moved = torch.empty(h, dtype=torch.int32, device=dev) if want_moved else None
    rng = torch.empty((h, 4), dtype=torch.float32, device=dev) if want_moved else None
    with _lib.on_device(dev):
        rc = lib.aimet_b200_histogram_merge_ex(*[t.data_ptr() for t in args], h, num_bins, out_min.data_ptr(),
                                               out_max.data_ptr(), carry.data_ptr(), edges.data_ptr(), _lib.ptr(moved),
                                               _lib.ptr(rng), _stat_dtype_code(stat_dtype), _lib.stream_ptr(dev))
    _lib.check(rc)
    return (out_min, out_max, carry, edges, moved, rng) if want_moved else (out_min, out_max, carry, edges)


# --------------------------------------------------------------------------------------------
# observers
# --------------------------------------------------------------------------------------------
class _Observer:
    def __init__(self, shape, block_size=None):
        if isinstance(shape, int):
            shape = (shape,)
        self.shape = tuple(shape)
        self.block_size = tuple(block_size) if block_size is not None else None


class _MinMaxObserver(_Observer):
    """Running elementwise min / max of everything observed (encoding_analyzer.py:69-118)."""

    def __init__(self, shape, block_size=None):
        super().__init__(shape, block_size)
        self.stats = _MinMaxRange()

    @torch.no_grad()
    def collect_stats(self, input_tensor: torch.Tensor) -> _MinMaxRange:
        x = _check_input(input_tensor)
        if x.numel() == 0:
            raise RuntimeError("cannot collect statistics of an empty tensor")
        mn, mx = _minmax(_StatLayout(x, self.shape, self.block_size), finite_only=False)
        return _MinMaxRange(mn.view(self.shape), mx.view(self.shape))

    @torch.no_grad()
    def merge_stats(self, stats: _MinMaxRange):
        new_min, new_max = self.stats.min, self.stats.max
        if stats.min is not None:
            new_min = stats.min.clone() if new_min is None else torch.minimum(new_min, stats.min)
        if stats.max is not None:
            new_max = stats.max.clone() if new_max is None else torch.maximum(new_max, stats.max)
        self.stats = _MinMaxRange(new_min, new_max)

    @torch.no_grad()
    def observe(self, input_tensor: torch.Tensor) -> None:
        """``collect_stats`` + ``merge_stats`` for a caller that does not want the batch's own
        statistics back (a model-level calibration in pass-through mode observes a hundred tensors per
        forward): the kernel updates the running min / max in place, two launches and no temporary
        tensors, and the description of the tensor's layout is kept between calls."""
        x = _check_input(input_tensor)
        if x.numel() == 0:
            raise RuntimeError("cannot collect statistics of an empty tensor")
        key = (tuple(x.shape), x.stride(), x.dtype, x.device)
        cached = self.__dict__.get("_layout_cache")
        if cached is None or cached[0] != key:
            lay = _StatLayout(x, self.shape, self.block_size)
            with _lib.on_device(x.device):
                nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
            _lib.check(nbytes)
            in_place = lay.x.data_ptr() == x.data_ptr()  # a permuted view of x itself (no copy was needed)
            cached = (key, lay, nbytes, in_place)
            self.__dict__["_layout_cache"] = cached
        _, lay, nbytes, in_place = cached
        if not in_place:
            lay = _StatLayout(x, self.shape, self.block_size)
        st = self.stats
        first = st.min is None
        if first or st.min.dtype != x.dtype or st.min.device != x.device:
            if not first:  # statistics of another dtype exist: fall back to the general path
                return self.merge_stats(self.collect_stats(x))
            # the first tensor's min / max are the running ones: written, not merged into +-inf
            st = _MinMaxRange(torch.empty(self.shape, dtype=x.dtype, device=x.device),
                              torch.empty(self.shape, dtype=x.dtype, device=x.device))
        entry = lib.aimet_b200_minmax if first else lib.aimet_b200_minmax_running
        with _lib.on_device(x.device):
            scratch = _lib.scratch.get(x.device, nbytes)
            rc = entry(x.data_ptr() if in_place else lay.x.data_ptr(), lay.layout, lay.io, 0, st.min.data_ptr(),
                       st.max.data_ptr(), _lib.ptr(scratch), 0 if scratch is None else scratch.numel(),
                       _lib.stream_ptr(x.device))
        if rc == _lib.AB_ERR_UNSUPPORTED:
            return self.merge_stats(self.collect_stats(x))
        if first and rc == 0:
            self.stats = st
        _lib.check(rc)
        return None

    def reset_stats(self):
        self.stats = _MinMaxRange()

    def get_stats(self) -> _MinMaxRange:
        return self.stats


class _HistogramObserver(_Observer):
    """One ``num_bins`` histogram per element of ``shape`` (encoding_analyzer.py:121-338)."""

    def __init__(self, shape, *, block_size=None, num_bins: int, growth_limit: Optional[float] = None):
        super().__init__(shape, block_size)
        self.num_bins = num_bins
        self.num_histograms = int(np.prod(self.shape, dtype=np.int64)) if len(self.shape) else 1
        if growth_limit is None:
            growth_limit = float("inf")
        if growth_limit < 1.0:
            raise RuntimeError(f"Growth limit must be at least 1.0. Got {growth_limit}")
        self.growth_limit = growth_limit
        self._state: Optional[_HistogramList] = None
        self._histogram_range_limit = None

    def _create_bin_edges(self, min_val: torch.Tensor, max_val: torch.Tensor) -> torch.Tensor:
        """[H, bins + 1] edges; a degenerate range is widened by 0.5 each side (:221-229)."""
        same = min_val == max_val
        lo = torch.where(same, min_val - 0.5, min_val).float()
        hi = torch.where(same, max_val + 0.5, max_val).float()
        step = _div(hi - lo, self.num_bins)
        ticks = torch.arange(0, self.num_bins + 1, device=min_val.device)
        return ticks[None, :] * step[:, None] + lo[:, None]

    @torch.no_grad()
    def collect_stats(self, input_tensor: torch.Tensor) -> _HistogramList:
        x = _check_input(input_tensor)
        if x.numel() == 0:
            raise RuntimeError("cannot collect statistics of an empty tensor")
        lay = _StatLayout(x, self.shape, self.block_size)
        mn, mx = _minmax(lay, finite_only=True)
        edges = self._create_bin_edges(mn, mx)
        if self._state is not None:  # statistics exist already: this batch's own histogram may never be read
            return _LazyHistogramList(lambda: _histogram(lay, self.num_bins, edges[:, 0], edges[:, -1]), edges, mn, mx)
        hist = _histogram(lay, self.num_bins, edges[:, 0], edges[:, -1])
        return _HistogramList(hist, edges, mn, mx)

    def _bin_index(self, width, base, data):
        idx = ((data - base[:, None]) / width[:, None]).to(torch.int32)
        return idx.clamp(max=self.num_bins - 1)

    @torch.no_grad()
    def merge_stats(self, new_stats_list, input_tensor: torch.Tensor):
        new = _HistogramList.from_stats(new_stats_list)
        n = self.num_bins
        if self._state is None:
            self._state = new
            e0, e1 = new.bin_edges[:, 0], new.bin_edges[:, -1]
            span = e1 - e0
            self._histogram_range_limit = torch.stack(
                (e0 - _div(span * self.growth_limit, 2), e1 + _div(span * self.growth_limit, 2)), dim=1
            )
            return
        cur = self._state
        x = _check_input(input_tensor)
        # the accumulated counts moved into the bins of the updated range, the updated range and its
        # edges: one kernel (a source bin that straddles a destination edge is split proportionally
        # and rounded, :274-310)
        umin, umax, carry, edges = _merge_histograms(new, cur, self._histogram_range_limit, n)
        lay = _StatLayout(x, self.shape, self.block_size)
        hist = _histogram(lay, n, umin, umax)
        hist += carry
        self._state = _HistogramList(hist, edges, umin, umax)

    @torch.no_grad()
    def observe(self, input_tensor: torch.Tensor):
        """``collect_stats`` + ``merge_stats`` of one batch with a single pass over the tensor where
        that is possible (what ``update_stats`` of the histogram analyzers runs).

        Once statistics exist, one kernel bins the batch against the *current* range and finds the
        batch's own finite min / max on the way.  The merge kernel then decides, on the device,
        whether the range had to move (growth, or a first range that the batch exceeds); only then
        are the counts wrong, and a second binning pass over the moved range runs -- launched
        always, skipped on the device when the flag says so, so the host never waits.  The batch's
        own histogram (which the reference computes on every update and most callers never read)
        is produced only when someone asks for it."""
        x = _check_input(input_tensor)
        if x.numel() == 0:
            raise RuntimeError("cannot collect statistics of an empty tensor")
        if self._state is None:
            new = self.collect_stats(x)
            self.merge_stats(new, x)
            return new
        n = self.num_bins
        cur = self._state
        if self.num_histograms == 1 and x.dtype in (torch.float32, torch.float16, torch.bfloat16):
            batch = self._observe_one_call(x, cur, n)
            if batch is not None:
                return batch
        lay = _StatLayout(x, self.shape, self.block_size)
        if lay.x.dtype == torch.float64:
            new = self.collect_stats(x)
            self.merge_stats(new, x)
            return new
        # first / last edge of the current range and the two rounded to the tensor dtype: kept from
        # the previous update (the merge kernel writes them) as long as the dtype stays the same
        rng = getattr(cur, "_range", None)
        if rng is None or rng[1] != lay.x.dtype:
            e0, e1 = cur.bin_edges[:, 0], cur.bin_edges[:, -1]
            rng = (torch.stack((e0, e1, e0.to(lay.x.dtype).to(torch.float32), e1.to(lay.x.dtype).to(torch.float32)),
                               dim=1).contiguous(), lay.x.dtype)
        r = rng[0]
        lo, hi, below, above = r[:, 0], r[:, 1], r[:, 2], r[:, 3]  # strided views: only their first element is read per histogram

        def bin_over(lo, hi, below, above, **kw):
            cols = [c.contiguous() for c in (lo, hi, below, above)] if r.shape[0] > 1 else [lo, hi, below, above]
            try:
                return _histogram_batches([lay], n, *cols, **kw)
            except NotImplementedError:
                lay.densify()
                return _histogram_batches([lay], n, *cols, **kw)

        counts, bmin, bmax = bin_over(lo, hi, below, above, want_minmax=True)
        batch = _LazyHistogramList(None, None, bmin, bmax)
        batch._edges = lambda: self._create_bin_edges(bmin, bmax)  # pylint: disable=protected-access
        batch._compute = lambda: _histogram(lay, n, batch.bin_edges[:, 0], batch.bin_edges[:, -1])  # pylint: disable=protected-access
        umin, umax, carry, edges, moved, nr = _merge_histograms(batch, cur, self._histogram_range_limit, n, want_moved=True,
                                                                stat_dtype=lay.x.dtype)
        # the second pass: over the moved range, skipped on the device for histograms whose range held
        redo = torch.zeros_like(counts)
        bin_over(nr[:, 0], nr[:, 1], nr[:, 2], nr[:, 3], counts=redo, run_if=moved)
        hist = torch.empty((counts.shape[0], n), dtype=torch.float32, device=counts.device)
        with _lib.on_device(counts.device):
            rc = lib.aimet_b200_histogram_combine(counts.data_ptr(), redo.data_ptr(), carry.data_ptr(), moved.data_ptr(),
                                                  counts.shape[0], n, hist.data_ptr(), _lib.stream_ptr(counts.device))
        _lib.check(rc)
        self._state = _HistogramList(hist, edges, umin, umax)
        self._state._range = (nr, lay.x.dtype)  # pylint: disable=protected-access
        return batch

    def _observe_one_call(self, x: torch.Tensor, cur: "_HistogramList", n: int):
        """The update of a single (per-tensor) histogram enqueued by one library call
        (``aimet_b200_histogram_update``: the same launches as the general path below, without the
        Python between them).  ``None`` when the tensor's layout needs the general path."""
        key = (tuple(x.shape), x.stride(), x.dtype, x.device)
        cached = self.__dict__.get("_one_call_cache")
        if cached is None or cached[0] != key:
            lay = _StatLayout(x, self.shape, self.block_size)
            if lay.x.data_ptr() != x.data_ptr():  # a copy was needed: leave it to the general path
                return None
            with _lib.on_device(x.device):
                nbytes = lib.aimet_b200_stats_scratch_bytes(lay.layout, lay.io)
            _lib.check(nbytes)
            dev = x.device
            work = (torch.empty((2, n), dtype=torch.int64, device=dev), torch.empty(n, dtype=torch.float32, device=dev),
                    torch.empty(1, dtype=torch.int32, device=dev))
            cached = (key, lay.layout, lay.io, nbytes, work)
            self.__dict__["_one_call_cache"] = cached
        _, layout, io, nbytes, (counts, carry, moved) = cached
        dev = x.device
        rng = getattr(cur, "_range", None)
        if rng is None or rng[1] != x.dtype:
            e0, e1 = cur.bin_edges[:, 0], cur.bin_edges[:, -1]
            rng = (torch.stack((e0, e1, e0.to(x.dtype).to(torch.float32), e1.to(x.dtype).to(torch.float32)),
                               dim=1).contiguous(), x.dtype)
        # the state after the update in one allocation: counts, edges, min, max, range
        buf = torch.empty(2 * n + 7, dtype=torch.float32, device=dev)
        hist, edges = buf[:n].view(1, n), buf[n:2 * n + 1].view(1, n + 1)
        umin, umax, nr = buf[2 * n + 1:2 * n + 2], buf[2 * n + 2:2 * n + 3], buf[2 * n + 3:].view(1, 4)
        bm = torch.empty(2, dtype=x.dtype, device=dev)
        bmin, bmax = bm[0:1], bm[1:2]
        scratch = _lib.scratch.get(dev, max(nbytes, 1))
        with _lib.on_device(dev):
            rc = lib.aimet_b200_histogram_update(
                x.data_ptr(), layout, io, n, _f32c(cur.histogram).data_ptr(), _f32c(cur.bin_edges).data_ptr(),
                _f32c(cur.min).data_ptr(), _f32c(cur.max).data_ptr(), rng[0].data_ptr(),
                _f32c(self._histogram_range_limit).data_ptr(), hist.data_ptr(), edges.data_ptr(), umin.data_ptr(),
                umax.data_ptr(), nr.data_ptr(), bmin.data_ptr(), bmax.data_ptr(), counts[0].data_ptr(),
                counts[1].data_ptr(), carry.data_ptr(), moved.data_ptr(), _lib.ptr(scratch), scratch.numel(),
                _lib.stream_ptr(dev))
        if rc == _lib.AB_ERR_UNSUPPORTED:
            return None
        _lib.check(rc)
        self._state = _HistogramList(hist, edges, umin, umax)
        self._state._range = (nr, x.dtype)  # pylint: disable=protected-access
        batch = _LazyHistogramList(None, None, bmin, bmax)
        batch._edges = lambda: self._create_bin_edges(bmin, bmax)  # pylint: disable=protected-access
        batch._compute = lambda: _histogram(_StatLayout(x, self.shape, self.block_size), n, batch.bin_edges[:, 0],  # pylint: disable=protected-access
                                            batch.bin_edges[:, -1])
        return batch

    def reset_stats(self):
        self._state = None
        self._histogram_range_limit = None

    @property
    def stats(self):
        return self.get_stats()

    def get_stats(self):
        if self._state is None:
            return [_Histogram() for _ in range(self.num_histograms)]
        return self._state


# --------------------------------------------------------------------------------------------
# analyzers
# --------------------------------------------------------------------------------------------
class EncodingAnalyzer:
    """Gathers statistics of observed tensors and turns them into an encoding range (:341-394)."""

    def __init__(self, observer: _Observer):
        self.observer = observer

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        new_stats = self.observer.collect_stats(input_tensor)
        self.observer.merge_stats(new_stats)
        return new_stats

    @torch.no_grad()
    def observe(self, input_tensor: torch.Tensor) -> None:
        """``update_stats`` for callers that do not use the returned per-batch statistics."""
        fast = getattr(self.observer, "observe", None)
        if fast is not None:
            fast(input_tensor)
        else:
            self.update_stats(input_tensor)

    def reset_stats(self):
        self.observer.reset_stats()

    def compute_encodings(self, num_steps: int, is_symmetric: bool):
        return self.compute_encodings_from_stats(self.observer.get_stats(), num_steps, is_symmetric)

    def compute_dynamic_encodings(self, input_tensor: torch.Tensor, num_steps: int, is_symmetric: bool):
        return self.compute_encodings_from_stats(self.observer.collect_stats(input_tensor), num_steps, is_symmetric)

    def compute_encodings_from_stats(self, stats, num_steps: int, is_symmetric: bool):
        raise NotImplementedError


def _check_num_steps(num_steps):
    if num_steps <= 0:
        raise ValueError("The number of quantization bins cannot be less than or equal to 0.")


class MinMaxEncodingAnalyzer(EncodingAnalyzer):
    """Range = [min(input), max(input)], made to contain zero and at least ``minimum_scale`` wide,
    fitted to a symmetric grid on request (:397-481)."""

    def __init__(self, shape, block_size=None):
        super().__init__(_MinMaxObserver(shape, block_size))

    @torch.no_grad()
    def compute_encodings_from_stats(self, stats: _MinMaxRange, num_steps: int, is_symmetric: bool):
        _check_num_steps(num_steps)
        if stats.min is None or stats.max is None:
            raise StatisticsNotFoundError("No statistics present to compute encodings.")
        min_scale = _get_minimum_scale(num_steps)
        lo = torch.clamp(stats.min, max=0)
        hi = torch.clamp(stats.max, min=0)
        widen = min_scale * (_div(hi - lo, num_steps) < min_scale)
        pos, neg = math.floor(num_steps / 2), math.ceil(num_steps / 2)
        if is_symmetric:
            hi = hi + pos * widen
            lo = lo - neg * widen
            # a 2-bit grid would waste its only positive step on symmetric data: calibrate as if it had two
            extra = 1 if num_steps == 3 else 0
            delta = torch.maximum(_div(hi, pos + extra), _div(-lo, neg))
            lo = -1 * neg * delta
            hi = pos * delta
        else:
            hi = hi + num_steps * widen
        hi = torch.clamp(hi, max=torch.finfo(stats.min.dtype).max).to(stats.min.dtype)
        lo = torch.clamp(lo, min=torch.finfo(stats.max.dtype).min).to(stats.max.dtype)
        return lo, hi


class _HistogramAnalyzer(EncodingAnalyzer):
    observer: _HistogramObserver

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        return self.observer.observe(input_tensor)

    @staticmethod
    def _batched(stats) -> _HistogramList:
        if not isinstance(stats, _HistogramList) and stats[0].histogram is None:
            raise StatisticsNotFoundError("No statistics present to compute encodings.")
        return _HistogramList.from_stats(stats)


def _adjust_min_max(cmin, cmax, num_steps, is_symmetric):
    """Batched adjust_min_max (:501-534): include zero, keep finite, keep a minimum width, fit a
    symmetric grid."""
    min_scale = _get_minimum_scale(num_steps)
    cmin = torch.minimum(cmin, torch.zeros_like(cmin))
    cmax = torch.maximum(cmax, torch.zeros_like(cmax))
    cmin = cmin.clamp(min=torch.finfo(cmax.dtype).min, max=0)
    cmax = cmax.clamp(min=0, max=torch.finfo(cmax.dtype).max)
    narrow = _div(cmax - cmin, num_steps) < min_scale
    pos, neg = math.floor(num_steps / 2), math.ceil(num_steps / 2)
    if is_symmetric:
        cmin = torch.where(narrow, cmin - min_scale * neg, cmin)
        cmax = torch.where(narrow, cmax + min_scale * pos, cmax)
        a, b = _div(cmax, pos), _div(-cmin, neg)
        delta = torch.where(b > a, b, a)
        return -1 * neg * delta, pos * delta
    return cmin, torch.where(narrow, cmax + min_scale * num_steps, cmax)


class PercentileEncodingAnalyzer(_HistogramAnalyzer):
    """Range that clips the (100 - percentile)% smallest and largest observed values (:537-650)."""

    def __init__(self, shape, num_bins: int = 2048, percentile: float = 100, block_size=None):
        if num_bins <= 0:
            raise ValueError("Number of bins cannot be less than or equal to 0.")
        super().__init__(_HistogramObserver(shape=shape, num_bins=num_bins, block_size=block_size))
        self.set_percentile(percentile)

    def set_percentile(self, percentile):
        if percentile < 50 or percentile > 100:
            raise ValueError("Percentile value must be within 50-100 range")
        self.percentile = percentile

    @torch.no_grad()
    def compute_encodings_from_stats(self, stats, num_steps: int, is_symmetric: bool):
        _check_num_steps(num_steps)
        st = self._batched(stats)
        # prefix sums of integer counts: exact in float64, then rounded once like the reference's
        # double-accumulating cumsum
        cum = torch.cumsum(st.histogram.double(), dim=1).to(st.histogram.dtype)
        total = cum[:, -1:]
        hi_idx = torch.searchsorted(cum, _div(total * self.percentile, 100))
        lo_idx = torch.searchsorted(cum, total * (1 - self.percentile / 100))
        if self.percentile == 100:
            lo_idx = torch.zeros_like(lo_idx)
            hi_idx = torch.full_like(hi_idx, st.bin_edges.shape[1] - 1)
        cmin = torch.gather(st.bin_edges, 1, lo_idx)[:, 0]
        cmax = torch.gather(st.bin_edges, 1, hi_idx)[:, 0]
        emin, emax = _adjust_min_max(cmin, cmax, num_steps, is_symmetric)
        shape = self.observer.shape
        return emin.to(st.min.dtype).reshape(shape), emax.to(st.max.dtype).reshape(shape)


class _LpNormEncodingAnalyzer(_HistogramAnalyzer):
    """Searches (delta, offset) candidates for the lowest expected clipping + rounding noise,
    estimated from the histogram (:653-899)."""

    def __init__(self, shape, num_bins: int, *, p: float, asymmetric_delta_candidates: int,
                 symmetric_delta_candidates: int, offset_candidates: int, max_parallelism: int, gamma: float,
                 histogram_growth_limit: Optional[float] = None, block_size=None):
        if num_bins <= 0:
            raise ValueError("Number of bins cannot be less than or equal to 0.")
        if not p > 0:
            raise ValueError("The exponent p of the error must be positive.")
        super().__init__(_HistogramObserver(shape=shape, num_bins=num_bins, growth_limit=histogram_growth_limit,
                                            block_size=block_size))
        self.p = p
        self.asym_delta_candidates = asymmetric_delta_candidates
        self.sym_delta_candidates = symmetric_delta_candidates
        self.num_offset_candidates = offset_candidates
        self.gamma = gamma
        self.max_parallelism = max_parallelism  # kept for interface parity; all histograms run in one launch

    @torch.no_grad()
    def compute_encodings_from_stats(self, stats, num_steps: int, is_symmetric: bool):
        st = self._batched(stats)
        _check_num_steps(num_steps)
        emin, emax, _ = self._search(st, num_steps, is_symmetric)
        shape = self.observer.shape
        return emin.to(st.min.dtype).view(shape), emax.to(st.max.dtype).view(shape)

    _OFFSET_GRIDS = {}

    def _offset_grid(self, num_steps, device) -> torch.Tensor:
        """round(arange(-num_steps, step, step)), step = num_steps / (O - 2): the asymmetric offset
        candidates before the observed offset is appended (:754-766).  Built on the host (so that every
        device sees the CPU kernel's values) once per (num_steps, O, device)."""
        n_off = min(num_steps + 2, self.num_offset_candidates)
        key = (num_steps, n_off, str(device))
        grid = self._OFFSET_GRIDS.get(key)
        if grid is None:
            step = num_steps / (n_off - 2)
            grid = torch.round(torch.arange(start=-num_steps, end=step, step=step, dtype=torch.float32)).to(device)
            self._OFFSET_GRIDS[key] = grid
        return grid

    def _search(self, st: _HistogramList, num_steps, symmetric, want_candidates: bool = False):
        """Candidates, their noise and the winner's range in two launches (the candidates are formed on
        the device).  Returns (min, max, details): float32 [H] each; ``details`` holds the noise and,
        on request, the candidate grids for inspection."""
        hist = st.histogram.to(torch.float32).contiguous()
        edges = st.bin_edges.to(torch.float32).contiguous()
        h, bins = hist.shape
        dev = hist.device
        smin, smax = st.min.reshape(-1).to(torch.float32).contiguous(), st.max.reshape(-1).to(torch.float32).contiguous()
        k = self.sym_delta_candidates if symmetric else self.asym_delta_candidates
        grid = None if symmetric else self._offset_grid(num_steps, dev)
        ncand = k if symmetric else k * (grid.numel() + 1)
        noise = torch.empty((h, ncand), dtype=torch.float32, device=dev)
        deltas = torch.empty((h, ncand), dtype=torch.float32, device=dev) if want_candidates else None
        offsets = torch.empty((h, ncand), dtype=torch.float32, device=dev) if want_candidates else None
        emin = torch.empty(h, dtype=torch.float32, device=dev)
        emax = torch.empty(h, dtype=torch.float32, device=dev)
        best = torch.empty(h, dtype=torch.int32, device=dev)
        with _lib.on_device(dev):
            rc = lib.aimet_b200_sqnr_encodings(hist.data_ptr(), edges.data_ptr(), smin.data_ptr(), smax.data_ptr(),
                                               _lib.ptr(grid), 0 if grid is None else grid.numel(), k, int(symmetric),
                                               _stat_dtype_code(st.min.dtype), h, bins, float(num_steps),
                                               float(self.gamma), float(self.p), _get_minimum_scale(num_steps),
                                               noise.data_ptr(),
                                               _lib.ptr(deltas), _lib.ptr(offsets), emin.data_ptr(), emax.data_ptr(),
                                               best.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc)
        return emin, emax, dict(noise=noise, deltas=deltas, offsets=offsets, best=best)

    # candidate grids -----------------------------------------------------------------------
    def _pick_test_candidates(self, st: _HistogramList, num_steps, symmetric):
        min_scale = _get_minimum_scale(num_steps)
        mn = torch.min(st.min, torch.zeros_like(st.min))
        mx = torch.max(st.max, torch.zeros_like(st.max))
        mx = torch.max(mx, mn + min_scale * num_steps)
        if symmetric:
            return self._pick_test_candidates_symmetric(mn, mx, num_steps)
        return self._pick_test_candidates_asymmetric(mn, mx, num_steps)

    @staticmethod
    def _host_arange(device, **kw):
        # built on the host so that every device sees the CPU kernel's values
        return torch.arange(dtype=torch.float32, **kw).to(device)

    def _pick_test_candidates_asymmetric(self, mn, mx, num_steps):
        """K deltas = max_delta * k / (K - 1), k = 1..K, times O offsets spread over [-steps, 0] plus the
        observed one; every pair is then clipped to the observed range (:740-776, 797-820)."""
        dev = mn.device
        max_delta = _div((mx - mn).to(torch.float32), num_steps)
        obs_offset = torch.round(mn / max_delta)
        obs_min = max_delta * obs_offset
        obs_max = obs_min + max_delta * num_steps
        k = self.asym_delta_candidates
        deltas = _div(max_delta[:, None] * self._host_arange(dev, start=1, end=1 + k, step=1)[None, :], k - 1)
        n_off = min(num_steps + 2, self.num_offset_candidates)
        step = num_steps / (n_off - 2)
        offsets = torch.round(self._host_arange(dev, start=-num_steps, end=step, step=step))
        offsets = torch.concat((offsets[None, :].expand(mn.shape[0], -1), obs_offset[:, None]), dim=1)
        return self._clamp_delta_offset_values(obs_min, obs_max, num_steps, deltas, offsets)

    def _pick_test_candidates_symmetric(self, mn, mx, num_steps):
        """K deltas up to 2 * max|x| / steps with the single offset -steps // 2 (:778-795)."""
        dev = mn.device
        min_scale = _get_minimum_scale(num_steps)
        max_delta = _div(2 * torch.max(mx, -mn).to(torch.float32), num_steps)
        offsets = torch.full((1,), (-num_steps) // 2, dtype=torch.float32, device=dev)
        k = self.sym_delta_candidates
        deltas = _div(max_delta[:, None] * self._host_arange(dev, start=1, end=1 + k, step=1)[None, :], k - 1)
        deltas = torch.max(deltas, _scalar(min_scale, torch.float32, dev))
        return deltas[:, :, None], offsets[:, None, None]

    @staticmethod
    def _clamp_delta_offset_values(min_vals, max_vals, num_steps, deltas, offsets):
        min_scale = _get_minimum_scale(num_steps)
        tmin = deltas[:, :, None] * offsets[:, None, :]
        tmax = tmin + deltas[:, :, None] * num_steps
        tmin = torch.max(min_vals[:, None, None], tmin)
        tmax = torch.min(max_vals[:, None, None], tmax)
        deltas = _div(tmax - tmin, num_steps)
        deltas = torch.max(deltas, _scalar(min_scale, deltas.dtype, deltas.device))
        return deltas, torch.round(tmin / deltas)

    # sweep -----------------------------------------------------------------------------------
    def _select_best_candidates(self, deltas, offsets, st: _HistogramList, num_steps):
        noise, best = self._estimate_clip_and_quant_noise(st, deltas, offsets, num_steps, self.p, self.gamma,
                                                          return_best=True)
        idx = best.long()[:, None]
        best_delta = torch.gather(deltas.flatten(start_dim=1), 1, idx)
        if offsets.numel() == 1:
            return best_delta, offsets
        return best_delta, torch.gather(offsets.flatten(start_dim=1), 1, idx)

    @staticmethod
    def _estimate_clip_and_quant_noise(stats, test_deltas, test_offsets, num_steps, p, gamma=1.0, return_best=False):
        """Noise of every candidate, shape (hists, deltas, offsets): one kernel over the histogram."""
        st = _HistogramList.from_stats(stats)
        hist = st.histogram.to(torch.float32).contiguous()
        h, bins = hist.shape
        dev = hist.device
        edge0 = st.bin_edges[:, 0].to(torch.float32).contiguous()
        width = (st.bin_edges[:, 1] - st.bin_edges[:, 0]).to(torch.float32).contiguous()
        out_shape = torch.broadcast_shapes(test_deltas.shape, test_offsets.shape)
        deltas = test_deltas.to(torch.float32).expand(out_shape).reshape(h, -1).contiguous()
        per_hist = test_offsets.numel() != 1
        offs = (test_offsets.to(torch.float32).expand(out_shape).reshape(h, -1) if per_hist
                else test_offsets.to(torch.float32).reshape(1).expand(deltas.shape[1])).contiguous()
        ncand = deltas.shape[1]
        noise = torch.empty((h, ncand), dtype=torch.float32, device=dev)
        best = torch.empty(h, dtype=torch.int32, device=dev)
        with _lib.on_device(dev):
            rc = lib.aimet_b200_sqnr_sweep(hist.data_ptr(), edge0.data_ptr(), width.data_ptr(), deltas.data_ptr(),
                                           offs.data_ptr(), int(per_hist), h, bins, ncand, float(num_steps),
                                           float(gamma), float(p), noise.data_ptr(), best.data_ptr(),
                                           _lib.stream_ptr(dev))
        _lib.check(rc)
        noise = noise.view(out_shape)
        return (noise, best) if return_best else noise


class SqnrEncodingAnalyzer(_LpNormEncodingAnalyzer):
    """Range with the lowest expected squared error; clipping noise weighted by ``gamma`` (:902-953)."""

    def __init__(self, shape, num_bins: int = 2048, *, asymmetric_delta_candidates=17, symmetric_delta_candidates=101,
                 offset_candidates=21, max_parallelism=64, gamma=3.0, histogram_growth_limit: Optional[float] = None,
                 block_size=None):
        super().__init__(shape=shape, num_bins=num_bins, p=2.0,
                         asymmetric_delta_candidates=asymmetric_delta_candidates,
                         symmetric_delta_candidates=symmetric_delta_candidates, offset_candidates=offset_candidates,
                         max_parallelism=max_parallelism, gamma=gamma, histogram_growth_limit=histogram_growth_limit,
                         block_size=block_size)


class TfEnhancedEncodingAnalyzer(SqnrEncodingAnalyzer):
    """SQNR analyzer with the legacy tf-enhanced constants: 512 bins, 17 x 21 asymmetric and 101
    symmetric candidates, gamma 3, histogram range limited to 3x the first batch's (:956-1002)."""

    _V1_HISTOGRAM_NUM_BINS = 512
    _V1_ASYMMETRIC_DELTA_CANDIDATES = 17
    _V1_SYMMETRIC_DELTA_CANDIDATES = 101
    _V1_OFFSET_CANDIDATES = 21
    _V1_GAMMA = 3.0
    _V1_HISTOGRAM_MAX_GROWTH_RATE = 3.0

    def __init__(self, shape, block_size=None):
        super().__init__(shape=shape, num_bins=self._V1_HISTOGRAM_NUM_BINS,
                         asymmetric_delta_candidates=self._V1_ASYMMETRIC_DELTA_CANDIDATES,
                         symmetric_delta_candidates=self._V1_SYMMETRIC_DELTA_CANDIDATES,
                         offset_candidates=self._V1_OFFSET_CANDIDATES, gamma=self._V1_GAMMA,
                         histogram_growth_limit=self._V1_HISTOGRAM_MAX_GROWTH_RATE, block_size=block_size)

    @classmethod
    def set_growth_limit(cls, growth_limit: float):
        if growth_limit < 1.0:
            raise RuntimeError(f"Growth limit must be at least 1.0. Got {growth_limit}")
        cls._V1_HISTOGRAM_MAX_GROWTH_RATE = growth_limit
