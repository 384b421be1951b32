"""Multi-GPU partitioning of the hot path: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-process; these helpers add the two partitionings the work allows, with
results defined against the single-process computation:

* **Calibration statistics** -- batches are dealt out to the ranks, every rank observes only its
  own batches, and the statistics are combined with all-reduces: MIN / MAX for the running range,
  SUM of integer bin counts for histograms.  For histograms the exchange has two phases (agree on
  the range first, then bin over the common range), so the combined histogram is exactly the one a
  single ``collect_stats`` call on the concatenation of all batches yields
  (quantization/encoding_analyzer.py:194-211) -- not the order-dependent result of merging batch
  after batch.  Payloads are tiny (2 values, or ``num_bins`` counters, per statistic).
* **Per-output-channel work** (weight quantize-dequantize, SeqMSE) -- rows of the weight are split
  across ranks, no reduction crosses rows, and an all-gather of the per-channel results (best
  candidate index, encoding min / max) reassembles the answer.

No activation ever crosses a link.  Every collective is preceded by nothing that can fault a GPU;
a missing peer surfaces as ``PeerFailure`` (from the process group's time-out) on the host.
"""

from __future__ import annotations

import datetime
from typing import Callable, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = [
    "ALONE",
    "PeerFailure",
    "shard_range",
    "my_batches",
    "allreduce_minmax",
    "allreduce_counts",
    "calibrate_minmax",
    "calibrate_histogram",
    "gather_rows",
    "optimize_module_sharded",
]


class PeerFailure(RuntimeError):
    """A collective did not complete because another rank failed, left or timed out."""


class _Alone:
    """Stands for "no exchange: this process alone" where a process group is expected (``None`` means
    the default group once one is initialised)."""

    def __repr__(self):
        return "aimet_b200.distributed.ALONE"


ALONE = _Alone()


def _world(group) -> Tuple[int, int]:
    if group is ALONE or not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) slice of ``n`` items for ``rank``; sizes differ by at most one."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def my_batches(num_batches: int, rank: int, world: int) -> List[int]:
    """Round-robin assignment of calibration batches: batch b goes to rank b mod world."""
    return list(range(rank, num_batches, world))


def _collective(fn: Callable, *args, **kwargs):
    try:
        return fn(*args, **kwargs)
    except (RuntimeError, dist.DistBackendError) as e:  # time-out, connection reset, peer exit
        raise PeerFailure(f"collective failed: {e}") from e


def check_peers(group=None, timeout_s: float = 30.0):
    """Host-side liveness check before entering collectives (gloo: monitored barrier that names the
    missing rank; other backends: a plain barrier under the group's own time-out)."""
    rank, world = _world(group)
    if world == 1:
        return
    if dist.get_backend(group) == "gloo":
        _collective(dist.monitored_barrier, group=group, timeout=datetime.timedelta(seconds=timeout_s))
    else:
        _collective(dist.barrier, group=group)


def allreduce_minmax(mn: torch.Tensor, mx: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Element-wise MIN / MAX over ranks in ONE collective: MIN over the pair (lo, -hi) -- the
    exchange is latency-bound, so one call instead of two halves its cost.  16-bit statistics travel
    as float32 (exact, as is the negation) because not every backend reduces them natively."""
    rank, world = _world(group)
    if world == 1:
        return mn, mx
    dt = mn.dtype
    packed = torch.stack((mn.to(torch.float32), -mx.to(torch.float32))).contiguous()
    _collective(dist.all_reduce, packed, op=dist.ReduceOp.MIN, group=group)
    return packed[0].to(dt), (-packed[1]).to(dt)


def allreduce_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """Integer SUM of histogram counts over ranks (int64: exact and order-independent)."""
    rank, world = _world(group)
    if counts.dtype != torch.int64:
        raise TypeError("histogram counts are exchanged as int64")
    if world == 1:
        return counts
    counts = counts.contiguous()
    _collective(dist.all_reduce, counts, op=dist.ReduceOp.SUM, group=group)
    return counts


# --------------------------------------------------------------------------------------------
# calibration
# --------------------------------------------------------------------------------------------
def _default_minmax(x, shape, block_size, finite_only):
    from .encoding_analyzer import _check_input, _minmax, _StatLayout

    return _minmax(_StatLayout(_check_input(x), tuple(shape), block_size), finite_only)


def _default_counts(x, shape, block_size, num_bins, lo, hi):
    from .encoding_analyzer import _check_input, _histogram_counts, _StatLayout

    return _histogram_counts(_StatLayout(_check_input(x), tuple(shape), block_size), num_bins, lo, hi)


def _stat_device(batches, device):
    if batches:
        return batches[0].device
    if device is not None:
        return torch.device(device)
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def calibrate_minmax(analyzer, batches: Iterable[torch.Tensor], group=None, device=None):
    """Observe this rank's batches with a min-max analyzer and combine the ranges over all ranks.
    Afterwards ``analyzer.compute_encodings`` gives the same result on every rank, equal to
    observing all batches in one process.  A rank without a batch (fewer batches than ranks) takes
    part in the exchange with an empty range (+inf, -inf) on ``device`` (default: the current CUDA
    device); if no rank has one, every rank raises together after the exchange."""
    from .encoding_analyzer import _MinMaxRange

    batches = list(batches)
    for x in batches:
        analyzer.update_stats(x)
    st = analyzer.observer.get_stats()
    rank, world = _world(group)
    if world > 1:
        mn, mx = st.min, st.max
        if mn is None:
            dev = _stat_device(batches, device)
            shape = analyzer.observer.shape
            mn = torch.full(shape, float("inf"), dtype=torch.float32, device=dev)
            mx = torch.full(shape, float("-inf"), dtype=torch.float32, device=dev)
        mn, mx = allreduce_minmax(mn, mx, group)
        if bool((mn > mx).all()):  # the same on every rank: nobody observed anything
            raise PeerFailure("no rank observed a calibration batch")
        analyzer.observer.stats = _MinMaxRange(mn, mx)
    return analyzer.observer.get_stats()


def calibrate_histogram(analyzer, batches: Sequence[torch.Tensor], group=None, *,
                        minmax_fn: Optional[Callable] = None, counts_fn: Optional[Callable] = None, device=None,
                        timings: Optional[dict] = None):
    """Two-phase histogram calibration of this rank's batches for a histogram-based analyzer
    (percentile / SQNR / TF-enhanced).

    Phase 1: finite min / max of every local batch, combined locally and then over ranks.
    Phase 2: every batch is binned over the common range (integer counts, values outside the range
    or infinite go to the edge bins); counts are summed locally and then over ranks.
    The analyzer's observer is left holding the combined statistics.  By default every phase is a
    handful of launches however many batches there are (the kernels take lists of tensors, the
    bin edges come from one launch): with the passes over the data cut eight ways, per-batch
    launches and small tensor operations are what a calibration would otherwise spend its time
    on.  ``minmax_fn`` / ``counts_fn`` replace the per-batch statistics; they exist so that the
    exchange logic can be exercised with CPU tensors.  A rank without a batch contributes an empty range and
    zero counts (on ``device``); if no rank has a batch every rank raises together.
    ``timings``: a dict that receives CUDA events at the phase boundaries (``t0`` .. ``t4``: start,
    local ranges done, ranges exchanged, local counts done, counts exchanged).
    """
    from .encoding_analyzer import _HistogramList

    obs = analyzer.observer
    shape, block, nbins = obs.shape, obs.block_size, obs.num_bins
    batches = list(batches)
    rank, world = _world(group)
    dev = _stat_device(batches, device)
    if not batches and world == 1:
        raise PeerFailure("no calibration batch")

    def mark(name):
        if timings is not None and dev.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(dev))
            timings[name] = ev

    mark("t0")
    fast = minmax_fn is None and counts_fn is None and dev.type == "cuda" and all(
        x.dtype != torch.float64 for x in batches)
    minmax_fn, counts_fn = minmax_fn or _default_minmax, counts_fn or _default_counts
    lays = None
    if batches and fast:
        from .encoding_analyzer import _layouts_of, _minmax_batches, _same_layout

        lays = _layouts_of(batches, tuple(shape), block)
        if not _same_layout(lays):
            lays = None
    if lays is not None:
        try:
            mn, mx = _minmax_batches(lays, True)
        except NotImplementedError:
            for lay in lays:
                lay.densify()
            mn, mx = _minmax_batches(lays, True)
    elif batches:
        # per-batch statistics are kept and combined once (one stack + reduce instead of a small
        # kernel per batch)
        mins, maxs = zip(*(minmax_fn(x, shape, block, True) for x in batches))
        mn = torch.stack(mins).amin(dim=0) if len(mins) > 1 else mins[0]
        mx = torch.stack(maxs).amax(dim=0) if len(maxs) > 1 else maxs[0]
    else:
        mn = torch.full((obs.num_histograms,), float("inf"), dtype=torch.float32, device=dev)
        mx = torch.full((obs.num_histograms,), float("-inf"), dtype=torch.float32, device=dev)
    mark("t1")
    if world > 1:
        mn, mx = allreduce_minmax(mn, mx, group)
    mark("t2")
    limit = None
    if lays is not None:
        from .encoding_analyzer import _histogram_batches, _range_edges

        edges, lo, hi, below, above, limit = _range_edges(mn, mx, nbins, obs.growth_limit)
        counts = _histogram_batches(lays, nbins, lo, hi, below, above)
    else:
        edges = obs._create_bin_edges(mn, mx)  # pylint: disable=protected-access
        lo, hi = edges[:, 0].contiguous(), edges[:, -1].contiguous()
        if batches:
            per_batch = [counts_fn(x, shape, block, nbins, lo, hi) for x in batches]
            counts = torch.stack(per_batch).sum(dim=0) if len(per_batch) > 1 else per_batch[0]
        else:
            counts = torch.zeros((obs.num_histograms, nbins), dtype=torch.int64, device=dev)
    mark("t3")
    counts = allreduce_counts(counts, group)
    mark("t4")
    if world > 1 and not batches and int(counts.sum()) == 0:
        # this rank had nothing; if the sum over all ranks is empty too, nobody had (every rank sees
        # the same counts and raises the same way)
        raise PeerFailure("no rank observed a calibration batch")
    obs._state = _HistogramList(counts.to(torch.float32), edges, mn, mx)  # pylint: disable=protected-access
    if limit is None:
        e0, e1 = edges[:, 0], edges[:, -1]
        span = e1 - e0
        limit = torch.stack((e0 - span * obs.growth_limit / 2, e1 + span * obs.growth_limit / 2), dim=1)
    obs._histogram_range_limit = limit  # pylint: disable=protected-access
    return obs.get_stats()


# --------------------------------------------------------------------------------------------
# per-output-channel work
# --------------------------------------------------------------------------------------------
def gather_rows(local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """Reassemble a tensor whose dim 0 was split with :func:`shard_range` (shards may differ by one
    row, so they are padded to the longest for the all-gather)."""
    rank, world = _world(group)
    if world == 1:
        return local
    longest = -(-total_rows // world)
    pad = longest - local.shape[0]
    buf = torch.cat([local, local.new_zeros((pad, *local.shape[1:]))]) if pad else local.contiguous()
    parts = [torch.empty_like(buf) for _ in range(world)]
    _collective(dist.all_gather, parts, buf, group=group)
    out = []
    for r, p in enumerate(parts):
        lo, hi = shard_range(total_rows, r, world)
        out.append(p[: hi - lo])
    return torch.cat(out)


def optimize_module_sharded(quant_module, x, xq, params, group=None):
    """SeqMSE with the output channels of the weight split across ranks.

    Every rank holds the whole layer and the whole calibration input (replicated once into its own
    memory), searches the candidates for its slice of output channels only, and the per-channel
    winners are all-gathered so that every rank ends with the full, identical encodings.  Needs a
    per-channel or blockwise weight quantizer (a per-tensor range couples all channels)."""
    from .seq_mse import QuantizedLinear, SequentialMse

    rank, world = _world(group)
    qtz = quant_module.param_quantizers["weight"]
    if world == 1:
        return SequentialMse.optimize_module(quant_module, x, xq, params)
    out_ch = quant_module.weight.shape[0]
    if len(qtz.shape) == 0 or qtz.shape[0] != out_ch:
        raise RuntimeError("output-channel sharding needs a per-channel or blockwise weight quantizer")
    lo, hi = shard_range(out_ch, rank, world)
    if hi == lo:
        raise PeerFailure(f"rank {rank} received no output channel ({out_ch} channels over {world} ranks)")

    # a view of the layer restricted to this rank's rows, with a quantizer of the matching shape
    # (built without initialising a weight of its own: its weight is this rank's rows of the layer's)
    dev = quant_module.weight.device
    part = QuantizedLinear(quant_module.in_features, hi - lo, bias=False, device="meta", dtype=quant_module.weight.dtype)
    part.weight = torch.nn.Parameter(quant_module.weight.detach()[lo:hi], requires_grad=False)
    with torch.device(dev):  # parameters are created where they will live: no host-to-device copies
        pq = type(qtz)((hi - lo, *qtz.shape[1:]), qtz.bitwidth, qtz.symmetric, block_size=qtz.block_size,
                       zero_point_shift=qtz.zero_point_shift)
    pq.set_range(qtz.min.detach()[lo:hi], qtz.max.detach()[lo:hi])
    part.param_quantizers["weight"] = pq
    best = SequentialMse.optimize_module(part, x, xq, params)

    # ranges and winners travel together: one all-gather of [rows, min | max | winner] (the winners are
    # small integers, exact in the parameters' float type)
    rows = hi - lo
    pmin, pmax = pq.min.detach().reshape(rows, -1), pq.max.detach().reshape(rows, -1)
    ncol = pmin.shape[1]
    packed = gather_rows(torch.cat([pmin, pmax, best.reshape(rows, -1).to(pmin.dtype)], dim=1), out_ch, group)
    qtz.set_range(packed[:, :ncol].reshape(qtz.shape), packed[:, ncol:2 * ncol].reshape(qtz.shape))
    SequentialMse._freeze_quantizer_encoding(qtz)  # pylint: disable=protected-access
    return packed[:, 2 * ncol:].to(best.dtype)
