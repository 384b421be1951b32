"""World-size-2 gloo tests (CPU) of the multi-GPU exchange logic: statistics combined over ranks
equal a single-process computation on all batches; a missing peer is reported, not waited for."""

import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _batches(n=4):
    g = torch.Generator().manual_seed(77)
    out = []
    for b in range(n):
        x = torch.randn(6, 32, 16, generator=g) * (1 + b)
        x[..., 3] *= 20
        out.append(x.to(torch.bfloat16))
    out[1][0, 0, 0] = float("inf")
    return out


# per-batch statistics on CPU tensors, standing in for the CUDA kernels
def _cpu_minmax(x, shape, block, finite_only):
    from oracle.encoding_analyzer import _finite_min_max, _stat_matrix

    rows = _stat_matrix(x, shape, block)
    mm = [_finite_min_max(r) for r in rows]
    return torch.stack([m[0] for m in mm]), torch.stack([m[1] for m in mm])


def _cpu_counts(x, shape, block, nbins, lo, hi):
    from oracle.encoding_analyzer import _stat_matrix

    rows = _stat_matrix(x, shape, block)
    out = []
    for r, l, h in zip(rows, lo, hi):
        c = torch.histc(r.float(), bins=nbins, min=float(l), max=float(h))
        c[0] += torch.sum(r < l)
        c[-1] += torch.sum(r > h)
        out.append(c.to(torch.int64))
    return torch.stack(out)


def _worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if mode == "missing_peer" and rank == 1:
        return  # this rank never joins
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    except Exception as e:  # noqa: BLE001  rendezvous itself may time out when the peer is missing
        ret[rank] = ("error", type(e).__name__)
        return
    try:
        from aimet_b200 import distributed as D
        from aimet_b200 import encoding_analyzer as EA

        batches = _batches()
        mine = [batches[i] for i in D.my_batches(len(batches), rank, world)]
        if mode == "histogram":
            an = EA.SqnrEncodingAnalyzer((16,), num_bins=64)
            st = D.calibrate_histogram(an, mine, minmax_fn=_cpu_minmax, counts_fn=_cpu_counts)
            ret[rank] = ("ok", st.histogram.clone(), st.bin_edges.clone(), st.min.clone(), st.max.clone())
        elif mode == "one_rank_empty":
            # fewer batches than ranks: rank 1 has nothing, takes part with an empty range and zero
            # counts, and ends with the same statistics as rank 0
            mine = batches[:1] if rank == 0 else []
            an = EA.SqnrEncodingAnalyzer((16,), num_bins=64)
            st = D.calibrate_histogram(an, mine, minmax_fn=_cpu_minmax, counts_fn=_cpu_counts, device="cpu")
            ret[rank] = ("ok", st.histogram.clone(), st.bin_edges.clone(), st.min.clone(), st.max.clone())
        elif mode == "all_ranks_empty":
            an = EA.SqnrEncodingAnalyzer((16,), num_bins=64)
            try:
                D.calibrate_histogram(an, [], minmax_fn=_cpu_minmax, counts_fn=_cpu_counts, device="cpu")
                ret[rank] = ("no error",)
            except D.PeerFailure as e:
                ret[rank] = ("peer failure", str(e)[:60])
        elif mode == "minmax":
            mn = torch.stack([b.amin() for b in mine]).amin()
            mx = torch.stack([b.amax() for b in mine]).amax()
            ret[rank] = ("ok",) + D.allreduce_minmax(mn.reshape(1), mx.reshape(1))
        elif mode == "gather":
            lo, hi = D.shard_range(7, rank, world)
            ret[rank] = ("ok", D.gather_rows(torch.arange(lo, hi).float()[:, None] * torch.ones(1, 3), 7))
        elif mode == "late_failure":
            if rank == 1:
                ret[rank] = ("left",)
                dist.destroy_process_group()
                return
            try:
                D.check_peers(timeout_s=3)
                D.allreduce_counts(torch.ones(4, dtype=torch.int64))
                ret[rank] = ("no error",)
            except D.PeerFailure as e:
                ret[rank] = ("peer failure", str(e)[:60])
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, mode, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(90)
            if p.is_alive():
                p.terminate()
                pytest.fail(f"rank hung in mode {mode}")
        return dict(ret)


def test_sharded_histogram_equals_single_process_collect():
    from oracle import encoding_analyzer as OA

    ret = _run("histogram")
    want = OA.hist_collect(torch.cat(_batches(), dim=0), (16,), 64)
    for rank in (0, 1):
        status, hist, edges, mn, mx = ret[rank]
        assert status == "ok"
        for i, w in enumerate(want):
            assert torch.equal(hist[i], w["histogram"]), f"rank {rank} histogram {i}"
            assert torch.equal(edges[i], w["bin_edges"])
            assert torch.equal(mn[i], w["min"]) and torch.equal(mx[i], w["max"])
    assert torch.equal(ret[0][1], ret[1][1])


def test_rank_without_a_batch_takes_part_instead_of_raising_alone():
    """A rank that received no batch must not leave the others waiting inside the collective: it
    contributes an empty range and zero counts; only when no rank has a batch do all raise, together."""
    from oracle import encoding_analyzer as OA

    ret = _run("one_rank_empty")
    want = OA.hist_collect(_batches()[0], (16,), 64)
    for rank in (0, 1):
        status, hist, edges, mn, mx = ret[rank]
        assert status == "ok"
        for i, w in enumerate(want):
            assert torch.equal(hist[i], w["histogram"]) and torch.equal(edges[i], w["bin_edges"])
            assert float(mn[i]) == float(w["min"]) and float(mx[i]) == float(w["max"])
    ret = _run("all_ranks_empty")
    assert ret[0][0] == "peer failure" and ret[1][0] == "peer failure"


def test_minmax_allreduce_and_row_gather():
    ret = _run("minmax")
    allb = torch.cat(_batches())
    for rank in (0, 1):
        assert ret[rank][1].dtype == torch.bfloat16
        assert ret[rank][1].item() == allb.amin().item() and ret[rank][2].item() == allb.amax().item()
    ret = _run("gather")
    for rank in (0, 1):
        assert torch.equal(ret[rank][1][:, 0], torch.arange(7).float())


def test_peer_that_leaves_is_reported_not_waited_for():
    ret = _run("late_failure")
    assert ret[1] == ("left",)
    assert ret[0][0] == "peer failure"


def test_shard_helpers():
    from aimet_b200 import distributed as D

    assert [D.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert D.shard_range(2, 3, 4) == (2, 2)
    assert D.my_batches(7, 1, 3) == [1, 4]
    assert D.allreduce_counts(torch.ones(3, dtype=torch.int64)).sum() == 3  # no process group: identity
    with pytest.raises(TypeError):
        D.allreduce_counts(torch.ones(3))
