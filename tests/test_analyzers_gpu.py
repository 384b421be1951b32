"""CUDA encoding analyzers against the golden fixtures (reference outputs) and the CPU oracle."""

import warnings

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import encoding_analyzer as OA

pytestmark = pytest.mark.gpu

CASES = load_golden("analyzer_cases.pt")


def make_analyzer(case):
    from aimet_b200 import encoding_analyzer as EA

    kind, kw, shape, block = case["kind"], case["kwargs"], case["shape"], case["block_size"]
    if kind == "minmax":
        return EA.MinMaxEncodingAnalyzer(shape, block_size=block)
    if kind == "sqnr":
        return EA.SqnrEncodingAnalyzer(shape, block_size=block, **kw)
    if kind == "tfe":
        return EA.TfEnhancedEncodingAnalyzer(shape, block_size=block)
    return EA.PercentileEncodingAnalyzer(shape, block_size=block, **kw)


def assert_stats_same(got, want, what):
    if isinstance(want, list):
        assert len(got) == len(want)
        for i, w in enumerate(want):
            g = got[i]
            assert_same(g.histogram, w["histogram"], f"{what}[{i}].histogram")  # counts: bit-exact
            assert_same(g.bin_edges, w["bin_edges"], f"{what}[{i}].bin_edges")
            assert_same(g.min, w["min"], f"{what}[{i}].min")
            assert_same(g.max, w["max"], f"{what}[{i}].max")
    else:
        assert_same(got.min, want["min"], f"{what}.min")  # min/max: bit-exact
        assert_same(got.max, want["max"], f"{what}.max")


@pytest.mark.parametrize("name", sorted(CASES))
def test_statistics_golden(name):
    case = CASES[name]
    an = make_analyzer(case)
    for i, (x, want) in enumerate(zip(case["batches"], case["updates"])):
        ret = an.update_stats(x.cuda())
        assert_stats_same(ret, want["returned"], f"update {i} returned")
        assert_stats_same(an.observer.get_stats(), want["merged"], f"update {i} merged")


def _close_encoding(got, want, what):
    """Encodings of the SQNR search depend on sums over 2048 bins: the arg-min can legitimately move
    between candidates whose noise differs in the last float32 bits.  Everything else is exact."""
    assert got.shape == want.shape and got.dtype == want.dtype, what
    g, w = got.double().cpu(), want.double()
    assert torch.allclose(g, w, rtol=1e-5, atol=0), f"{what}: {g.flatten()[:4]} vs {w.flatten()[:4]}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_encodings_golden(name):
    case = CASES[name]
    an = make_analyzer(case)
    for x in case["batches"]:
        an.update_stats(x.cuda())
    exact = case["kind"] in ("minmax", "percentile")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for (num_steps, sym), (want_min, want_max) in case["encodings"].items():
            got_min, got_max = an.compute_encodings(num_steps, sym)
            if exact:
                assert_same(got_min, want_min, f"min @ {num_steps},{sym}")
                assert_same(got_max, want_max, f"max @ {num_steps},{sym}")
            else:
                _close_encoding(got_min, want_min, f"min @ {num_steps},{sym}")
                _close_encoding(got_max, want_max, f"max @ {num_steps},{sym}")


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if c["kind"] in ("sqnr", "tfe")))
@pytest.mark.parametrize("grid", [(255, False), (255, True), (15, True)])
def test_sqnr_noise_vs_oracle(name, grid):
    """Per-candidate noise within 1e-5 relative of the oracle's float32 evaluation, and the same
    arg-min wherever the two best candidates are further apart than that."""
    case = CASES[name]
    num_steps, sym = grid
    an = make_analyzer(case)
    for x in case["batches"]:
        an.update_stats(x.cuda())
    st = an.observer.get_stats()
    deltas, offsets = an._pick_test_candidates(st, num_steps, sym)
    noise, best = an._estimate_clip_and_quant_noise(st, deltas, offsets, num_steps, 2.0, an.gamma, return_best=True)

    ostats = case["updates"][-1]["merged"]
    kw = case["kwargs"]
    od, oo = OA.sqnr_candidates(ostats, num_steps, sym, sym_deltas=kw.get("symmetric_delta_candidates", 101))
    assert_same(deltas, od, "candidate deltas")      # candidate grids are elementwise float32: bit-exact
    assert_same(offsets, oo, "candidate offsets")
    onoise = OA.sqnr_noise(ostats, od, oo, num_steps, gamma=3.0)
    assert torch.allclose(noise.cpu().double(), onoise.double(), rtol=1e-5, atol=0)
    flat = onoise.flatten(start_dim=1).double()
    top2 = flat.topk(2, dim=1, largest=False).values
    decisive = (top2[:, 1] - top2[:, 0]) > 1e-5 * top2[:, 1].abs()
    obest = flat.argmin(dim=1)
    assert torch.equal(best.cpu().long()[decisive], obest[decisive])


def test_large_counts_and_histc_rule():
    """Counts beyond float32's exact range are accumulated as integers; the binning rule is
    torch.histc's on this device as well as in the oracle."""
    from aimet_b200 import encoding_analyzer as EA

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(1 << 22, generator=g) * 3).cuda()
    obs = EA._HistogramObserver((), num_bins=2048)
    st = obs.collect_stats(x)
    ref = torch.histc(x, bins=2048, min=float(st.bin_edges[0, 0]), max=float(st.bin_edges[0, -1]))
    assert torch.equal(st.histogram[0], ref)
    cpu = torch.histc(x.cpu(), bins=2048, min=float(st.bin_edges[0, 0]), max=float(st.bin_edges[0, -1]))
    assert torch.equal(st.histogram[0].cpu(), cpu)
    assert float(st.histogram.sum()) == x.numel()
    # all mass in one bin, > 2^24 elements: integer accumulation keeps the exact count
    big = torch.zeros(1 << 25, dtype=torch.bfloat16, device="cuda")
    big[0], big[1] = -1.0, 1.0
    st = obs.collect_stats(big)
    assert int(st.histogram[0].double().sum()) == big.numel()


def test_errors():
    from aimet_b200 import encoding_analyzer as EA

    an = EA.MinMaxEncodingAnalyzer(())
    with pytest.raises(EA.StatisticsNotFoundError):
        an.compute_encodings(255, False)
    an.update_stats(torch.randn(10).cuda())
    with pytest.raises(ValueError):
        an.compute_encodings(0, False)
    with pytest.raises(RuntimeError):
        an.update_stats(torch.randn(10))  # CPU tensor
    with pytest.raises(RuntimeError):
        EA.MinMaxEncodingAnalyzer((3,)).update_stats(torch.randn(10, 4).cuda())
    sq = EA.SqnrEncodingAnalyzer(())
    with pytest.raises(EA.StatisticsNotFoundError):
        sq.compute_encodings(255, False)
    with pytest.raises(ValueError):
        EA.PercentileEncodingAnalyzer((), percentile=20)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("channels", [1, 3])
def test_large_histograms_with_outliers_and_non_finite_values(dtype, channels):
    """The large-histogram kernel (lane-private counters, arithmetic binning) against torch.histc
    plus the outlier rule, with a binning range narrower than the data, thresholds rounded to the
    tensor dtype, infinities and NaN."""
    from aimet_b200 import encoding_analyzer as EA

    g = torch.Generator().manual_seed(5 + channels)
    n = (1 << 20) + 4096
    x = torch.randn(4, channels, n // 4, generator=g) * torch.tensor([1.0, 7.0, 0.01][:channels]).view(1, -1, 1)
    x[0, 0, :6] = torch.tensor([float("inf"), -float("inf"), float("nan"), 1e30, -1e30, 0.0])
    x = x.to(dtype).cuda()
    shape = (1, channels, 1) if channels > 1 else ()
    lay = EA._StatLayout(x, shape, None)
    lo = torch.tensor([-2.3017, -20.0, -0.02][:channels], device="cuda")
    hi = torch.tensor([2.7011, 13.0, 0.03][:channels], device="cuda")
    got = EA._histogram_counts(lay, 2048, lo, hi).cpu()
    xf = x.float().cpu()
    for c in range(channels):
        v = xf[:, c].flatten() if channels > 1 else xf.flatten()
        below = lo[c].to(dtype).float().cpu()
        above = hi[c].to(dtype).float().cpu()
        want = torch.histc(v[(v >= lo[c].cpu()) & (v <= hi[c].cpu())], bins=2048, min=float(lo[c]), max=float(hi[c])).long()
        want[0] += int((v < below).sum())
        want[-1] += int((v > above).sum())
        assert torch.equal(got[c], want), f"channel {c}: {(got[c] != want).sum()} bins differ"


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if c["kind"] in ("sqnr", "tfe")))
@pytest.mark.parametrize("grid", [(255, False), (255, True), (15, True), (65535, False)])
def test_candidates_formed_on_the_device_equal_the_reference_grids(name, grid):
    """The search kernel forms its (delta, offset) candidates itself.  They must be, bit for bit, the
    grids the reference builds with tensor operations (checked against the oracle in
    test_sqnr_noise_vs_oracle), the noise must be what the stand-alone noise kernel returns for
    those grids, and the range it reports the one of its own arg-min."""
    case = CASES[name]
    num_steps, sym = grid
    an = make_analyzer(case)
    for x in case["batches"]:
        an.update_stats(x.cuda())
    st = an._batched(an.observer.get_stats())
    deltas, offsets = an._pick_test_candidates(st, num_steps, sym)
    noise, best = an._estimate_clip_and_quant_noise(st, deltas, offsets, num_steps, 2.0, an.gamma, return_best=True)
    emin, emax, det = an._search(st, num_steps, sym, want_candidates=True)
    shape = torch.broadcast_shapes(deltas.shape, offsets.shape)
    h = st.histogram.shape[0]
    assert_same(det["deltas"], deltas.expand(shape).reshape(h, -1), "deltas")
    assert_same(det["offsets"], offsets.expand(shape).reshape(h, -1), "offsets")
    assert_same(det["noise"], noise.reshape(h, -1), "noise")
    assert torch.equal(det["best"], best)
    idx = best.long()[:, None]
    bd = torch.gather(det["deltas"], 1, idx)[:, 0]
    bo = torch.gather(det["offsets"], 1, idx)[:, 0]
    assert_same(emin, bo * bd, "range min")
    assert_same(emax, bo * bd + num_steps * bd, "range max")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_bin_edges_in_one_launch(dtype):
    """aimet_b200_histogram_edges against the tensor expression of _create_bin_edges, including a
    degenerate range (widened by 0.5 in the statistics dtype) and the growth limit."""
    from aimet_b200 import encoding_analyzer as EA

    mn = torch.tensor([-3.17, 0.0, 5.5, -1e-3, 2048.0], device="cuda").to(dtype)
    mx = torch.tensor([7.01, 0.0, 5.5, 9e4 if dtype != torch.float16 else 6e4, 2050.0], device="cuda").to(dtype)
    for bins, growth in ((2048, float("inf")), (512, 3.0), (7, 1.0)):
        obs = EA._HistogramObserver((5,), num_bins=bins, growth_limit=growth)
        want = obs._create_bin_edges(mn, mx)
        edges, lo, hi, below, above, limit = EA._range_edges(mn, mx, bins, growth)
        assert_same(edges, want, "edges")
        assert_same(lo, want[:, 0].contiguous(), "first edge")
        assert_same(hi, want[:, -1].contiguous(), "last edge")
        assert_same(below, want[:, 0].to(dtype).float(), "below")
        assert_same(above, want[:, -1].to(dtype).float(), "above")
        span = want[:, -1] - want[:, 0]
        assert_same(limit[:, 0].contiguous(), want[:, 0] - EA._div(span * growth, 2), "lower limit")
        assert_same(limit[:, 1].contiguous(), want[:, -1] + EA._div(span * growth, 2), "upper limit")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_lists_of_tensors_in_one_launch(dtype):
    """Min / max and counts of a list of batches (one launch for up to 32 tensors of a per-tensor
    statistic) equal the per-tensor results combined; more than 32 tensors, a tensor whose size is
    not a multiple of the vector width, and a per-channel layout (one launch per tensor)."""
    from aimet_b200 import encoding_analyzer as EA

    g = torch.Generator().manual_seed(9)
    for shape, qshape, count in (((1 << 20) + 3, (), 3), ((1 << 18), (), 35), ((64, 1 << 15), (64, 1), 3)):
        xs = [(torch.randn(shape, generator=g) * (1 + i)).to(dtype).cuda() for i in range(count)]
        xs[1].view(-1)[5] = float("inf")
        xs[0].view(-1)[7] = float("nan")
        lays = [EA._StatLayout(x, qshape, None) for x in xs]
        mn, mx = EA._minmax_batches(lays, True)
        singles = [EA._minmax(EA._StatLayout(x, qshape, None), True) for x in xs]
        assert_same(mn, torch.stack([s[0] for s in singles]).amin(0), "min over the list")
        assert_same(mx, torch.stack([s[1] for s in singles]).amax(0), "max over the list")
        edges, lo, hi, below, above, _ = EA._range_edges(mn * 0.5, mx * 0.5, 256, float("inf"))  # narrower than the data
        counts, fmn, fmx = EA._histogram_batches(lays, 256, lo, hi, below, above, want_minmax=True)
        want = sum(EA._histogram_counts(EA._StatLayout(x, qshape, None), 256, lo, hi) for x in xs)
        assert torch.equal(counts, want)
        assert_same(fmn, mn, "min from the histogram pass")
        assert_same(fmx, mx, "max from the histogram pass")
        # a conditional launch leaves the counts of switched-off histograms alone
        keep = counts.clone()
        EA._histogram_batches(lays, 256, lo, hi, below, above, counts=counts, run_if=torch.zeros(lays[0].count, dtype=torch.int32, device="cuda"))
        assert torch.equal(counts, keep)
        EA._histogram_batches(lays, 256, lo, hi, below, above, counts=counts, run_if=torch.ones(lays[0].count, dtype=torch.int32, device="cuda"))
        assert torch.equal(counts, 2 * keep)


def test_sequential_updates_in_one_pass_when_the_range_holds():
    """update_stats after the first batch bins against the current range and learns the batch's own
    range in the same pass; batches that stay inside the range, that exceed it, and (with a growth
    limit) that exceed what the range may grow to -- every intermediate state equals the oracle's
    (the reference's two-pass procedure)."""
    from aimet_b200 import encoding_analyzer as EA

    g = torch.Generator().manual_seed(21)
    n = (1 << 20) + 64
    scales = [4.0, 1.0, 2.0, 9.0, 3.0, 40.0, 1.0]
    batches = [(torch.randn(n, generator=g) * s).to(torch.bfloat16) for s in scales]
    for growth in (None, 3.0):
        an = EA.SqnrEncodingAnalyzer((), num_bins=2048, histogram_growth_limit=growth)
        state = None
        for i, x in enumerate(batches):
            ret = an.update_stats(x.cuda())
            new = OA.hist_collect(x, (), 2048)
            state = OA.hist_merge(state, new, x, (), 2048, growth if growth is not None else float("inf"))
            got = an.observer.get_stats()
            merged = state["stats"] if isinstance(state, dict) else state
            assert_stats_same(got, merged, f"growth {growth} update {i} merged")
            assert_same(ret.min, torch.stack([w["min"] for w in new]), "returned min")
            if i in (2, 5):  # the batch's own histogram on request
                assert_stats_same(ret, new, f"update {i} returned")


LP_CASES = load_golden("lpnorm_cases.pt")


@pytest.mark.parametrize("name", sorted(LP_CASES))
def test_lp_norm_search(name):
    """Error exponents other than 2: per-candidate noise within 1e-5 of the reference's, the
    reference's range wherever the two best candidates are further apart than that."""
    from aimet_b200 import encoding_analyzer as EA

    case = LP_CASES[name]
    an = EA._LpNormEncodingAnalyzer(case["shape"], case["num_bins"], p=case["p"], asymmetric_delta_candidates=17,
                                    symmetric_delta_candidates=101, offset_candidates=21, max_parallelism=64, gamma=3.0)
    for x in case["batches"]:
        an.update_stats(x.cuda())
    st = an.observer.get_stats()
    for (num_steps, sym), want in case["grids"].items():
        deltas, offsets = an._pick_test_candidates(st, num_steps, sym)
        assert_same(deltas, want["deltas"], "candidate deltas")
        assert_same(offsets, want["offsets"], "candidate offsets")
        noise = an._estimate_clip_and_quant_noise(st, deltas, offsets, num_steps, case["p"], 3.0)
        assert torch.allclose(noise.cpu().double(), want["noise"].double(), rtol=1e-5, atol=0), (num_steps, sym)
        flat = want["noise"].flatten(start_dim=1).double()
        top2 = flat.topk(2, dim=1, largest=False).values
        decisive = ((top2[:, 1] - top2[:, 0]) > 1e-5 * top2[:, 1].abs()).reshape(want["min"].shape)
        mn, mx = an.compute_encodings(num_steps, sym)
        assert torch.equal(mn.cpu()[decisive], want["min"][decisive]) and torch.equal(mx.cpu()[decisive], want["max"][decisive])
    with pytest.raises(ValueError):
        EA._LpNormEncodingAnalyzer((), 16, p=0.0, asymmetric_delta_candidates=17, symmetric_delta_candidates=101,
                                   offset_candidates=21, max_parallelism=64, gamma=3.0)
