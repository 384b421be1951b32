"""The CPU oracle of the encoding analyzers against fixtures produced by the reference itself."""

import warnings

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import encoding_analyzer as OA

CASES = load_golden("analyzer_cases.pt")


def run_oracle(case):
    """Replays the batches of a fixture through the oracle.  Returns (updates, encode_fn)."""
    kind, kw, shape, block = case["kind"], case["kwargs"], case["shape"], case["block_size"]
    updates = []
    if kind == "minmax":
        state = None
        for x in case["batches"]:
            new = OA.minmax_collect(x, shape, block)
            state = OA.minmax_merge(state, new)
            updates.append(dict(returned=dict(min=new[0], max=new[1]), merged=dict(min=state[0], max=state[1])))
        return updates, lambda n, sym: OA.minmax_encodings(state[0], state[1], n, sym)
    num_bins = kw.get("num_bins", 2048) if kind != "tfe" else 512
    growth = 3.0 if kind == "tfe" else float("inf")
    state = None
    for x in case["batches"]:
        new = OA.hist_collect(x, shape, num_bins, block)
        state = OA.hist_merge(state, new, x, shape, num_bins, growth, block)
        updates.append(dict(returned=new, merged=state["stats"]))
    if kind == "percentile":
        return updates, lambda n, sym: OA.percentile_encodings(state["stats"], shape, kw["percentile"], n, sym)
    sym_deltas = kw.get("symmetric_delta_candidates", 101)
    return updates, lambda n, sym: OA.sqnr_encodings(state["stats"], shape, n, sym, sym_deltas=sym_deltas)


def assert_stats_same(got, want, what):
    if isinstance(want, list):
        assert len(got) == len(want)
        for i, (g, w) in enumerate(zip(got, want)):
            for k in ("histogram", "bin_edges", "min", "max"):
                assert_same(g[k], w[k], f"{what}[{i}].{k}")
    else:
        for k in ("min", "max"):
            assert_same(got[k], want[k], f"{what}.{k}")


@pytest.mark.parametrize("name", sorted(CASES))
def test_statistics_match_reference(name):
    case = CASES[name]
    updates, _ = run_oracle(case)
    for i, (got, want) in enumerate(zip(updates, case["updates"])):
        assert_stats_same(got["returned"], want["returned"], f"update {i} returned")
        assert_stats_same(got["merged"], want["merged"], f"update {i} merged")


@pytest.mark.parametrize("name", sorted(CASES))
def test_encodings_match_reference(name):
    case = CASES[name]
    _, encode = run_oracle(case)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for (num_steps, sym), (want_min, want_max) in case["encodings"].items():
            got_min, got_max = encode(num_steps, sym)
            assert_same(got_min, want_min, f"min @ {num_steps},{sym}")
            assert_same(got_max, want_max, f"max @ {num_steps},{sym}")


def test_histc_binning_rule():
    """torch.histc's bin of a value is (int)((v - lo) * bins / (hi - lo)) in float32, v == hi in the
    last bin -- the rule the CUDA histogram kernel implements."""
    g = torch.Generator().manual_seed(7)
    for bins, lo, hi in ((2048, -6400.0, 5536.0), (512, -1.0, 1.0), (7, 0.1, 0.9), (100, -3.3, 17.7)):
        v = torch.empty(400000).uniform_(lo, hi, generator=g)
        edges = torch.arange(0, bins + 1) * ((torch.tensor(hi) - torch.tensor(lo)) / bins) + lo
        v = torch.cat([v, edges.float(), torch.nextafter(edges, torch.tensor(1e30)), torch.nextafter(edges, torch.tensor(-1e30))])
        v = v[(v >= lo) & (v <= hi)]
        ref = torch.histc(v, bins=bins, min=lo, max=hi)
        lo32, hi32 = torch.tensor(lo, dtype=torch.float32), torch.tensor(hi, dtype=torch.float32)
        b = ((v - lo32) * bins / (hi32 - lo32)).to(torch.int64).clamp(max=bins - 1)
        mine = torch.bincount(b, minlength=bins).to(torch.float32)
        assert torch.equal(ref, mine)


LP_CASES = load_golden("lpnorm_cases.pt")


@pytest.mark.parametrize("name", sorted(LP_CASES))
def test_lp_norm_search_matches_reference(name):
    """Error exponents other than 2 (_LpNormEncodingAnalyzer with p set freely): candidates,
    per-candidate noise and chosen range against the reference's own evaluation."""
    case = LP_CASES[name]
    for (num_steps, sym), want in case["grids"].items():
        deltas, offsets = OA.sqnr_candidates(case["stats"], num_steps, sym)
        assert_same(deltas, want["deltas"], "deltas")
        assert_same(offsets, want["offsets"], "offsets")
        assert_same(OA.sqnr_noise(case["stats"], deltas, offsets, num_steps, gamma=3.0, p=case["p"]), want["noise"], "noise")
        mn, mx = OA.sqnr_encodings(case["stats"], case["shape"], num_steps, sym, p=case["p"])
        assert_same(mn, want["min"], "min")
        assert_same(mx, want["max"], "max")
