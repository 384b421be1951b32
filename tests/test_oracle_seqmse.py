"""Oracle of the SeqMSE candidate search against fixtures from the reference's optimize_module."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import seq_mse as OS

CASES = load_golden("seqmse_cases.pt")


@pytest.mark.parametrize("name", sorted(CASES))
def test_optimize_linear_matches_reference(name):
    c = CASES[name]
    steps = 2 ** c["bitwidth"] - 1
    qmin, qmax = -((steps + 1) // 2), steps // 2
    losses, best, emin, emax = OS.optimize_linear(
        c["w"], list(c["x"]), list(c["x"]), c["min_before"], c["max_before"], qmin, qmax, True,
        block_size=c["block_size"], num_candidates=c["num_candidates"], loss_fn=c["loss_fn"])
    assert_same(losses, c["losses"], "per-candidate losses")
    assert torch.equal(losses.min(0)[1], c["best"])
    assert_same(emin.reshape(c["min_after"].shape), c["min_after"], "final min")
    assert_same(emax.reshape(c["max_after"].shape), c["max_after"], "final max")


EXTRA = load_golden("seqmse_extra_cases.pt")


@pytest.mark.parametrize("name", sorted(EXTRA))
def test_optimize_conv_and_distinct_inputs_match_reference(name):
    """Conv2d layers (per-channel, blockwise, grouped), blockwise Linear and inputs that differ
    between the floating-point and the quantized model."""
    c = EXTRA[name]
    steps = 2 ** c["bitwidth"] - 1
    qmin, qmax = -((steps + 1) // 2), steps // 2
    conv = None
    if c["layer"][0] == "conv":
        conv = dict(stride=1, padding=0, dilation=1, groups=1)
        conv.update(c["conv"])
    losses, best, emin, emax = OS.optimize_linear(
        c["w"], list(c["x"]), list(c["xq"]), c["min_before"], c["max_before"], qmin, qmax, True,
        block_size=c["block_size"], num_candidates=c["num_candidates"], loss_fn=c["loss_fn"], conv=conv)
    assert_same(losses, c["losses"], "per-candidate losses")
    assert torch.equal(losses.min(0)[1], c["best"])
    assert_same(emin.reshape(c["min_after"].shape), c["min_after"], "final min")
    assert_same(emax.reshape(c["max_after"].shape), c["max_after"], "final max")
