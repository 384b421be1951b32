"""Oracle of the quantizer parameter arithmetic against reference fixtures."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import affine as OA
from oracle import quantizer as OQ

CASES = load_golden("quantizer_cases.pt")


def _grid(kw):
    steps = 2 ** kw["bitwidth"] - 1
    if kw["symmetric"]:
        return -((steps + 1) // 2), steps // 2
    return 0, steps


@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_matches_reference(name):
    c = CASES[name]
    kw = c["kwargs"]
    qmin, qmax = _grid(kw)
    scale, offset = OQ.scale_offset_from_min_max(c["min"], c["max"], qmin, qmax, kw["symmetric"])
    if c["cls"] == "GroupedBlockQuantizeDequantize":
        scale, _ = OQ.lpbq_scale(scale, kw["bitwidth"], kw["decompressed_bw"], kw["block_grouping"])
    assert_same(scale, c["scale"], "scale")
    assert_same(offset, c["offset"], "offset")
    block = kw.get("block_size")
    if c["cls"] == "Quantize":
        out = OA.quantize(c["x"], scale, offset, qmin, qmax, block)
    else:
        out = OA.quantize_dequantize(c["x"], scale, offset, qmin, qmax, block, kw.get("zero_point_shift") or 0.0)
    assert_same(out, c["out"], "output")
