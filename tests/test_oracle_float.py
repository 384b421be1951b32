"""Oracle of the floating-point fake-cast against fixtures from the reference's float quantizers."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import float_cast as OF

CASES = load_golden("float_cases.pt")


def _format(c):
    kw = c["kwargs"]
    if c["kind"] in ("mxfp4", "nvfp4"):
        return (2, 1, True, False)
    if "dtype" in kw:
        return next(k for k, v in OF.TORCH_DTYPES.items() if v == kw["dtype"])
    return (kw["exponent_bits"], kw["mantissa_bits"], kw.get("finite", False), kw.get("unsigned_zero", False))


@pytest.mark.parametrize("name", sorted(CASES))
def test_float_fake_cast_matches_reference(name):
    c = CASES[name]
    fmt = _format(c)
    scale = OF.scale_from_maxval(c["maxval"], OF.format_max(*fmt), power_of_two=c["kind"] == "mxfp4")
    assert_same(scale, c["scale"], "scale")
    for key, x in (("y", c["x"]), ("y2", c["x2"]), ("dynamic", c["x"])):
        assert_same(OF.float_quantize_dequantize(x, c["scale"], *fmt, block_size=c["block_size"]), c[key], key)
