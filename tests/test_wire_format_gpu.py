"""The encodings wire format (``to_qnn_encoding_dict``, versions 0.6.1 / 1.0.0 / 2.0.0 / 2.1.0) and the
LPBQ integer block scales, against dictionaries exported by the reference's own encoding objects."""

import math

import pytest
import torch

from conftest import assert_same, load_golden

pytestmark = pytest.mark.gpu

CASES = load_golden("wire_cases.pt")


def _same(a, b, path=""):
    """Equal structure; floats equal to the last bit except where the reference computed them on the
    CPU from values that differ in the last bit on the device (none do here)."""
    if isinstance(b, dict):
        assert isinstance(a, dict) and list(a.keys()) == list(b.keys()), f"{path}: keys {list(a)} vs {list(b)}"
        for k in b:
            _same(a[k], b[k], f"{path}.{k}")
    elif isinstance(b, (list, tuple)):
        assert isinstance(a, (list, tuple)) and len(a) == len(b), f"{path}: length"
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, f"{path}[{i}]")
    elif isinstance(b, float):
        assert a == b or (math.isnan(a) and math.isnan(b)), f"{path}: {a!r} vs {b!r}"
    else:
        assert a == b and type(a) is type(b), f"{path}: {a!r} vs {b!r}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_exported_dictionaries(name):
    from aimet_b200.quantizer import GroupedBlockQuantizeDequantize, QuantizeDequantize

    c = CASES[name]
    cls = QuantizeDequantize if c["kind"] == "qdq" else GroupedBlockQuantizeDequantize
    q = cls(*c["args"], **c["kwargs"]).cuda()
    with q.compute_encodings():
        q(c["w"].cuda())
    assert_same(q.min.detach(), c["min"], "calibrated min")
    assert_same(q.max.detach(), c["max"], "calibrated max")
    enc = q.get_encodings()._hint_input_shape(c["w"].shape)
    assert enc.granularity == c["granularity"]
    for version, want in c["dicts"].items():
        if isinstance(want, tuple):
            with pytest.raises(Exception) as e:
                enc.to_qnn_encoding_dict(version)
            assert type(e.value).__name__ == want[1]
        else:
            _same(enc.to_qnn_encoding_dict(version), want, version)
    if "per_block_int_scale" in c:
        assert_same(enc.per_block_int_scale, c["per_block_int_scale"], "per-block integer scales")  # exact integer codes


def test_round_trip_and_errors():
    from aimet_b200.quantizer import AffineEncoding, QuantizeDequantize

    q = QuantizeDequantize((), 8, False).cuda()
    with q.compute_encodings():
        q(torch.linspace(-1, 3, 100).cuda())
    enc = q.get_encodings()
    back = AffineEncoding._from_qnn_encoding_dict(enc.to_qnn_encoding_dict("2.0.0"))
    assert back.qmin == 0 and back.qmax == 255 and not back.symmetry
    assert float(back.scale) == float(enc.scale) and float(back.offset) == float(enc.offset)
    with pytest.raises(AssertionError):
        enc.to_qnn_encoding_dict("3.0.0")
    pc = QuantizeDequantize((4, 1), 8, True).cuda()
    with pc.compute_encodings():
        pc(torch.randn(4, 8).cuda())
    with pytest.raises(RuntimeError, match="input shape hint"):
        pc.get_encodings().to_qnn_encoding_dict("2.0.0")
    with pytest.raises(NotImplementedError):
        AffineEncoding._from_qnn_encoding_dict({"y_scale": [1.0], "axis": 0, "output_dtype": "int8"})
