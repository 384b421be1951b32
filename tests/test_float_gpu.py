"""Float fake-cast quantizers on CUDA against fixtures produced by the reference's quantizers (fp16, bf16,
the four fp8 formats, IEEE-style exponent / mantissa splits, fp4 e2m1, MXFP4, NVFP4; per-tensor,
per-channel and blockwise scales; float32, bfloat16 and float16 inputs)."""

import pytest
import torch

from conftest import assert_same, load_golden

pytestmark = pytest.mark.gpu

CASES = load_golden("float_cases.pt")


def _make(c):
    from aimet_b200 import float_quantizer as F

    if c["kind"] == "mxfp4":
        return F._MXFP4QuantizeDequantize(c["qshape"], c["block_size"]).cuda()
    if c["kind"] == "nvfp4":
        return F._NVFP4QuantizeDequantize(c["qshape"], c["block_size"]).cuda()
    return F.FloatQuantizeDequantize(shape=c["qshape"], block_size=c["block_size"], **c["kwargs"]).cuda()


@pytest.mark.parametrize("name", sorted(CASES))
def test_float_quantizer_golden(name):
    """The calibrated ``maxval`` is bit-exact.  The scale is ``2 ** (log2(maxval) - log2(format max))``
    evaluated with torch's own log2 / pow kernels, whose CPU (fixture) and CUDA versions differ in
    the last bit, so it is compared to 1e-6 (the difference of two logarithms, then a power); the fake-cast itself is then
    checked bit for bit under the fixture's scale."""
    from aimet_b200 import float_quantizer as F

    c = CASES[name]
    q = _make(c)
    with q.compute_encodings():
        dyn = q(c["x"].cuda())
    assert_same(q.maxval, c["maxval"], "calibrated maxval")
    assert dyn.dtype == c["dynamic"].dtype and dyn.shape == c["dynamic"].shape
    scale = q.get_scale()
    assert scale.dtype == c["scale"].dtype and scale.shape == c["scale"].shape
    assert torch.allclose(scale.cpu(), c["scale"], rtol=1e-6, atol=0)
    enc = q(c["x"].cuda()).encoding
    assert enc.mapping == "float" and enc.bitwidth == q.bitwidth
    ref_scale = c["scale"].cuda()
    for key in ("y", "y2"):
        x = c["x" if key == "y" else "x2"].cuda()
        got = F.float_quantize_dequantize(x, q._finfo, ref_scale, c["block_size"])
        assert_same(got, c[key], key)                             # bit-exact, dtype included
    assert_same(F.float_quantize_dequantize(c["x"].cuda(), q._finfo, ref_scale, c["block_size"]), c["dynamic"],
                "output while calibrating")


def test_large_tensor_and_memory_format():
    """A tensor larger than the L2 cache through the vectorised body, a channels-last input and a size
    that is not a multiple of the vector width, against the elementwise conversion torch performs."""
    from aimet_b200 import float_quantizer as F

    g = torch.Generator().manual_seed(4)
    x = (torch.randn(4096, 4099, generator=g) * 3).cuda()
    q = F.FloatQuantizeDequantize(dtype=torch.float8_e4m3fn).cuda()
    with q.compute_encodings():
        q(x)
    s = q.get_scale()
    want = ((x / s).clamp(-448, 448).to(torch.float8_e4m3fn).to(torch.float32)) * s
    assert_same(q(x), want, "e4m3fn, per tensor")
    xc = torch.randn(8, 16, 12, 12, generator=g).cuda().to(memory_format=torch.channels_last)
    qc = F.FloatQuantizeDequantize(dtype=torch.float8_e5m2, shape=(16, 1, 1)).cuda()
    with qc.compute_encodings():
        qc(xc)
    sc = qc.get_scale()
    want = ((xc / sc).clamp(-57344, 57344).to(torch.float8_e5m2).to(torch.float32)) * sc
    got = qc(xc)
    assert got.shape == xc.shape
    assert_same(got.contiguous(), want.contiguous(), "e5m2, per channel, channels last")


def test_constructor_and_errors():
    from aimet_b200 import float_quantizer as F

    with pytest.raises(ValueError):
        F.FloatQuantizeDequantize()
    with pytest.raises(ValueError):
        F.FloatQuantizeDequantize(exponent_bits=4, mantissa_bits=3, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="unkown"):  # the reference's message, spelling included
        F.FloatQuantizeDequantize(exponent_bits=3, mantissa_bits=2, finite=True)
    q16 = F.FloatQuantizeDequantize(dtype=torch.float16)
    assert q16.encoding_analyzer is None and q16.is_float16() and q16.bitwidth == 16  # 16-bit formats: scale fixed at 1
    q8 = F.FloatQuantizeDequantize(exponent_bits=4, mantissa_bits=3)
    assert q8.encoding_analyzer is not None and q8.bitwidth == 8 and not q8.is_bfloat16()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        q16(torch.randn(4))
    ints = torch.arange(4).cuda()
    assert q16.cuda()(ints) is ints
    assert "dtype=torch.float16" in repr(q16)
    back = F.FloatQuantizeDequantize.from_encodings(q8.cuda().get_encodings())
    assert back._finfo == q8._finfo
