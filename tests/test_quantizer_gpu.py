"""Quantizer modules on CUDA against fixtures produced by the reference's modules."""

import pytest
import torch

from conftest import assert_same, load_golden

pytestmark = pytest.mark.gpu

CASES = load_golden("quantizer_cases.pt")


def build(case):
    from aimet_b200 import encoding_analyzer as EA
    from aimet_b200 import quantizer as Q

    kw = dict(case["kwargs"])
    if case["analyzer"] == "sqnr":
        kw["encoding_analyzer"] = EA.SqnrEncodingAnalyzer(kw["shape"])
    return getattr(Q, case["cls"])(**kw).cuda()


def _internal_is_16bit(case):
    kw = case["kwargs"]
    steps = 2 ** kw["bitwidth"] - 1
    return case["x"].dtype in (torch.float16, torch.bfloat16) and not torch.finfo(case["x"].dtype).eps > 0.25 / steps


@pytest.mark.parametrize("name", sorted(CASES))
def test_calibrate_forward_backward(name):
    c = CASES[name]
    q = build(c)
    assert not q.is_initialized()
    x = c["x"].cuda()
    with q.compute_encodings():
        dyn = q(x)
    assert q.is_initialized()
    assert_same(dyn, c["dynamic_out"], "output while calibrating")
    assert_same(q.min.detach(), c["min"], "calibrated min")  # encodings: bit-exact
    assert_same(q.max.detach(), c["max"], "calibrated max")
    assert_same(q.get_scale().detach(), c["scale"], "scale")
    assert_same(q.get_offset().detach(), c["offset"], "offset")

    xi = x.clone().requires_grad_(True)
    y = q(xi)
    y.backward(c["grad"].cuda())
    assert_same(y.detach(), c["out"], "output")
    assert_same(xi.grad, c["grad_x"], "grad_x")
    for got, want, what in ((q.min.grad, c["grad_min"], "grad_min"), (q.max.grad, c["grad_max"], "grad_max")):
        got, want = got.double().cpu(), want.double()
        if _internal_is_16bit(c):
            # the reference sums these in the 16-bit internal dtype: one unit in its last place per entry
            tol = torch.finfo(c["x"].dtype).eps * want.abs().clamp_min(1e-6) * 1.01
            assert bool(((got - want).abs() <= tol).all()), what
        else:
            assert (got - want).abs().max() <= 1e-5 * want.abs().max().clamp_min(1e-30), what


def test_uninitialized_and_errors():
    from aimet_b200 import quantizer as Q

    q = Q.QuantizeDequantize((), 8, False).cuda()
    with pytest.raises(RuntimeError):
        q(torch.randn(4).cuda())
    assert q(torch.empty(0).cuda()).numel() == 0
    with pytest.raises(ValueError):
        Q.QuantizeDequantize((), qmin=5, qmax=5, symmetric=False)
    with pytest.raises(ValueError):
        Q.QuantizeDequantize((), 8, False, zero_point_shift=0.3)
    with pytest.raises(RuntimeError):
        Q.GroupedBlockQuantizeDequantize((4, 4), 4, False, decompressed_bw=8, block_size=(1, 8))
    with pytest.raises(RuntimeError):
        Q.Quantize((), 8, False, zero_point_shift=0.5)
    q2 = Q.QuantizeDequantize((), qmin=0, qmax=255, symmetric=False).cuda()
    q2.set_range(-1.0, 1.0)
    assert q2.is_initialized()
    q2.allow_overwrite(False)
    with q2.compute_encodings():
        q2(torch.randn(10).cuda() * 10)
    assert float(q2.min) == -1.0 and float(q2.max) == 1.0
    sd = q2.state_dict()
    q3 = Q.QuantizeDequantize((), 4, True).cuda()
    q3.load_state_dict(sd)
    assert q3.qmax == 255 and q3.is_initialized() and not q3.symmetric


def test_learning_moves_the_range():
    from aimet_b200 import quantizer as Q

    torch.manual_seed(0)
    q = Q.QuantizeDequantize((8, 1), 4, True).cuda()
    x = torch.randn(8, 256).cuda()
    with q.compute_encodings():
        q(x)
    opt = torch.optim.SGD(q.parameters(), lr=1e-2)
    before = (q(x) - x).pow(2).mean().item()
    for _ in range(50):
        opt.zero_grad()
        loss = (q(x) - x).pow(2).mean()
        loss.backward()
        opt.step()
    assert loss.item() < before


def _mixed_quantizers(device):
    from aimet_b200 import quantizer as Q

    torch.manual_seed(0)
    qs = []
    for i, (shape, bw, sym) in enumerate([((8, 1), 8, True), ((), 8, False), ((4, 1, 1, 1), 4, True), ((), 8, False),
                                          ((3,), 16, False), ((8, 1), 8, True), ((5, 1), 8, False)]):
        q = Q.QuantizeDequantize(shape, bw, sym)
        lo, hi = -torch.rand(shape) * 3, torch.rand(shape) * 2
        q.set_range(lo, lo.clone() if i == 3 else hi)  # one empty range: the minimum scale applies
        qs.append(q)
    qs.append(Q.QuantizeDequantize((2,), 8, True))  # never initialised: no encoding
    lpbq = Q.GroupedBlockQuantizeDequantize((4, 2), 4, True, 8, block_size=(1, 8), block_grouping=(1, -1))
    lpbq.set_range(-torch.rand(4, 2) - 0.1, torch.rand(4, 2) + 0.1)
    if device == "cuda":
        qs.append(lpbq)  # a quantizer with rules of its own is asked directly (its scale runs a kernel)
    return [q.to(device) for q in qs]


def check_batched_derivation(device):
    from aimet_b200 import quantizer as Q

    qs = _mixed_quantizers(device)
    encs = Q.derive_encodings(qs)
    assert len(encs) == len(qs)
    for q, got in zip(qs, encs):
        want = q.get_encodings()
        if want is None:
            assert got is None
            continue
        assert type(got) is type(want)
        assert_same(got.scale, want.scale, "scale")
        assert_same(got.offset, want.offset, "offset")
        assert got.scale.shape == want.scale.shape and got.offset.shape == want.offset.shape
        assert (got.qmin, got.qmax, got.symmetry, got.block_size, got.zero_point_shift) == \
            (want.qmin, want.qmax, want.symmetry, want.block_size, want.zero_point_shift)
        assert getattr(got.offset, "_b200_constant", None) == getattr(want.offset, "_b200_constant", None)
        assert not got.scale.requires_grad and not got.offset.requires_grad


def test_batched_derivation_of_encodings():
    check_batched_derivation("cuda")
