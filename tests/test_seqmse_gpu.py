"""SeqMSE on CUDA (tcgen05 reconstruction-loss kernel) against reference fixtures and the oracle."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import seq_mse as OS

pytestmark = pytest.mark.gpu

CASES = load_golden("seqmse_cases.pt")


def _setup(c):
    from aimet_b200.quantizer import QuantizeDequantize
    from aimet_b200.seq_mse import QuantizedLinear

    co, ci = c["w"].shape
    lin = QuantizedLinear(ci, co, bias=False).to(c["dtype"]).cuda()
    with torch.no_grad():
        lin.weight.copy_(c["w"].cuda())
    q = QuantizeDequantize(c["qshape"], c["bitwidth"], True, block_size=c["block_size"]).cuda()
    lin.param_quantizers["weight"] = q
    with q.compute_encodings():
        q(lin.weight.data)
    return lin, q


def _decisive(losses, rel):
    """Channels whose two best candidates differ by more than ``rel`` of the loss."""
    flat = losses.double()
    top2 = flat.topk(2, dim=0, largest=False).values
    return (top2[1] - top2[0]).abs() > rel * top2[1].abs().clamp_min(1e-30)


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if c["dtype"] == torch.float32))
def test_optimize_module_fp32(name):
    """float32 operands.  The loss is a sum of squared differences of two nearly equal products, so
    float32 arithmetic -- the reference's as much as this kernel's -- is only good to about 1e-5
    relative to a float64 evaluation (measured: reference 5e-6..9e-6, this kernel 5e-6..2.5e-5).
    Losses are therefore compared at 5e-5; the chosen candidate must agree wherever the decision is
    not inside that noise, and the final encodings are then bit-identical."""
    from aimet_b200.seq_mse import SeqMseParams, SequentialMse

    c = CASES[name]
    lin, q = _setup(c)
    assert_same(q.get_min().detach(), c["min_before"], "range before the search")
    x = c["x"].cuda()
    best = SequentialMse.optimize_module(lin, x, x, SeqMseParams(num_batches=None, num_candidates=c["num_candidates"],
                                                                 loss_fn=c["loss_fn"]))
    losses = SequentialMse.last_losses.cpu()
    want = c["losses"]
    if c["loss_fn"] == "sqnr":
        assert torch.allclose(losses, want, rtol=5e-5, atol=2e-4)  # decibels: absolute tolerance
    else:
        assert torch.allclose(losses, want, rtol=5e-5, atol=0), ((losses - want).abs() / want.abs()).max()
    dec = _decisive(want, 1e-4 if c["loss_fn"] != "sqnr" else 1e-6)
    assert torch.equal(losses.min(0)[1][dec], c["best"][dec])
    if torch.equal(losses.min(0)[1], c["best"]):
        assert_same(q.min.detach(), c["min_after"], "final min")
        assert_same(q.max.detach(), c["max_after"], "final max")
    assert not q.is_overwrite_allowed() and not q.min.requires_grad


def test_optimize_module_bf16():
    """bfloat16 operands: the reference accumulates its loss in bfloat16, so values are compared with
    the reference run on float32 copies of the same bfloat16-valued operands, and the chosen
    candidates with the bfloat16 run on channels where the decision is clear of bfloat16 noise."""
    from aimet_b200.seq_mse import SeqMseParams, SequentialMse

    c = CASES["per_channel_int4_mse_bf16"]
    ref32 = CASES["per_channel_int4_mse_bf16_values_fp32"]
    lin, q = _setup(c)
    x = c["x"].cuda()
    SequentialMse.optimize_module(lin, x, x, SeqMseParams(num_batches=None, num_candidates=c["num_candidates"]))
    losses = SequentialMse.last_losses.float().cpu()
    # the bf16 weight quantization itself is bit-faithful, so the only difference to the float32
    # reference run is that run's float32 (not bf16-rounded) quantized weights
    dec = _decisive(c["losses"].float(), 2 ** -6)
    assert torch.equal(losses.min(0)[1][dec], c["best"][dec])
    assert dec.float().mean() > 0.5
    # against the oracle on the same bf16 operands, products in float64
    w, xb = c["w"].double(), c["x"].double().reshape(-1, c["w"].shape[1])
    steps = 15
    wants = []
    for i in range(c["num_candidates"]):
        cmin, cmax = OS.candidate(i, c["num_candidates"], c["min_before"], c["max_before"])
        emin, emax = OS.encodings_for_candidate(cmin, cmax, c["min_before"].shape, -8, 7, True)
        wq = OS.quantized_weight(c["w"], emin, emax, -8, 7, True).double()
        wants.append(((xb @ w.T - xb @ wq.T) ** 2).sum(0))
    want = torch.stack(wants)[..., None]
    assert torch.allclose(losses.double(), want, rtol=2e-5, atol=0), ((losses.double() - want).abs() / want).max()
    del ref32, steps


def test_loss_kernel_shapes():
    """Ragged shapes: tokens / channels / K that are not multiples of the tile sizes."""
    from aimet_b200.seq_mse import linear_loss_all_candidates

    g = torch.Generator().manual_seed(11)
    for m, n, k, c in ((300, 130, 72, 3), (1000, 260, 200, 2), (17, 8, 64, 1), (513, 384, 1024, 5)):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
        wq = (w.float()[None] + 0.01 * torch.randn(c, n, k, generator=g)).to(torch.bfloat16)
        for fn in ("mse", "l1"):
            got = linear_loss_all_candidates(x.cuda(), x.cuda(), w.cuda(), wq.cuda(), fn).cpu().double()
            xw = x.double() @ w.double().T
            y = torch.einsum("mk,cnk->cmn", x.double(), wq.double())
            d = xw[None] - y
            want = (d ** 2).sum(1) if fn == "mse" else d.abs().sum(1)
            assert torch.allclose(got, want, rtol=2e-5, atol=1e-9), (fn, m, n, k, ((got - want).abs() / want).max())
        got16 = linear_loss_all_candidates(x.half().cuda(), x.half().cuda(), w.half().cuda(), wq.half().cuda(), "mse")
        y = torch.einsum("mk,cnk->cmn", x.half().double(), wq.half().double())
        want = ((x.half().double() @ w.half().double().T)[None] - y).pow(2).sum(1)
        assert torch.allclose(got16.cpu().double(), want, rtol=2e-5, atol=1e-9)
