"""SeqMSE on CUDA (tcgen05 reconstruction-loss kernel) against reference fixtures and the oracle."""

import pytest
import torch
import torch.nn.functional as F

from conftest import assert_same, load_golden
from oracle import seq_mse as OS

pytestmark = pytest.mark.gpu

CASES = load_golden("seqmse_cases.pt")
EXTRA = load_golden("seqmse_extra_cases.pt")


def _setup(c):
    from aimet_b200.quantizer import QuantizeDequantize
    from aimet_b200.seq_mse import QuantizedConv2d, QuantizedLinear

    layer = c.get("layer", ("linear",))
    if layer[0] == "conv":
        mod = QuantizedConv2d(layer[2], layer[1], layer[3], bias=False, **c["conv"]).to(c["dtype"]).cuda()
    else:
        co, ci = c["w"].shape
        mod = QuantizedLinear(ci, co, bias=False).to(c["dtype"]).cuda()
    with torch.no_grad():
        mod.weight.copy_(c["w"].cuda())
    q = QuantizeDequantize(c["qshape"], c["bitwidth"], True, block_size=c["block_size"]).cuda()
    mod.param_quantizers["weight"] = q
    with q.compute_encodings():
        q(mod.weight.data)
    return mod, q


def _decisive(losses, rel):
    """Channels whose two best candidates differ by more than ``rel`` of the loss."""
    flat = losses.double()
    top2 = flat.topk(2, dim=0, largest=False).values
    return (top2[1] - top2[0]).abs() > rel * top2[1].abs().clamp_min(1e-30)


def _float64_losses(c):
    """The losses of every candidate with the reference's quantized weights (oracle) and all
    products, differences and sums in float64."""
    steps = 2 ** c["bitwidth"] - 1
    qmin, qmax = -((steps + 1) // 2), steps // 2
    w = c["w"]
    conv = None
    if c.get("layer", ("linear",))[0] == "conv":
        conv = dict(stride=1, padding=0, dilation=1, groups=1)
        conv.update(c["conv"])
    in_block = w.shape[1] if c["block_size"] is None else w.shape[1] // c["min_before"].shape[1]
    xs, xqs = list(c["x"]), list(c.get("xq", c["x"]))
    out = []
    for i in range(c["num_candidates"]):
        cmin, cmax = OS.candidate(i, c["num_candidates"], c["min_before"], c["max_before"])
        emin, emax = OS.encodings_for_candidate(cmin, cmax, c["min_before"].shape, qmin, qmax, True)
        wq = OS.quantized_weight(w, emin, emax, qmin, qmax, True, c["block_size"])
        loss = 0
        for x, xq in zip(xs, xqs):
            if conv is None:
                loss = loss + OS.linear_loss(x.double(), xq.double(), w.double(), wq.double(), in_block, c["loss_fn"])
            else:
                loss = loss + OS.conv_loss(x.double(), xq.double(), w.double(), wq.double(), in_block, c["loss_fn"], **conv)
        out.append(loss)
    return torch.stack(out)


def _check_fp32_case(c):
    """float32 operands.  The kernel receives differences (x.w - xq.wq = xq.(w - wq) + (x - xq).w), so
    nothing cancels and its losses agree with a float64 evaluation to well below 1e-5.  The
    reference's own float32 result is itself up to 1e-5 away from that evaluation (it subtracts two
    nearly equal float32 products), hence the wider bound against the fixture."""
    from aimet_b200.seq_mse import SeqMseParams, SequentialMse

    mod, q = _setup(c)
    assert_same(q.get_min().detach(), c["min_before"], "range before the search")
    x, xq = c["x"].cuda(), c.get("xq", c["x"]).cuda()
    if "xq" not in c or c["xq"] is c["x"] or torch.equal(c["xq"], c["x"]):
        xq = x
    SequentialMse.optimize_module(mod, x, xq, SeqMseParams(num_batches=None, num_candidates=c["num_candidates"],
                                                            loss_fn=c["loss_fn"]))
    losses = SequentialMse.last_losses.cpu()
    want, exact = c["losses"], _float64_losses(c)
    assert losses.shape == want.shape
    if c["loss_fn"] == "sqnr":  # decibels: absolute tolerances (1e-5 relative of the ratio is 4.3e-5 dB)
        assert torch.allclose(losses.double(), exact, rtol=0, atol=5e-5), (losses.double() - exact).abs().max()
        assert torch.allclose(losses, want, rtol=0, atol=2e-4)
    else:
        assert torch.allclose(losses.double(), exact, rtol=1e-5, atol=0), ((losses.double() - exact).abs() / exact.abs()).max()
        assert torch.allclose(losses, want, rtol=2e-5, atol=0), ((losses - want).abs() / want.abs()).max()
    dec = _decisive(exact, 4e-5 if c["loss_fn"] != "sqnr" else 1e-6)
    assert torch.equal(losses.min(0)[1][dec], c["best"][dec])
    if torch.equal(losses.min(0)[1], c["best"]):
        assert_same(q.min.detach(), c["min_after"], "final min")
        assert_same(q.max.detach(), c["max_after"], "final max")
    assert not q.is_overwrite_allowed() and not q.min.requires_grad


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if c["dtype"] == torch.float32))
def test_optimize_module_fp32(name):
    _check_fp32_case(CASES[name])


@pytest.mark.parametrize("name", sorted(EXTRA))
def test_optimize_module_conv_blockwise_and_distinct_inputs(name):
    """Conv2d layers (per-channel, blockwise, grouped), blockwise Linear (all blocks in one
    launch) and inputs that differ between the floating-point and the quantized model."""
    _check_fp32_case(EXTRA[name])


def test_optimize_module_bf16():
    """bfloat16 operands: the reference accumulates its loss in bfloat16, so values are compared with
    a float64 evaluation on the same bfloat16 operands, and the chosen candidates with the
    reference's bfloat16 run on channels where the decision is clear of bfloat16 noise."""
    from aimet_b200.seq_mse import SeqMseParams, SequentialMse

    c = CASES["per_channel_int4_mse_bf16"]
    lin, q = _setup(c)
    x = c["x"].cuda()
    SequentialMse.optimize_module(lin, x, x, SeqMseParams(num_batches=None, num_candidates=c["num_candidates"]))
    losses = SequentialMse.last_losses.float().cpu()
    dec = _decisive(c["losses"].float(), 2 ** -6)
    assert torch.equal(losses.min(0)[1][dec], c["best"][dec])
    assert dec.float().mean() > 0.5
    want = _float64_losses(c)
    assert torch.allclose(losses.double(), want, rtol=1e-5, atol=0), ((losses.double() - want).abs() / want).max()


def _loss_reference(x, xq, w, wq, nb, fn):
    c, n, k = wq.shape
    kb = k // nb
    xw = torch.einsum("mbk,nbk->mnb", x.double().reshape(-1, nb, kb), w.double().reshape(n, nb, kb))
    y = torch.einsum("mbk,cnbk->cmnb", xq.double().reshape(-1, nb, kb), wq.double().reshape(c, n, nb, kb))
    d = xw[None] - y
    return (d ** 2).sum(1) if fn == "mse" else d.abs().sum(1)


def test_loss_kernel_shapes():
    """Ragged shapes: tokens / channels / K that are not multiples of the tile sizes, one CTA taking
    over a tile in the middle of its candidates, blocks narrower and wider than a pipeline stage."""
    from aimet_b200.seq_mse import block_losses_all_candidates

    g = torch.Generator().manual_seed(11)
    shapes = ((300, 130, 72, 3, 1), (1000, 260, 200, 2, 1), (17, 8, 64, 1, 1), (513, 384, 1024, 5, 1),
              (600, 200, 256, 3, 8), (300, 130, 192, 4, 2), (257, 129, 96, 7, 6), (2100, 1000, 128, 20, 2),
              (700, 300, 1024, 3, 2), (520, 512, 2048, 2, 4))  # blocks long enough for CTA pairs (odd / even tile counts)
    for m, n, k, c, nb in shapes:
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        xq = (x.float() + 0.02 * torch.randn(m, k, generator=g)).to(torch.bfloat16)
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
        wq = (w.float()[None] + 0.01 * torch.randn(c, n, k, generator=g)).to(torch.bfloat16)
        for fn in ("mse", "l1"):
            got = block_losses_all_candidates(x.cuda(), xq.cuda(), w.cuda(), wq.cuda(), nb, fn).cpu().double()
            want = _loss_reference(x, xq, w, wq, nb, fn)
            assert got.shape == want.shape
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-9), (fn, m, n, k, nb, ((got - want).abs() / want).max())
        xh, wh, wqh = x.half(), w.half(), wq.half()
        got16 = block_losses_all_candidates(xh.cuda(), xh.cuda(), wh.cuda(), wqh.cuda(), nb, "mse")
        assert torch.allclose(got16.cpu().double(), _loss_reference(xh, xh, wh, wqh, nb, "mse"), rtol=1e-5, atol=1e-9)


def test_float32_loss_at_a_long_contraction():
    """float32 operands at K = 4096 (the contraction length of a Llama-3-8B projection), inputs that
    differ between the two models: within 1e-5 of the float64 evaluation."""
    from aimet_b200.seq_mse import block_losses_all_candidates

    g = torch.Generator().manual_seed(12)
    m, n, k, c = 384, 96, 4096, 4
    x = torch.randn(m, k, generator=g)
    x[:, :20] *= 30
    xq = x + 0.01 * torch.randn(m, k, generator=g)
    w = torch.randn(n, k, generator=g) * 0.02
    scale = w.abs().amax(1, keepdim=True) / 7
    wq = torch.stack([torch.clamp(torch.round(w / (scale * f)), -8, 7) * (scale * f) for f in (0.4, 0.6, 0.8, 1.0)])
    for a, b in ((x, x), (x, xq)):
        for fn in ("mse", "l1"):
            got = block_losses_all_candidates(a.cuda(), a.cuda() if b is a else b.cuda(), w.cuda(), wq.cuda(), 1, fn)
            want = _loss_reference(a, b, w, wq, 1, fn)
            err = ((got.cpu().double() - want).abs() / want).max()
            assert err < 1e-5, (fn, float(err))
    # the same layer through 64 blocks of 64 input channels in one launch
    got = block_losses_all_candidates(x.cuda(), xq.cuda(), w.cuda(), wq.cuda(), 64, "mse").cpu().double()
    want = _loss_reference(x, xq, w, wq, 64, "mse")
    assert ((got - want).abs() / want).max() < 1e-5


def test_single_candidate_signatures():
    """_compute_linear_loss / _compute_conv_loss with the reference's signatures."""
    from aimet_b200.seq_mse import SeqMseParams, SequentialMse

    c = EXTRA["conv3x3_blockwise8_int4_mse_fp32"]
    mod, q = _setup(c)
    w = c["w"].cuda()
    wq = q(w).detach()
    params = SeqMseParams(num_batches=None, num_candidates=1, loss_fn="mse")
    got = SequentialMse._compute_loss(mod, c["x"][0].cuda(), c["xq"][0].cuda(), w, wq, params)
    want = OS.conv_loss(c["x"][0].double(), c["xq"][0].double(), c["w"].double(), wq.cpu().double(), 8, "mse",
                        stride=2, padding=1)
    assert got.shape == (24, 2) and got.dtype == torch.float32
    assert torch.allclose(got.cpu().double(), want, rtol=1e-5)


def test_bounded_wait_gives_up_and_reports():
    """The kernel's waits are bounded: a wait that nothing completes (a barrier no one arrives at)
    runs out after its limit, the status word is set and the kernel returns -- no fault, and the
    context stays usable."""
    from aimet_b200 import _lib

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib.aimet_b200_seqmse_wait_selftest(status.data_ptr(), 2000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 3
    # the device is still healthy
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
    from aimet_b200.seq_mse import _raise_on_status
    with pytest.raises(RuntimeError, match="gave up waiting"):
        _raise_on_status(status)


def test_second_device_in_one_process():
    """The kernel's shared-memory opt-in is a per-device attribute: a process that uses two GPUs must
    be able to launch on both."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from aimet_b200.seq_mse import block_losses_all_candidates

    g = torch.Generator().manual_seed(13)
    x = torch.randn(300, 128, generator=g).to(torch.bfloat16)
    w = (torch.randn(64, 128, generator=g) * 0.05).to(torch.bfloat16)
    wq = (w.float()[None] + 0.01 * torch.randn(2, 64, 128, generator=g)).to(torch.bfloat16)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        outs.append(block_losses_all_candidates(x.to(dev), x.to(dev), w.to(dev), wq.to(dev), 1, "mse").cpu())
    assert torch.equal(outs[0], outs[1])
