"""Parity at the full sizes of the benchmark configurations, against the CPU oracle on the same seeded
inputs: a float32 [4096, 4096] tensor under a per-tensor encoding, the [14336, 4096] bf16 MLP weight
under per-channel / blockwise / LPBQ encodings, a [16, 2048, 4096] bf16 activation batch through the
SQNR analyzer (collect + sequential update), and the SeqMSE loss of a [4096, 4096] projection on 8192
tokens (a subset of output channels, all 20 candidates)."""

import pytest
import torch

from conftest import assert_same
from oracle import affine as OA
from oracle import encoding_analyzer as OE
from oracle import quantizer as OQ
from oracle import seq_mse as OS

pytestmark = pytest.mark.gpu


def _grad_close(got, want, tol):
    want = want.reshape(got.shape).double()
    err = (got.double().cpu() - want).abs().max()
    assert err <= tol * want.abs().max().clamp_min(1e-30), float(err / want.abs().max())


def test_per_tensor_fp32_4096x4096():
    from aimet_b200.quantizer import QuantizeDequantize

    g = torch.Generator().manual_seed(1000)
    x, dy = torch.randn(4096, 4096, generator=g), torch.randn(4096, 4096, generator=g)
    q = QuantizeDequantize((), 8, False).cuda()
    xc = x.cuda().requires_grad_(True)
    with q.compute_encodings():
        q(xc.detach())
    y = q(xc)
    y.backward(dy.cuda())
    omn, omx = OE.minmax_collect(x, (), None)
    omn, omx = OE.minmax_encodings(omn, omx, 255, False)
    assert_same(q.min.detach(), omn.float().reshape(()), "calibrated min")
    assert_same(q.max.detach(), omx.float().reshape(()), "calibrated max")
    scale, offset = OQ.scale_offset_from_min_max(omn.float(), omx.float(), q.qmin, q.qmax, False)
    assert_same(y.detach(), OA.quantize_dequantize(x, scale, offset, q.qmin, q.qmax), "output")
    ogx, ogs, ogo = OA.quantize_dequantize_backward(x, dy, scale, offset, q.qmin, q.qmax)
    assert_same(xc.grad, ogx, "input gradient")
    # min / max gradients come from the scale / offset gradients through ordinary autograd: compare
    # those of the functional call
    from aimet_b200 import backend as B

    s = scale.cuda().requires_grad_(True)
    o = offset.cuda().requires_grad_(True)
    B.quantize_dequantize(x.cuda(), s, o, q.qmin, q.qmax).backward(dy.cuda())
    _grad_close(s.grad, ogs, 1e-5)
    assert float((o.grad.cpu() - ogo.reshape(o.grad.shape)).abs().max()) <= 1e-5 * max(1.0, float(ogo.abs().max()))


@pytest.mark.parametrize("variant", ["per_channel_int8", "blockwise_int4", "lpbq_int4"])
def test_mlp_weight_14336x4096_bf16(variant):
    from aimet_b200.quantizer import GroupedBlockQuantizeDequantize, QuantizeDequantize

    rows, cols, blk = 14336, 4096, 64
    g = torch.Generator().manual_seed(2000)
    w = torch.randn(rows, cols, generator=g) * 0.02
    w = (w * (1 + 19 * (torch.rand(rows, cols, generator=g) < 0.001))).to(torch.bfloat16)
    dy = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    if variant == "per_channel_int8":
        q, shape, bw, block = QuantizeDequantize((rows, 1), 8, True), (rows, 1), 8, None
    elif variant == "blockwise_int4":
        q, shape, bw, block = QuantizeDequantize((rows, cols // blk), 4, True, block_size=(1, blk)), (rows, cols // blk), 4, (1, blk)
    else:
        q = GroupedBlockQuantizeDequantize((rows, cols // blk), 4, True, decompressed_bw=8, block_size=(1, blk),
                                           block_grouping=(1, -1))
        shape, bw, block = (rows, cols // blk), 4, (1, blk)
    q = q.cuda()
    wc = w.cuda().requires_grad_(True)
    with q.compute_encodings():
        q(wc.detach())
    y = q(wc)
    y.backward(dy.cuda())
    steps = 2 ** bw - 1
    qmin, qmax = -((steps + 1) // 2), steps // 2
    mn, mx = OE.minmax_collect(w, shape, block)
    mn, mx = OE.minmax_encodings(mn, mx, steps, True)
    assert_same(q.min.detach(), mn.float().reshape(shape), "calibrated min")
    scale, offset = OQ.scale_offset_from_min_max(mn.float(), mx.float(), qmin, qmax, True)
    if variant == "lpbq_int4":
        scale, _ = OQ.lpbq_scale(scale, 4, 8, (1, -1))
    assert_same(y.detach(), OA.quantize_dequantize(w, scale, offset, qmin, qmax, block), "output")   # bit-exact
    ogx, ogs, _ = OA.quantize_dequantize_backward(w, dy, scale, offset, qmin, qmax, block)
    assert_same(wc.grad, ogx, "input gradient")                                                       # bit-exact
    # the scale gradient of the functional call (float32 internal dtype: 1e-5; bf16: one ulp of bf16)
    from aimet_b200 import backend as B

    s = scale.cuda().requires_grad_(True)
    B.quantize_dequantize(w.cuda(), s, offset.cuda(), qmin, qmax, block).backward(dy.cuda())
    if variant == "per_channel_int8":
        _grad_close(s.grad, ogs, 1e-5)
    else:
        a, b = s.grad.double().cpu(), ogs.reshape(s.grad.shape).double()
        assert bool(((a - b).abs() <= 2.0 ** -7 * torch.maximum(a.abs(), b.abs()) + 1e-30).all())


def _student_t(gen, hot):
    z = torch.randn((16 * 2048, 4096), generator=gen)
    chi = torch.randn((16 * 2048, 4096, 3), generator=gen).pow_(2).sum(-1)
    x = z / torch.sqrt(chi / 3)
    x[:, hot] *= 50
    return x.to(torch.bfloat16).view(16, 2048, 4096)


def test_activation_batches_16x2048x4096_through_the_sqnr_analyzer():
    from aimet_b200 import encoding_analyzer as EA

    gen = torch.Generator().manual_seed(3000)
    hot = torch.randperm(4096, generator=gen)[:32]
    x0, x1 = _student_t(gen, hot), _student_t(gen, hot) * 1.5
    an = EA.SqnrEncodingAnalyzer((), num_bins=2048)
    state = None

    def same_counts(got, want, what):
        # torch.histc keeps float32 counts: bins beyond 2^24 are inexact in the oracle itself
        g, w = got.double().cpu(), want.double()
        small = w < 2 ** 24
        assert bool((g[small] == w[small]).all()), what
        assert bool(((g[~small] - w[~small]).abs() <= 1e-6 * w[~small]).all()), what

    for i, x in enumerate((x0, x1)):
        an.update_stats(x.cuda())
        new = OE.hist_collect(x, (), 2048)
        state = OE.hist_merge(state, new, x, (), 2048)
        st = an.observer.get_stats()
        same_counts(st.histogram[0], state["stats"][0]["histogram"], f"update {i}: counts")
        assert_same(st.bin_edges[0], state["stats"][0]["bin_edges"], f"update {i}: edges")
        assert float(st.min[0]) == float(state["stats"][0]["min"]) and float(st.max[0]) == float(state["stats"][0]["max"])
    for steps, sym in ((255, False), (255, True)):
        gmin, gmax = an.compute_encodings(steps, sym)
        omin, omax = OE.sqnr_encodings(state["stats"], (), steps, sym)
        assert torch.allclose(gmin.double().cpu(), omin.double(), rtol=1e-5)
        assert torch.allclose(gmax.double().cpu(), omax.double(), rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_seqmse_projection_4096x4096_on_8192_tokens(dtype):
    """All 20 candidates of the reference's grid ((i + 1) / 20 of the range) and of a grid spread over
    [0.5 max, max], on the first output channels, against a float64 evaluation of the same operands.
    float32 operands: 1e-5.  bf16 operands: 1e-4 -- the tensor core truncates its float32 accumulator
    after each of the 256 steps of a K = 4096 contraction, which shrinks both products by up to
    256 * 2^-25 and the loss by a few times that (the reference's own bf16 evaluation rounds every
    product to bf16 and is 1e-2 away)."""
    from aimet_b200.seq_mse import block_losses_all_candidates

    m, n, k, c = 8192, 96, 4096, 20
    g = torch.Generator().manual_seed(5000)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[:20]] *= 30
    w = torch.randn(n, k, generator=g) * 0.02
    x, w = x.to(dtype), w.to(dtype)
    mx = w.float().abs().amax(1, keepdim=True)
    tol = 1e-5 if dtype == torch.float32 else 1e-4
    for grid in ("reference", "upper_half"):
        wqs = []
        for i in range(c):
            if grid == "reference":
                cmin, cmax = OS.candidate(i, c, -mx, mx)
            else:
                f = 0.5 + 0.5 * i / (c - 1)
                cmin, cmax = -mx * f, mx * f
            emin, emax = OS.encodings_for_candidate(cmin, cmax, (n, 1), -8, 7, True)
            wqs.append(OS.quantized_weight(w, emin, emax, -8, 7, True))
        wq = torch.stack(wqs)
        got = block_losses_all_candidates(x.cuda(), x.cuda(), w.cuda(), wq.cuda(), 1, "mse")[..., 0].cpu().double()
        xw = x.double() @ w.double().T
        want = torch.stack([((xw - x.double() @ wq[i].double().T) ** 2).sum(0) for i in range(c)])
        err = ((got - want).abs() / want).max()
        assert err <= tol, (grid, float(err))
        # the winners agree wherever the two best candidates are further apart than the tolerance
        top2 = want.topk(2, dim=0, largest=False).values
        decisive = (top2[1] - top2[0]) > 4 * tol * top2[1]
        assert torch.equal(got.argmin(0)[decisive], want.argmin(0)[decisive])
