"""Single-process (world size 1) checks of the sharding helpers on the CUDA kernels: the two-phase
histogram calibration equals one collect_stats call on the concatenated batches, and SeqMSE on row
shards reassembles to the unsharded result."""

import pytest
import torch

from conftest import assert_same
from oracle import encoding_analyzer as OA

pytestmark = pytest.mark.gpu


def _batches():
    g = torch.Generator().manual_seed(21)
    out = []
    for b in range(3):
        x = torch.randn(4, 64, 32, generator=g) * (1 + b)
        x[..., 5] *= 30
        out.append(x.to(torch.bfloat16))
    out[2][0, 0, 0] = -float("inf")
    return out


@pytest.mark.parametrize("shape", [(), (32,)])
def test_two_phase_histogram_equals_concatenated_collect(shape):
    from aimet_b200 import distributed as D
    from aimet_b200 import encoding_analyzer as EA

    batches = _batches()
    an = EA.SqnrEncodingAnalyzer(shape, num_bins=128)
    st = D.calibrate_histogram(an, [b.cuda() for b in batches])
    want = OA.hist_collect(torch.cat(batches, dim=0), shape, 128)
    for i, w in enumerate(want):
        assert_same(st[i].histogram, w["histogram"], f"histogram {i}")
        assert_same(st[i].bin_edges, w["bin_edges"], f"edges {i}")
        assert_same(st[i].min, w["min"], "min")
        assert_same(st[i].max, w["max"], "max")
    emin, emax = an.compute_encodings(255, False)
    omin, omax = OA.sqnr_encodings(want, shape, 255, False)
    assert torch.allclose(emin.cpu().float(), omin.float(), rtol=1e-5) and torch.allclose(emax.cpu().float(), omax.float(), rtol=1e-5)
    # the large-tensor kernel (replicated shared-memory counters) gives the same counts as the plain one
    big = torch.cat([b.flatten() for b in batches] * 40)[: 1 << 20].cuda().contiguous()
    an2 = EA.SqnrEncodingAnalyzer((), num_bins=128)
    st2 = D.calibrate_histogram(an2, [big, big[: 1 << 19]])
    ref = OA.hist_collect(torch.cat([big.cpu(), big[: 1 << 19].cpu()]), (), 128)[0]
    assert_same(st2[0].histogram, ref["histogram"], "large-tensor histogram")


def test_seqmse_on_row_shards_equals_unsharded():
    from aimet_b200 import distributed as D
    from aimet_b200.quantizer import QuantizeDequantize
    from aimet_b200.seq_mse import QuantizedLinear, SeqMseParams, SequentialMse

    torch.manual_seed(3)
    w = (torch.randn(96, 128) * 0.02).to(torch.bfloat16)
    x = torch.randn(1, 200, 128).to(torch.bfloat16).cuda()

    def build(rows):
        lin = QuantizedLinear(128, rows.shape[0], bias=False).to(torch.bfloat16).cuda()
        with torch.no_grad():
            lin.weight.copy_(rows.cuda())
        q = QuantizeDequantize((rows.shape[0], 1), 4, True).cuda()
        lin.param_quantizers["weight"] = q
        with q.compute_encodings():
            q(lin.weight.data)
        return lin, q

    full, qf = build(w)
    SequentialMse.optimize_module(full, x, x, SeqMseParams(num_batches=None))
    parts = []
    for r in range(3):
        lo, hi = D.shard_range(96, r, 3)
        lin, q = build(w[lo:hi])
        SequentialMse.optimize_module(lin, x, x, SeqMseParams(num_batches=None))
        parts.append((q.min.detach(), q.max.detach()))
    assert torch.equal(torch.cat([p[0] for p in parts]), qf.min.detach())
    assert torch.equal(torch.cat([p[1] for p in parts]), qf.max.detach())
    assert D.optimize_module_sharded(build(w)[0], x, x, SeqMseParams(num_batches=None)).shape[0] == 96
