"""Two NCCL ranks on two GPUs (skipped on a single-GPU box): statistics and SeqMSE results of the
sharded computation equal the unsharded one computed by a rank on its own."""

import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from aimet_b200 import distributed as D
        from aimet_b200 import encoding_analyzer as EA
        from aimet_b200.quantizer import QuantizeDequantize
        from aimet_b200.seq_mse import QuantizedLinear, SeqMseParams, SequentialMse

        g = torch.Generator().manual_seed(31)
        batches = [(torch.randn(4, 512, 1024, generator=g) * (1 + b)).to(torch.bfloat16).to(dev) for b in range(6)]
        mine = [batches[i] for i in D.my_batches(len(batches), rank, world)]
        ok = {}
        for shape in ((), (1024,)):
            an = EA.SqnrEncodingAnalyzer(shape, num_bins=2048)
            D.calibrate_histogram(an, mine, dist.group.WORLD)
            alone = EA.SqnrEncodingAnalyzer(shape, num_bins=2048)
            D.calibrate_histogram(alone, batches, D.ALONE)
            a, b = an.observer.get_stats(), alone.observer.get_stats()
            ok[f"histogram{shape}"] = (torch.equal(a.histogram, b.histogram) and torch.equal(a.bin_edges, b.bin_edges)
                                       and torch.equal(a.min, b.min) and torch.equal(a.max, b.max))
            ea, eb = an.compute_encodings(255, False), alone.compute_encodings(255, False)
            ok[f"encodings{shape}"] = torch.equal(ea[0], eb[0]) and torch.equal(ea[1], eb[1])
        mm = EA.MinMaxEncodingAnalyzer((1024,))
        D.calibrate_minmax(mm, mine, dist.group.WORLD)
        mm1 = EA.MinMaxEncodingAnalyzer((1024,))
        D.calibrate_minmax(mm1, batches, D.ALONE)
        ok["minmax"] = torch.equal(mm.observer.get_stats().min, mm1.observer.get_stats().min) and torch.equal(
            mm.observer.get_stats().max, mm1.observer.get_stats().max)

        w = (torch.randn(200, 256, generator=g) * 0.02).to(torch.bfloat16)
        x = torch.randn(1, 700, 256, generator=g).to(torch.bfloat16).to(dev)

        def build():
            lin = QuantizedLinear(256, 200, bias=False).to(torch.bfloat16).to(dev)
            with torch.no_grad():
                lin.weight.copy_(w.to(dev))
            q = QuantizeDequantize((200, 1), 4, True).to(dev)
            lin.param_quantizers["weight"] = q
            with q.compute_encodings():
                q(lin.weight.data)
            return lin, q

        params = SeqMseParams(num_batches=None, num_candidates=10)
        lin, q = build()
        best = D.optimize_module_sharded(lin, x, x, params, dist.group.WORLD)
        lin1, q1 = build()
        best1 = SequentialMse.optimize_module(lin1, x, x, params)
        ok["seqmse"] = (torch.equal(best.reshape(-1), best1.reshape(-1)) and torch.equal(q.min, q1.min)
                        and torch.equal(q.max, q1.max))
        # data-parallel calibration of a model: each rank runs its share of the images through its
        # replica; one all-reduce combines the min / max statistics of all quantizers
        from torch import nn as tnn

        from aimet_b200 import nn as qnn

        def make_model():
            torch.manual_seed(5)
            net = tnn.Sequential(tnn.Conv2d(3, 8, 3, padding=1), tnn.ReLU(), tnn.Conv2d(8, 8, 3, padding=1), tnn.Flatten(),
                                 tnn.Linear(8 * 12 * 12, 10)).to(dev).eval()
            return qnn.quantize_model(net)

        images = torch.randn(8, 3, 12, 12, generator=g).to(dev)
        sharded, whole = make_model(), make_model()
        with torch.no_grad(), qnn.compute_encodings(sharded, group=dist.group.WORLD):
            sharded(images[rank::world])
        with torch.no_grad(), qnn.compute_encodings(whole):
            whole(images)
        same = True
        for a, b in zip(qnn.quantized_layers(sharded), qnn.quantized_layers(whole)):
            for qa, qb in ((a.input_quantizers[0], b.input_quantizers[0]), (a.output_quantizers[0], b.output_quantizers[0])):
                same = same and torch.equal(qa.min, qb.min) and torch.equal(qa.max, qb.max)
        ok["model_calibration"] = same
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_ranks_equal_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            if p.is_alive():
                p.terminate()
                pytest.fail("a rank did not finish")
        result = dict(ret)
    assert sorted(result) == [0, 1], result
    for rank, ok in result.items():
        assert all(ok.values()), (rank, ok)
