"""Generates the golden fixtures under tests/golden/ by running the aimet_torch reference itself.

Run where the reference checkout is available (CPU is enough):

    AIMET_REFERENCE_ROOT=<checkout> python tests/golden/make_golden.py [affine|backend_vectors|analyzers|quantizers|seqmse|seqmse_extra|float|wire ...]

Every fixture stores the seeded inputs next to the reference's outputs, so the tests that read
them need neither the reference nor this script.  Nothing here is imported by the product.
"""

from __future__ import annotations

import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import _reference_shim  # noqa: E402

_reference_shim.install()

import aimet_torch.quantization as Q  # noqa: E402
from aimet_torch.quantization.affine.backends import torch_builtins  # noqa: E402
from aimet_torch.quantization import encoding_analyzer as ref_ea  # noqa: E402


def _save(name, obj):
    path = os.path.join(HERE, name)
    torch.save(obj, path)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KiB)")


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


# --------------------------------------------------------------------------------------------
# known-answer vector sets of the reference's own backend test
# --------------------------------------------------------------------------------------------
def gen_backend_vectors():
    test_dir = os.path.join(
        _reference_shim.REFERENCE_ROOT, "TrainingExtensions/torch/test/python/v2/quantization/affine/backends"
    )
    sys.path.insert(0, test_dir)
    import test_backend as tb  # the reference's test module: source of the hand-written vectors

    out = {}
    for name in (
        "bfloat16_compat_per_tensor_4b_test_set",
        "bfloat16_compat_per_tensor_8b_test_set",
        "per_tensor_4b_test_set",
        "per_tensor_8b_test_set",
        "per_channel_4b_test_set",
        "per_channel_8b_test_set",
    ):
        vs = getattr(tb, name)
        out[name] = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in vs._asdict().items()}
    _save("backend_vectors.pt", out)


# --------------------------------------------------------------------------------------------
# affine functionals, forward + backward, through torch_builtins
# --------------------------------------------------------------------------------------------
AFFINE_CASES = [
    # name, dtype, shape, param shape, block_size, qmin, qmax, zero_point_shift, symmetric, also Q/DQ
    ("fp32_per_tensor_asym8", torch.float32, (48, 128), (), None, 0, 255, 0.0, False, True),
    ("fp32_per_tensor_odd", torch.float32, (7, 13), (), None, 0, 255, 0.0, False, True),
    ("bf16_per_channel_int8", torch.bfloat16, (56, 128), (56, 1), None, -128, 127, 0.0, True, True),
    ("bf16_blockwise_int4", torch.bfloat16, (24, 256), (24, 4), (1, 64), -8, 7, 0.0, True, True),
    ("bf16_per_tensor_int4", torch.bfloat16, (32, 100), (), None, 0, 15, 0.0, False, False),
    ("fp16_per_tensor_int8", torch.float16, (32, 152), (), None, 0, 255, 0.0, False, True),
    ("fp16_per_channel_int16", torch.float16, (16, 64), (16, 1), None, 0, 65535, 0.0, False, False),
    ("fp32_channel_axis1_4d", torch.float32, (4, 6, 5, 7), (6, 1, 1), None, 0, 255, 0.0, False, True),
    ("fp32_channel_axis1_4d_big", torch.float32, (5, 8, 12, 8), (8, 1, 1), None, -128, 127, 0.0, True, False),
    ("fp32_channel_last", torch.float32, (67, 48), (48,), None, 0, 255, 0.0, False, True),
    ("bf16_channel_last", torch.bfloat16, (65, 136), (136,), None, -128, 127, 0.0, True, False),
    ("fp32_blocks_2d", torch.float32, (8, 12), (4, 3), (2, 4), 0, 15, 0.0, False, True),
    ("fp32_blocks_wildcard", torch.float32, (6, 2, 8, 10), (2, 2, 5), (1, -1, 2), 0, 255, 0.0, False, True),
    ("fp32_blockwise_small", torch.float32, (16, 24), (16, 6), (1, 4), -8, 7, 0.0, True, False),
    ("fp32_zero_point_shift", torch.float32, (64, 64), (64, 1), None, -8, 7, 0.5, True, False),
    ("bf16_zero_point_shift_int4", torch.bfloat16, (32, 128), (32, 2), (1, 64), -8, 7, 0.5, True, False),
    ("fp32_int32_grid", torch.float32, (16, 64), (), None, -(2**31), 2**31 - 1, 0.0, True, False),
    ("fp64_per_tensor", torch.float64, (16, 33), (), None, 0, 255, 0.0, False, True),
    ("fp32_long_rows", torch.float32, (3, 2600), (3, 1), None, -128, 127, 0.0, True, False),
]


def _make_affine_inputs(seed, dtype, shape, pshape, qmin, qmax, symmetric):
    g = _gen(seed)
    x = torch.randn(shape, generator=g)
    x = x * (1 + 4 * (torch.rand(shape, generator=g) < 0.01))  # a few outliers -> clipping
    x = x.to(dtype)
    grad = torch.randn(shape, generator=g).to(dtype)
    steps = qmax - qmin
    base = 6.0 / steps
    scale = base * (0.5 + torch.rand(pshape, generator=g))
    if symmetric:
        offset = torch.full(pshape, float(-round((qmin + qmax) / 2)))
    else:
        offset = torch.round(-steps * (0.3 + 0.4 * torch.rand(pshape, generator=g))) - qmin
    return x, grad, scale.to(torch.float32), offset.to(torch.float32)


def gen_affine():
    out = {}
    for idx, (name, dtype, shape, pshape, block, qmin, qmax, zps, sym, also_q) in enumerate(AFFINE_CASES):
        x, grad, scale, offset = _make_affine_inputs(100 + idx, dtype, shape, pshape, qmin, qmax, sym)
        rec = dict(dtype=dtype, shape=shape, pshape=pshape, block_size=block, qmin=qmin, qmax=qmax,
                   zero_point_shift=zps, x=x, grad=grad, scale=scale, offset=offset)

        def run(fn, inp, *args):
            xi = inp.clone().requires_grad_(True)
            s = scale.clone().requires_grad_(True)
            o = offset.clone().requires_grad_(True)
            y = fn(xi, s, o, *args)
            y.backward(grad)
            return y.detach(), xi.grad, s.grad, o.grad

        y, gx, gs, go = run(torch_builtins.quantize_dequantize, x, qmin, qmax, block, zps)
        rec.update(qdq=y, qdq_gx=gx, qdq_gs=gs, qdq_go=go)
        if also_q and zps == 0.0 and torch_builtins._is_grid_representable(dtype, qmin, qmax):
            q, gx, gs, go = run(torch_builtins.quantize, x, qmin, qmax, block)
            rec.update(q=q, q_gx=gx, q_gs=gs, q_go=go)
            dq, gx, gs, go = run(torch_builtins.dequantize, q, block)
            rec.update(dq=dq, dq_gx=gx, dq_gs=gs, dq_go=go)
        out[name] = rec
    _save("affine_cases.pt", out)


PGS_CASES = [
    # affine case it shares inputs with, eps, multiplier, parameter gradients wanted
    ("fp32_per_tensor_asym8", 0.05, 3.0, True),
    ("bf16_per_channel_int8", 0.2, 2.0, True),
    ("bf16_blockwise_int4", 0.5, 0.25, True),
    ("fp16_per_tensor_int8", 0.05, 3.0, False),
    ("fp32_zero_point_shift", 1.0, 5.0, True),
    ("fp32_channel_axis1_4d", 0.1, -1.5, False),
]


def gen_pgs():
    """quantize_dequantize backward with the experimental gradient multiplier near rounding
    boundaries switched on (experimental/pgs.py)."""
    from aimet_torch.experimental import pgs

    cases = {c[0]: (i, c) for i, c in enumerate(AFFINE_CASES)}
    out = {}
    for name, eps, mult, param_grads in PGS_CASES:
        idx, (_, dtype, shape, pshape, block, qmin, qmax, zps, sym, _q) = cases[name]
        x, grad, scale, offset = _make_affine_inputs(100 + idx, dtype, shape, pshape, qmin, qmax, sym)
        xi = x.clone().requires_grad_(True)
        s = scale.clone().requires_grad_(param_grads)
        o = offset.clone().requires_grad_(param_grads)
        pgs.enable_pgs(eps, mult)
        try:
            y = torch_builtins.quantize_dequantize(xi, s, o, qmin, qmax, block, zps)
        finally:
            pgs.disable_pgs()
        y.backward(grad)  # the switch is read when the forward runs
        out[name] = dict(dtype=dtype, shape=shape, pshape=pshape, block_size=block, qmin=qmin, qmax=qmax,
                         zero_point_shift=zps, eps=eps, multiplier=mult, param_grads=param_grads, x=x, grad=grad,
                         scale=scale, offset=offset, y=y.detach(), gx=xi.grad, gs=s.grad, go=o.grad)
    _save("pgs_cases.pt", out)


# --------------------------------------------------------------------------------------------
# encoding analyzers: statistics after every update and the encodings computed from them
# --------------------------------------------------------------------------------------------
def _student_t(g, shape, df=3.0):
    """Student-t samples from normals only (torch.distributions ignores generators)."""
    z = torch.randn(shape, generator=g)
    chi = torch.randn((*shape, int(df)), generator=g).pow(2).sum(-1)
    return z / torch.sqrt(chi / df)


def _analyzer_batches(kind, dtype, seed):
    g = _gen(seed)
    if kind == "activation":  # heavy tails + a few hot channels, later batches widen the range
        xs = []
        for b in range(3):
            x = _student_t(g, (4, 48, 32))
            x[..., [3, 17]] *= 50.0
            xs.append((x * (1.0 + 0.7 * b)).to(dtype))
        return xs
    if kind == "weight":
        w = torch.randn((12, 96), generator=g) * 0.02
        w = w * (1 + 19 * (torch.rand((12, 96), generator=g) < 0.01))
        return [w.to(dtype), (w * 0.5).to(dtype)]
    if kind == "inf":
        x = torch.randn((4, 500), generator=g)
        x[0, 0], x[1, 1], x[2, 2] = float("inf"), -float("inf"), float("inf")
        return [x.to(dtype), (2 * torch.randn((4, 500), generator=g)).to(dtype)]
    if kind == "constant":
        return [torch.full((3, 40), 1.25).to(dtype), torch.full((3, 40), 1.25).to(dtype),
                torch.randn((3, 40), generator=g).to(dtype)]
    if kind == "shrinking":  # later batches inside the first range: the histogram is carried over
        x = torch.randn((8, 256), generator=g)
        return [x.to(dtype), (0.5 * x).to(dtype), (0.25 * torch.randn((8, 256), generator=g)).to(dtype)]
    raise ValueError(kind)


ANALYZER_CASES = [
    # name, analyzer, kwargs, shape, block_size, data kind, dtype
    ("minmax_per_tensor_fp32", "minmax", {}, (), None, "activation", torch.float32),
    ("minmax_per_tensor_bf16", "minmax", {}, (), None, "activation", torch.bfloat16),
    ("minmax_per_channel_bf16", "minmax", {}, (12, 1), None, "weight", torch.bfloat16),
    ("minmax_last_dim_fp32", "minmax", {}, (32,), None, "activation", torch.float32),
    ("minmax_blockwise_fp32", "minmax", {}, (12, 3), (1, 32), "weight", torch.float32),
    ("minmax_constant", "minmax", {}, (), None, "constant", torch.float32),
    ("sqnr_per_tensor_fp32", "sqnr", dict(num_bins=2048), (), None, "activation", torch.float32),
    ("sqnr_per_tensor_bf16", "sqnr", dict(num_bins=2048), (), None, "activation", torch.bfloat16),
    ("sqnr_per_tensor_fp16", "sqnr", dict(num_bins=512), (), None, "shrinking", torch.float16),
    ("sqnr_per_channel_fp32", "sqnr", dict(num_bins=256), (12, 1), None, "weight", torch.float32),
    ("sqnr_blockwise_bf16", "sqnr", dict(num_bins=64), (12, 3), (1, 32), "weight", torch.bfloat16),
    ("sqnr_inf_fp32", "sqnr", dict(num_bins=128), (), None, "inf", torch.float32),
    ("sqnr_constant_bf16", "sqnr", dict(num_bins=32), (), None, "constant", torch.bfloat16),
    ("sqnr_100_sym_candidates", "sqnr", dict(num_bins=2048, symmetric_delta_candidates=100), (), None, "activation", torch.bfloat16),
    ("tfe_per_tensor_fp32", "tfe", {}, (), None, "activation", torch.float32),
    ("tfe_per_tensor_bf16", "tfe", {}, (), None, "activation", torch.bfloat16),
    ("tfe_last_dim_fp32", "tfe", {}, (32,), None, "activation", torch.float32),
    ("percentile_99_fp32", "percentile", dict(num_bins=2048, percentile=99), (), None, "activation", torch.float32),
    ("percentile_999_bf16", "percentile", dict(num_bins=2048, percentile=99.9), (), None, "activation", torch.bfloat16),
    ("percentile_100_fp32", "percentile", dict(num_bins=100, percentile=100), (12, 1), None, "weight", torch.float32),
    ("percentile_shrinking", "percentile", dict(num_bins=50, percentile=90), (), None, "shrinking", torch.float32),
]

ENCODING_GRIDS = [(255, False), (255, True), (15, True), (15, False), (3, True), (254, True), (65535, False)]


def _make_ref_analyzer(kind, kwargs, shape, block):
    if kind == "minmax":
        return ref_ea.MinMaxEncodingAnalyzer(shape, block_size=block)
    if kind == "sqnr":
        return ref_ea.SqnrEncodingAnalyzer(shape, block_size=block, **kwargs)
    if kind == "tfe":
        return ref_ea.TfEnhancedEncodingAnalyzer(shape, block_size=block)
    if kind == "percentile":
        return ref_ea.PercentileEncodingAnalyzer(shape, block_size=block, **kwargs)
    raise ValueError(kind)


def _stats_to_plain(stats):
    if isinstance(stats, list):
        return [dict(histogram=h.histogram.clone(), bin_edges=h.bin_edges.clone(), min=h.min.clone(), max=h.max.clone())
                for h in stats]
    return dict(min=stats.min.clone(), max=stats.max.clone())


def gen_analyzers():
    import warnings

    out = {}
    for idx, (name, kind, kwargs, shape, block, data, dtype) in enumerate(ANALYZER_CASES):
        batches = _analyzer_batches(data, dtype, 500 + idx)
        an = _make_ref_analyzer(kind, kwargs, shape, block)
        rec = dict(kind=kind, kwargs=kwargs, shape=shape, block_size=block, batches=batches, updates=[])
        for x in batches:
            ret = an.update_stats(x)
            rec["updates"].append(dict(returned=_stats_to_plain(ret), merged=_stats_to_plain(an.observer.get_stats())))
        rec["encodings"] = {}
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for num_steps, sym in ENCODING_GRIDS:
                mn, mx = an.compute_encodings(num_steps, sym)
                rec["encodings"][(num_steps, sym)] = (mn.clone(), mx.clone())
        out[name] = rec
    _save("analyzer_cases.pt", out)


LPNORM_CASES = [
    # name, p, num_bins, shape, data kind, dtype
    ("lp1_per_tensor_fp32", 1.0, 512, (), "activation", torch.float32),
    ("lp3_per_tensor_bf16", 3.0, 512, (), "activation", torch.bfloat16),
    ("lp2p5_per_channel_fp32", 2.5, 128, (12, 1), "weight", torch.float32),
    ("lp0p5_per_tensor_fp32", 0.5, 256, (), "shrinking", torch.float32),
]


def gen_lpnorm():
    """The range search with an error exponent other than 2 (the analyzer behind SqnrEncodingAnalyzer
    with ``p`` set freely): histograms, the noise of every candidate, the chosen range."""
    out = {}
    for idx, (name, p, bins, shape, data, dtype) in enumerate(LPNORM_CASES):
        batches = _analyzer_batches(data, dtype, 900 + idx)
        an = ref_ea._LpNormEncodingAnalyzer(shape, bins, p=p, asymmetric_delta_candidates=17, symmetric_delta_candidates=101,
                                            offset_candidates=21, max_parallelism=64, gamma=3.0)
        for x in batches:
            an.update_stats(x)
        stats = an.observer.get_stats()
        rec = dict(p=p, num_bins=bins, shape=shape, batches=batches, stats=_stats_to_plain(stats), grids={})
        for num_steps, sym in ((255, False), (255, True), (15, False)):
            deltas, offsets = an._pick_test_candidates(stats, num_steps, sym)
            noise = an._estimate_clip_and_quant_noise(stats, deltas, offsets, num_steps, p, 3.0)
            mn, mx = an.compute_encodings(num_steps, sym)
            rec["grids"][(num_steps, sym)] = dict(deltas=deltas.clone(), offsets=offsets.clone(), noise=noise.clone(),
                                                  min=mn.clone(), max=mx.clone())
        out[name] = rec
    _save("lpnorm_cases.pt", out)


# --------------------------------------------------------------------------------------------
# quantizer modules: calibrate, forward, backward
# --------------------------------------------------------------------------------------------
QUANTIZER_CASES = [
    # name, class, ctor kwargs, analyzer, dtype, input shape
    ("qdq_per_tensor_asym8_fp32", "QuantizeDequantize", dict(shape=(), bitwidth=8, symmetric=False), None, torch.float32, (64, 256)),
    ("qdq_per_channel_sym8_bf16", "QuantizeDequantize", dict(shape=(56, 1), bitwidth=8, symmetric=True), None, torch.bfloat16, (56, 128)),
    ("qdq_blockwise_sym4_bf16", "QuantizeDequantize", dict(shape=(24, 4), bitwidth=4, symmetric=True, block_size=(1, 32)), None, torch.bfloat16, (24, 128)),
    ("lpbq_sym4_bf16", "GroupedBlockQuantizeDequantize", dict(shape=(24, 4), bitwidth=4, symmetric=True, decompressed_bw=8, block_size=(1, 32), block_grouping=(1, -1)), None, torch.bfloat16, (24, 128)),
    ("lpbq_sym4_fp32", "GroupedBlockQuantizeDequantize", dict(shape=(16, 8), bitwidth=4, symmetric=True, decompressed_bw=8, block_size=(1, 16), block_grouping=(1, 4)), None, torch.float32, (16, 128)),
    ("q_per_tensor_asym8_fp32", "Quantize", dict(shape=(), bitwidth=8, symmetric=False), None, torch.float32, (32, 100)),
    ("qdq_sqnr_asym8_fp32", "QuantizeDequantize", dict(shape=(), bitwidth=8, symmetric=False), "sqnr", torch.float32, (64, 256)),
    ("qdq_zps_sym4_fp32", "QuantizeDequantize", dict(shape=(32, 1), bitwidth=4, symmetric=True, zero_point_shift=0.5), None, torch.float32, (32, 64)),
    ("qdq_per_tensor_asym8_fp16", "QuantizeDequantize", dict(shape=(), bitwidth=8, symmetric=False), None, torch.float16, (32, 160)),
    ("qdq_per_tensor_sym16_bf16", "QuantizeDequantize", dict(shape=(), bitwidth=16, symmetric=True), None, torch.bfloat16, (32, 160)),
]


def gen_quantizers():
    from aimet_torch.quantization import affine as ref_affine

    out = {}
    for idx, (name, cls, kwargs, analyzer, dtype, shape) in enumerate(QUANTIZER_CASES):
        g = _gen(900 + idx)
        x = torch.randn(shape, generator=g) * 0.5
        x = (x * (1 + 9 * (torch.rand(shape, generator=g) < 0.005))).to(dtype)
        grad = torch.randn(shape, generator=g).to(dtype)
        kw = dict(kwargs)
        if analyzer == "sqnr":
            kw["encoding_analyzer"] = ref_ea.SqnrEncodingAnalyzer(kw["shape"])
        q = getattr(ref_affine, cls)(**kw)
        with q.compute_encodings():
            dyn = q(x)
        rec = dict(cls=cls, kwargs=kwargs, analyzer=analyzer, x=x, grad=grad,
                   dynamic_out=dyn.detach().as_subclass(torch.Tensor).clone(),
                   min=q.min.detach().clone(), max=q.max.detach().clone())
        xi = x.clone().requires_grad_(True)
        y = q(xi)
        y.backward(grad)
        rec.update(out=y.detach().as_subclass(torch.Tensor).clone(), grad_x=xi.grad.clone(),
                   grad_min=q.min.grad.clone(), grad_max=q.max.grad.clone(),
                   scale=q.get_scale().detach().clone(), offset=q.get_offset().detach().clone())
        out[name] = rec
    _save("quantizer_cases.pt", out)


# --------------------------------------------------------------------------------------------
# SeqMSE: optimize_module on a Linear layer
# --------------------------------------------------------------------------------------------
SEQMSE_CASES = [
    # name, dtype, (out, in), quantizer shape, block_size, bitwidth, loss_fn, num_candidates, x shape (batches first)
    ("per_channel_int4_mse_fp32", torch.float32, (48, 64), (48, 1), None, 4, "mse", 20, (2, 24, 64)),
    ("per_channel_int4_l1_fp32", torch.float32, (48, 64), (48, 1), None, 4, "l1", 20, (2, 24, 64)),
    ("per_channel_int4_sqnr_fp32", torch.float32, (48, 64), (48, 1), None, 4, "sqnr", 20, (2, 24, 64)),
    ("per_tensor_int4_mse_fp32", torch.float32, (48, 64), (), None, 4, "mse", 10, (2, 24, 64)),
    ("blockwise_int4_mse_fp32", torch.float32, (48, 64), (48, 4), (-1, -1), 4, "mse", 20, (2, 24, 64)),
    ("per_channel_int4_mse_bf16", torch.bfloat16, (64, 128), (64, 1), None, 4, "mse", 20, (1, 256, 128)),
    ("per_channel_int4_mse_bf16_values_fp32", torch.float32, (64, 128), (64, 1), None, 4, "mse", 20, (1, 256, 128)),
]


def gen_seqmse():
    from aimet_torch.nn import QuantizationMixin
    from aimet_torch.quantization.affine import QuantizeDequantize
    from aimet_torch.seq_mse import SequentialMse, SeqMseParams

    out = {}
    for idx, (name, dtype, (co, ci), qshape, block, bw, loss_fn, ncand, xshape) in enumerate(SEQMSE_CASES):
        g = _gen(1300 + (idx if "values_fp32" not in name else idx - 1))
        w = torch.randn(co, ci, generator=g) * 0.02
        x = torch.randn(xshape, generator=g)
        x[..., :2] *= 30.0
        if dtype == torch.bfloat16 or "values_fp32" in name:
            w, x = w.to(torch.bfloat16), x.to(torch.bfloat16)  # bf16-representable values
        w, x = w.to(dtype), x.to(dtype)
        linear = torch.nn.Linear(ci, co, bias=False).to(dtype)
        with torch.no_grad():
            linear.weight.copy_(w)
        qlin = QuantizationMixin.from_module(linear)
        qtz = QuantizeDequantize(shape=qshape, bitwidth=bw, symmetric=True, block_size=block)
        qlin.param_quantizers["weight"] = qtz
        with qtz.compute_encodings():
            qtz(qlin.weight.data)
        min_t, max_t = qtz.get_min().detach().clone(), qtz.get_max().detach().clone()
        captured = []
        orig = SequentialMse._compute_loss.__func__

        def spy(cls, *a, **k):
            r = orig(cls, *a, **k)
            captured.append(r.detach().clone())
            return r

        SequentialMse._compute_loss = classmethod(spy)
        try:
            SequentialMse.optimize_module(qlin, x, x, SeqMseParams(num_batches=None, num_candidates=ncand, loss_fn=loss_fn))
        finally:
            SequentialMse._compute_loss = classmethod(orig)
        nb = xshape[0]
        losses = torch.stack([sum(captured[c * nb:(c + 1) * nb]) for c in range(ncand)])
        out[name] = dict(dtype=dtype, w=w, x=x, qshape=qshape, block_size=block, bitwidth=bw, loss_fn=loss_fn,
                         num_candidates=ncand, min_before=min_t, max_before=max_t, losses=losses,
                         best=losses.min(0)[1], min_after=qtz.min.detach().clone(), max_after=qtz.max.detach().clone())
    _save("seqmse_cases.pt", out)


# name, dtype, layer, conv args, quantizer shape, block size, bitwidth, loss, candidates, x shape, xq differs
SEQMSE_EXTRA_CASES = [
    ("linear_int4_mse_fp32_distinct_inputs", torch.float32, ("linear", 48, 64), {}, (48, 1), None, 4, "mse", 8,
     (2, 50, 64), True),
    ("linear_blockwise16_int4_mse_fp32_distinct_inputs", torch.float32, ("linear", 32, 64), {}, (32, 4), (1, 16), 4,
     "mse", 6, (2, 40, 64), True),
    ("conv3x3_per_channel_int4_mse_fp32", torch.float32, ("conv", 24, 16, 3), dict(stride=1, padding=1), (24, 1, 1, 1),
     None, 4, "mse", 8, (2, 2, 16, 10, 10), True),
    ("conv3x3_blockwise8_int4_mse_fp32", torch.float32, ("conv", 24, 16, 3), dict(stride=2, padding=1), (24, 2, 1, 1),
     (1, 8, 3, 3), 4, "mse", 6, (2, 2, 16, 11, 11), False),
    ("conv3x3_groups2_int4_sqnr_fp32", torch.float32, ("conv", 24, 16, 3), dict(stride=1, padding=0, groups=2),
     (24, 1, 1, 1), None, 4, "sqnr", 6, (1, 3, 16, 9, 9), True),
    ("conv1x1_per_channel_int8_l1_fp32", torch.float32, ("conv", 20, 32, 1), dict(stride=1, padding=0), (20, 1, 1, 1),
     None, 8, "l1", 5, (1, 4, 32, 7, 7), True),
]


def gen_seqmse_extra():
    """SeqMSE fixtures for Conv2d layers, blockwise Linear and inputs that differ between the
    floating-point and the quantized model."""
    from aimet_torch.nn import QuantizationMixin
    from aimet_torch.quantization.affine import QuantizeDequantize
    from aimet_torch.seq_mse import SequentialMse, SeqMseParams

    out = {}
    for idx, (name, dtype, layer, conv, qshape, block, bw, loss_fn, ncand, xshape, distinct) in enumerate(SEQMSE_EXTRA_CASES):
        g = _gen(1400 + idx)
        if layer[0] == "linear":
            mod = torch.nn.Linear(layer[2], layer[1], bias=False)
        else:
            mod = torch.nn.Conv2d(layer[2], layer[1], layer[3], bias=False, **conv)
        w = torch.randn(mod.weight.shape, generator=g) * 0.05
        x = torch.randn(xshape, generator=g)
        xq = x + 0.02 * torch.randn(xshape, generator=g) if distinct else x
        w, x, xq = w.to(dtype), x.to(dtype), xq.to(dtype)
        with torch.no_grad():
            mod.weight.copy_(w)
        qmod = QuantizationMixin.from_module(mod.to(dtype))
        qtz = QuantizeDequantize(shape=qshape, bitwidth=bw, symmetric=True, block_size=block)
        qmod.param_quantizers["weight"] = qtz
        with qtz.compute_encodings():
            qtz(qmod.weight.data)
        min_t, max_t = qtz.get_min().detach().clone(), qtz.get_max().detach().clone()
        captured = []
        orig = SequentialMse._compute_loss.__func__

        def spy(cls, *a, **k):
            r = orig(cls, *a, **k)
            captured.append(r.detach().clone())
            return r

        SequentialMse._compute_loss = classmethod(spy)
        try:
            SequentialMse.optimize_module(qmod, x, xq, SeqMseParams(num_batches=None, num_candidates=ncand, loss_fn=loss_fn))
        finally:
            SequentialMse._compute_loss = classmethod(orig)
        nb = xshape[0]
        losses = torch.stack([sum(captured[c * nb:(c + 1) * nb]) for c in range(ncand)])
        out[name] = dict(dtype=dtype, layer=layer, conv=conv, w=w, x=x, xq=xq, qshape=qshape, block_size=block,
                         bitwidth=bw, loss_fn=loss_fn, num_candidates=ncand, min_before=min_t, max_before=max_t,
                         losses=losses, best=losses.min(0)[1], min_after=qtz.min.detach().clone(),
                         max_after=qtz.max.detach().clone())
    _save("seqmse_extra_cases.pt", out)


# name, constructor kwargs, input dtype, input shape, quantizer shape, block size, class
FLOAT_CASES = [
    ("fp16_per_tensor", dict(dtype=torch.float16), torch.float32, (64, 96), (), None, "float"),
    ("bf16_per_tensor", dict(dtype=torch.bfloat16), torch.float32, (64, 96), (), None, "float"),
    ("e4m3fn_per_tensor", dict(dtype=torch.float8_e4m3fn), torch.float32, (64, 96), (), None, "float"),
    ("e4m3fn_per_tensor_bf16_input", dict(dtype=torch.float8_e4m3fn), torch.bfloat16, (64, 96), (), None, "float"),
    ("e4m3fn_per_tensor_fp16_input", dict(dtype=torch.float8_e4m3fn), torch.float16, (64, 96), (), None, "float"),
    ("e5m2_per_channel", dict(dtype=torch.float8_e5m2), torch.float32, (48, 80), (48, 1), None, "float"),
    ("e5m2_per_channel_bf16_input", dict(dtype=torch.float8_e5m2), torch.bfloat16, (48, 80), (48, 1), None, "float"),
    ("e4m3fnuz_blockwise", dict(dtype=torch.float8_e4m3fnuz), torch.float32, (32, 128), (32, 4), (1, 32), "float"),
    ("e5m2fnuz_per_tensor", dict(dtype=torch.float8_e5m2fnuz), torch.float32, (64, 96), (), None, "float"),
    ("e4m3_ieee_per_tensor", dict(exponent_bits=4, mantissa_bits=3), torch.float32, (64, 96), (), None, "float"),
    ("e4m3_ieee_per_tensor_bf16_input", dict(exponent_bits=4, mantissa_bits=3), torch.bfloat16, (64, 96), (), None, "float"),
    ("e3m4_ieee_per_channel", dict(exponent_bits=3, mantissa_bits=4), torch.float32, (48, 80), (48, 1), None, "float"),
    ("e5m6_ieee_per_tensor_fp16_input", dict(exponent_bits=5, mantissa_bits=6), torch.float16, (64, 96), (), None, "float"),
    ("fp4_e2m1_blockwise", dict(exponent_bits=2, mantissa_bits=1, finite=True), torch.float32, (32, 128), (32, 4), (1, 32), "float"),
    ("mxfp4_blocks_of_32", {}, torch.float32, (16, 256), (16, 8), (1, 32), "mxfp4"),
    ("nvfp4_blocks_of_16", {}, torch.float32, (16, 256), (16, 16), (1, 16), "nvfp4"),
]


def gen_float():
    """Float fake-cast quantizers: calibrated on the input, then applied to it and to a second tensor
    with values beyond the calibrated range, infinities, NaN, zeros of both signs and tiny values."""
    from aimet_torch.quantization.float import FloatQuantizeDequantize
    from aimet_torch.quantization.float.quantizer import _MXFP4QuantizeDequantize, _NVFP4QuantizeDequantize

    out = {}
    for idx, (name, kw, in_dtype, xshape, qshape, block, kind) in enumerate(FLOAT_CASES):
        g = _gen(1500 + idx)
        x = torch.randn(xshape, generator=g) * torch.exp(torch.randn(xshape[0], 1, generator=g))
        x2 = torch.randn(xshape, generator=g) * 4
        flat = x2.view(-1)
        flat[:12] = torch.tensor([float("inf"), -float("inf"), float("nan"), 0.0, -0.0, 1e-30, -1e-30, 1e30, -1e30, 1e-6,
                                  1.0, -2.0])
        x, x2 = x.to(in_dtype), x2.to(in_dtype)
        if kind == "mxfp4":
            q = _MXFP4QuantizeDequantize(qshape, block)
        elif kind == "nvfp4":
            q = _NVFP4QuantizeDequantize(qshape, block)
        else:
            q = FloatQuantizeDequantize(shape=qshape, block_size=block, **kw)
        with q.compute_encodings():
            dyn = q(x)
        y, y2 = q(x), q(x2)
        out[name] = dict(kwargs=kw, kind=kind, in_dtype=in_dtype, x=x, x2=x2, qshape=qshape, block_size=block,
                         maxval=q.maxval.detach().clone(), scale=q.get_scale().detach().clone(),
                         dynamic=dyn.as_subclass(torch.Tensor).detach().clone(),
                         y=y.as_subclass(torch.Tensor).detach().clone(), y2=y2.as_subclass(torch.Tensor).detach().clone())
    _save("float_cases.pt", out)


# name, class, ctor args, ctor kwargs, weight shape
WIRE_CASES = [
    ("per_tensor_asym_uint8", "qdq", ((), 8, False), {}, (16, 24)),
    ("per_tensor_sym_int8", "qdq", ((), 8, True), {}, (16, 24)),
    ("per_channel_sym_int4", "qdq", ((16, 1), 4, True), {}, (16, 24)),
    ("per_channel_asym_uint8_axis1", "qdq", ((1, 24), 8, False), {}, (16, 24)),
    ("blockwise_sym_int4", "qdq", ((16, 3), 4, True), dict(block_size=(1, 8)), (16, 24)),
    ("blockwise_conv_sym_int8", "qdq", ((8, 2, 1, 1), 8, True), dict(block_size=(1, 4, 3, 3)), (8, 8, 3, 3)),
    ("sym_int4_half_step_shift", "qdq", ((), 4, True), dict(zero_point_shift=0.5), (16, 24)),
    ("lpbq_int4_in_int8", "lpbq", ((16, 3), 4, True, 8), dict(block_size=(1, 8), block_grouping=(1, -1)), (16, 24)),
    ("lpbq_ungrouped", "lpbq", ((16, 3), 4, True, 8), dict(block_size=(1, 8), block_grouping=(1, 1)), (16, 24)),
]


def gen_wire():
    """Exported encoding dictionaries (all four versions of the format) of calibrated quantizers."""
    from aimet_torch.quantization.affine import GroupedBlockQuantizeDequantize, QuantizeDequantize

    out = {}
    for idx, (name, kind, args, kw, wshape) in enumerate(WIRE_CASES):
        g = _gen(1600 + idx)
        w = torch.randn(wshape, generator=g) * 0.3 + 0.05
        q = (QuantizeDequantize if kind == "qdq" else GroupedBlockQuantizeDequantize)(*args, **kw)
        with q.compute_encodings():
            q(w)
        enc = q.get_encodings()._hint_input_shape(w.shape)
        dicts = {}
        for version in ("0.6.1", "1.0.0", "2.0.0", "2.1.0"):
            try:
                dicts[version] = enc.to_qnn_encoding_dict(version)
            except Exception as e:  # noqa: BLE001  the reference refuses some combinations
                dicts[version] = ("error", type(e).__name__)
        extra = {}
        if kind == "lpbq":
            extra["per_block_int_scale"] = enc.per_block_int_scale.as_subclass(torch.Tensor).detach().clone()
        out[name] = dict(kind=kind, args=args, kwargs=kw, w=w, min=q.min.detach().clone(), max=q.max.detach().clone(),
                         granularity=enc.granularity, dicts=dicts, **extra)
    _save("wire_cases.pt", out)


GENERATORS = {
    "backend_vectors": gen_backend_vectors,
    "affine": gen_affine,
    "pgs": gen_pgs,
    "analyzers": gen_analyzers,
    "lpnorm": gen_lpnorm,
    "quantizers": gen_quantizers,
    "seqmse": gen_seqmse,
    "seqmse_extra": gen_seqmse_extra,
    "float": gen_float,
    "wire": gen_wire,
}


if __name__ == "__main__":
    which = sys.argv[1:] or list(GENERATORS)
    for w in which:
        GENERATORS[w]()
