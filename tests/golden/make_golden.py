"""Generates the golden fixtures under tests/golden/ by running the aimet_torch reference itself.

Run where the reference checkout is available (CPU is enough):

    python tests/golden/make_golden.py [affine|backend_vectors|analyzers|quantizers|seqmse ...]

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


GENERATORS = {
    "backend_vectors": gen_backend_vectors,
    "affine": gen_affine,
}


if __name__ == "__main__":
    which = sys.argv[1:] or list(GENERATORS)
    for w in which:
        GENERATORS[w]()
