"""CUDA affine functionals (through the C ABI) against the golden fixtures and the CPU oracle."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import affine as O

pytestmark = pytest.mark.gpu

CASES = load_golden("affine_cases.pt")
VECTORS = load_golden("backend_vectors.pt")


def _backend():
    from aimet_b200 import backend

    return backend


def _ulp_close(a, b, dtype, ulps=1):
    """|a - b| <= ulps * ulp(dtype) relative to the larger magnitude."""
    a, b = a.double().cpu(), b.double().cpu()
    eps = torch.finfo(dtype).eps
    tol = ulps * eps * torch.maximum(a.abs(), b.abs()) + 1e-30
    return bool(((a - b).abs() <= tol).all())


def _check_param_grad(got, want, internal_dtype, what):
    """Scale / offset gradients are sums: the reduction order differs from torch's, so they are
    compared within 1e-5 relative (float32 / float64 internal dtype) or one unit in the last
    place of the 16-bit internal dtype the reference sums in."""
    assert got.shape == want.shape and got.dtype == want.dtype, what
    if internal_dtype in (torch.float16, torch.bfloat16):
        assert _ulp_close(got, want, internal_dtype, ulps=1), what
    else:
        scale = want.double().abs().max().clamp_min(1e-30)
        err = (got.double().cpu() - want.double()).abs().max()
        assert err <= 1e-5 * scale, f"{what}: max abs err {err} vs scale {scale}"


def _run(fn, x, grad, scale, offset, *args):
    xi = x.clone().cuda().requires_grad_(True)
    s = scale.clone().cuda().requires_grad_(True)
    o = offset.clone().cuda().requires_grad_(True)
    y = fn(xi, s, o, *args)
    y.backward(grad.cuda())
    torch.cuda.synchronize()
    return y.detach(), xi.grad, s.grad, o.grad


@pytest.mark.parametrize("name", sorted(CASES))
def test_quantize_dequantize_golden(name):
    c = CASES[name]
    B = _backend()
    idt = O.internal_dtype(c["dtype"], c["qmin"], c["qmax"])
    y, gx, gs, go = _run(B.quantize_dequantize, c["x"], c["grad"], c["scale"], c["offset"], c["qmin"], c["qmax"],
                         c["block_size"], c["zero_point_shift"])
    assert_same(y, c["qdq"], "qdq")          # bit-exact (north-star allows 1 ulp)
    assert_same(gx, c["qdq_gx"], "grad_x")   # bit-exact
    _check_param_grad(gs, c["qdq_gs"], idt, "grad_scale")
    _check_param_grad(go, c["qdq_go"], idt, "grad_offset")


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if "q" in c))
def test_quantize_and_dequantize_golden(name):
    c = CASES[name]
    B = _backend()
    idt = O.internal_dtype(c["dtype"], c["qmin"], c["qmax"])
    q, gx, gs, go = _run(B.quantize, c["x"], c["grad"], c["scale"], c["offset"], c["qmin"], c["qmax"], c["block_size"])
    assert_same(q, c["q"], "codes")  # integer codes: bit-exact
    assert_same(gx, c["q_gx"], "q grad_x")
    _check_param_grad(gs, c["q_gs"], idt, "q grad_scale")
    _check_param_grad(go, c["q_go"], idt, "q grad_offset")
    dq, gx, gs, go = _run(B.dequantize, c["q"], c["grad"], c["scale"], c["offset"], c["block_size"])
    assert_same(dq, c["dq"], "dq")
    assert_same(gx, c["dq_gx"], "dq grad_x")
    _check_param_grad(gs, c["dq_gs"], c["dtype"], "dq grad_scale")
    _check_param_grad(go, c["dq_go"], c["dtype"], "dq grad_offset")


@pytest.mark.parametrize("name", sorted(VECTORS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_known_answer_vectors(name, dtype):
    v = VECTORS[name]
    if dtype != torch.float32 and not name.startswith("bfloat16_compat"):
        pytest.skip("inputs of this set are not exact in 16-bit floats")
    B = _backend()
    x = v["tensor"].to(dtype).cuda().requires_grad_(True)
    scale, offset = v["delta"].to(dtype).cuda(), v["offset"].to(dtype).cuda()
    q = B.quantize(x.detach(), scale, offset, v["qmin"], v["qmax"])
    assert torch.equal(q.cpu(), v["tensor_q"].to(dtype))
    assert torch.equal(B.dequantize(q, scale, offset).cpu(), v["tensor_qdq"].to(dtype))
    y = B.quantize_dequantize(x, scale, offset, v["qmin"], v["qmax"])
    assert torch.equal(y.detach().cpu(), v["tensor_qdq"].to(dtype))
    y.backward(torch.ones_like(y))
    assert torch.equal(x.grad.cpu(), (~v["mask"]).to(dtype))


# ---- larger shapes against the oracle: every kernel variant (vector / scalar, segment / column /
# ---- chunked / general) gets exercised -------------------------------------------------------
ORACLE_CASES = [
    # dtype, shape, pshape, block, qmin, qmax, zps
    (torch.float32, (512, 1024), (), None, 0, 255, 0.0),            # chunked per-tensor
    (torch.float32, (1, 100003), (), None, 0, 255, 0.0),            # scalar path, chunked
    (torch.bfloat16, (300, 4096), (300, 1), None, -128, 127, 0.0),  # one CTA per row
    (torch.bfloat16, (64, 20480), (64, 1), None, -128, 127, 0.0),   # chunked rows
    (torch.bfloat16, (128, 4096), (128, 64), (1, 64), -8, 7, 0.0),  # blockwise int4, bf16 internal
    (torch.float16, (128, 1024), (128, 16), (1, 64), -8, 7, 0.0),
    (torch.float32, (64, 96, 14, 14), (96, 1, 1), None, 0, 255, 0.0),  # NCHW per-channel: seg + partials
    (torch.float32, (8, 32, 3, 3), (32, 1, 1), None, 0, 255, 0.0),     # small inner: column mode
    (torch.bfloat16, (4096, 520), (520,), None, 0, 255, 0.0),          # channel-last: column mode
    (torch.float32, (1000, 77), (77,), None, -8, 7, 0.5),              # scalar column mode + zps
    (torch.float32, (48, 64), (6, 8), (8, 8), 0, 15, 0.0),             # 2-d blocks: general path
    (torch.bfloat16, (6, 40, 50), (3, 1, 5), (2, -1, 10), -8, 7, 0.0),
    (torch.float32, (5000, 4096), (), None, 0, 255, 0.0),              # per-tensor cut into whole waves of chunks
    (torch.bfloat16, (32, 4104), (32, 1), None, -128, 127, 0.0),       # 513 vectors per row: ragged loop ends
    (torch.bfloat16, (16, 65536), (16, 1), None, -128, 127, 0.0),      # 32 vectors per thread: the copy ring wraps
    (torch.float16, (16, 65536), (16, 1), None, -8, 7, 0.0),           # float16 internal, packed arithmetic
]


@pytest.mark.parametrize("case", ORACLE_CASES, ids=lambda c: f"{str(c[0])[6:]}-{'x'.join(map(str, c[1]))}-p{'x'.join(map(str, c[2]))}")
def test_quantize_dequantize_vs_oracle(case):
    dtype, shape, pshape, block, qmin, qmax, zps = case
    B = _backend()
    g = torch.Generator().manual_seed(hash(shape) % 10000)
    x = (torch.randn(shape, generator=g) * (1 + 5 * (torch.rand(shape, generator=g) < 0.01))).to(dtype)
    grad = torch.randn(shape, generator=g).to(dtype)
    scale = (4.0 / (qmax - qmin)) * (0.5 + torch.rand(pshape, generator=g))
    offset = torch.round(-(qmax - qmin) * (0.3 + 0.4 * torch.rand(pshape, generator=g))) - qmin
    idt = O.internal_dtype(dtype, qmin, qmax)
    y, gx, gs, go = _run(B.quantize_dequantize, x, grad, scale, offset, qmin, qmax, block, zps)
    assert_same(y, O.quantize_dequantize(x, scale, offset, qmin, qmax, block, zps), "qdq")
    ogx, ogs, ogo = O.quantize_dequantize_backward(x, grad, scale, offset, qmin, qmax, block, zps)
    assert_same(gx, ogx, "grad_x")
    _check_param_grad(gs, ogs, idt, "grad_scale")
    _check_param_grad(go, ogo, idt, "grad_offset")
    # deterministic: a second run is bit-identical
    y2, gx2, gs2, go2 = _run(B.quantize_dequantize, x, grad, scale, offset, qmin, qmax, block, zps)
    assert torch.equal(gs, gs2) and torch.equal(go, go2) and torch.equal(gx, gx2)


def test_memory_format_and_strides():
    B = _backend()
    x = torch.randn(4, 8, 6, 6).cuda().to(memory_format=torch.channels_last)
    scale = (torch.rand(8, 1, 1) * 0.05 + 0.01).cuda()
    offset = torch.zeros(8, 1, 1).cuda()
    y = B.quantize_dequantize(x, scale, offset, -128, 127)
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert_same(y, O.quantize_dequantize(x.cpu(), scale.cpu(), offset.cpu(), -128, 127), "channels_last")
    xt = torch.randn(33, 20).cuda().t()  # transposed view
    y = B.quantize_dequantize(xt, torch.tensor(0.02).cuda(), torch.tensor(0.0).cuda(), -128, 127)
    assert_same(y, O.quantize_dequantize(xt.cpu(), torch.tensor(0.02), torch.tensor(0.0), -128, 127), "transposed")
    xs = torch.randn(16, 40).cuda()[:, ::2]  # not dense
    y = B.quantize_dequantize(xs, torch.tensor(0.02).cuda(), torch.tensor(0.0).cuda(), -128, 127)
    assert_same(y, O.quantize_dequantize(xs.cpu(), torch.tensor(0.02), torch.tensor(0.0), -128, 127), "strided")


def test_special_values_and_empty():
    B = _backend()
    x = torch.tensor([float("nan"), float("inf"), -float("inf"), 0.0, -0.0, 1e30, -1e-30, 0.25]).cuda()
    s, o = torch.tensor(0.5).cuda(), torch.tensor(-3.0).cuda()
    # QuantDequantFunc arithmetic (a parameter wants a gradient): NaN propagates like torch.clamp
    sg = s.clone().requires_grad_(True)
    assert_same(B.quantize_dequantize(x, sg, o, 0, 15).detach(), O.quantize_dequantize(x.cpu(), s.cpu(), o.cpu(), 0, 15), "special")
    assert_same(B.quantize(x, s, o, 0, 15), O.quantize(x.cpu(), s.cpu(), o.cpu(), 0, 15), "special codes")
    # fake-quantize arithmetic: what the float -> int64 cast does with NaN / inf is device-defined in
    # ATen; the kernel follows the CUDA behaviour (saturate, NaN -> 0)
    dev = torch.fake_quantize_per_tensor_affine(x, s, (-o).to(torch.int32), 0, 15)
    assert_same(B.quantize_dequantize(x, s, o, 0, 15), dev.cpu(), "special, fake-quantize path")
    e = torch.empty(0, 4).cuda()
    assert B.quantize_dequantize(e, s, o, 0, 15).shape == (0, 4)


@pytest.mark.parametrize("dtype,qmin,qmax", [(torch.bfloat16, -128, 127), (torch.bfloat16, -8, 7), (torch.float16, -128, 127),
                                             (torch.float32, 0, 255)])
def test_non_finite_and_huge_inputs_in_the_vector_kernels(dtype, qmin, qmax):
    """Infinities, NaN and magnitudes far outside the grid scattered through large rows: the fast
    bodies (bounded input instead of a per-element overflow guard) must agree with the oracle bit
    for bit, forward and backward."""
    B = _backend()
    g = torch.Generator().manual_seed(7)
    x = torch.randn(24, 8192, generator=g)
    idx = torch.randperm(x.numel(), generator=g)
    flat = x.view(-1)
    big = 6.0e4 if dtype == torch.float16 else 3.0e38
    for k, v in enumerate([float("inf"), -float("inf"), float("nan"), big, -big, 1e-30, -0.0]):
        flat[idx[k * 50:(k + 1) * 50]] = v
    x = x.to(dtype)
    grad = torch.randn(24, 8192, generator=g).to(dtype)
    scale = (3.0 / (qmax - qmin)) * (0.5 + torch.rand(24, 1, generator=g))
    offset = torch.zeros(24, 1) if qmin < 0 else torch.full((24, 1), -128.0)
    idt = O.internal_dtype(dtype, qmin, qmax)
    y, gx, gs, go = _run(B.quantize_dequantize, x, grad, scale, offset, qmin, qmax, None, 0.0)
    assert_same(y, O.quantize_dequantize(x, scale, offset, qmin, qmax, None, 0.0), "qdq")
    ogx, ogs, ogo = O.quantize_dequantize_backward(x, grad, scale, offset, qmin, qmax, None, 0.0)
    assert_same(gx, ogx, "grad_x")
    # rows that hold a NaN have NaN sums in both; the others follow the usual tolerance
    ok = ~(ogs.isnan() | ogo.isnan()).flatten()
    assert torch.equal(gs.cpu().isnan().flatten(), ~ok | ogs.isnan().flatten())
    _check_param_grad(gs.cpu().flatten()[ok], ogs.flatten()[ok], idt, "grad_scale")
    _check_param_grad(go.cpu().flatten()[ok], ogo.flatten()[ok], idt, "grad_offset")


def test_float16_scale_too_large_for_the_input_bound():
    """float16 tensors with a scale so large that (qmax + 4) * scale overflows float16: the packed
    bound on |x| does not exist and the kernels fall back to the guarded arithmetic."""
    B = _backend()
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(8, 4096, generator=g) * 2.0e4).to(torch.float16)
    x[0, :4] = torch.tensor([float("inf"), -float("inf"), 65504.0, -65504.0], dtype=torch.float16)
    grad = torch.randn(8, 4096, generator=g).to(torch.float16)
    scale = torch.full((8, 1), 600.0)
    offset = torch.zeros(8, 1)
    y, gx, gs, go = _run(B.quantize_dequantize, x, grad, scale, offset, -128, 127, None, 0.0)
    assert_same(y, O.quantize_dequantize(x, scale, offset, -128, 127, None, 0.0), "qdq")
    ogx, ogs, ogo = O.quantize_dequantize_backward(x, grad, scale, offset, -128, 127, None, 0.0)
    assert_same(gx, ogx, "grad_x")
    _check_param_grad(gs, ogs, torch.float16, "grad_scale")


def test_error_contracts():
    B = _backend()
    x = torch.randn(4, 6).cuda()
    s, o = torch.ones(()).cuda(), torch.zeros(()).cuda()
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x.cpu(), s.cpu(), o.cpu(), 0, 15)      # no CPU path
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x, torch.ones(5).cuda(), torch.zeros(5).cuda(), 0, 15)  # not broadcastable
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x, torch.ones(2, 4, 6).cuda(), torch.zeros(2, 4, 6).cuda(), 0, 15)  # inverse broadcast
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x, s, o, 16, 15)                        # qmin > qmax
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x, s.cpu(), o, 0, 15)                   # devices differ
    with pytest.raises(RuntimeError):
        B.quantize_dequantize(x, torch.ones(2, 2).cuda(), torch.zeros(2, 2).cuda(), 0, 15, block_size=(2, 2))
    with pytest.raises(RuntimeError):
        B.quantize(x.to(torch.bfloat16), s, o, 0, 2**16 - 1)           # grid not representable in bf16


# ---- no parameter gradients: the reference switches to torch.fake_quantize_* arithmetic --------
FQ_CASES = sorted(
    n for n, c in CASES.items()
    if c["dtype"] != torch.float64 and O.takes_fake_quantize_path(c["x"], c["scale"], c["offset"], c["block_size"], c["zero_point_shift"])
)


@pytest.mark.parametrize("name", FQ_CASES)
def test_fake_quantize_path(name):
    c = CASES[name]
    B = _backend()
    x = c["x"].cuda().requires_grad_(True)
    y = B.quantize_dequantize(x, c["scale"].cuda(), c["offset"].cuda(), c["qmin"], c["qmax"])
    want = O.fake_quantize(c["x"], c["scale"], c["offset"], c["qmin"], c["qmax"])
    assert_same(y.detach(), want, "fake-quantize output")
    y.backward(c["grad"].cuda())
    assert_same(x.grad, O.fake_quantize_backward(c["x"], c["grad"], c["scale"], c["offset"], c["qmin"], c["qmax"]), "grad_x")
    with torch.no_grad():  # parameters that require grad still take this path when grad mode is off
        y2 = B.quantize_dequantize(c["x"].cuda(), c["scale"].cuda().requires_grad_(True), c["offset"].cuda(), c["qmin"], c["qmax"])
    assert_same(y2, want, "no_grad output")
    # the device's own ATen kernel agrees too
    s32 = c["scale"].cuda().float()
    zp = -c["offset"].cuda().to(torch.int32)
    if s32.numel() == 1:
        dev = torch.fake_quantize_per_tensor_affine(c["x"].cuda(), s32.reshape(()), zp.reshape(()), c["qmin"], c["qmax"])
        assert_same(y.detach(), dev.cpu(), "device ATen kernel")


def test_fake_quantize_large_per_channel():
    B = _backend()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 96, 28, 28, generator=g).to(torch.bfloat16)
    scale = torch.rand(96, 1, 1, generator=g) * 0.02 + 0.005
    offset = torch.zeros(96, 1, 1)
    y = B.quantize_dequantize(x.cuda(), scale.cuda(), offset.cuda(), -128, 127)
    assert_same(y, O.fake_quantize(x, scale, offset, -128, 127), "per-channel fake-quantize")


def test_per_channel_zero_point_outside_the_grid_takes_the_division_arithmetic():
    """torch.fake_quantize_per_channel_affine refuses zero points outside [qmin, qmax] and the reference
    then runs QuantDequantFunc (true division) for the whole tensor (torch_builtins.py:418-425); so does
    this backend, whether it learns the zero points from the device or from a host-known constant."""
    B = _backend()
    g = torch.Generator().manual_seed(6)
    x = torch.randn(7, 12, 33, generator=g) * 3
    scale = torch.rand(12, 1, generator=g) * 0.05 + 0.01
    inside = torch.full((12, 1), -100.0)
    outside = inside.clone()
    outside[5] = 40.0  # zero point -40 < qmin = 0
    with torch.no_grad():
        y_in = B.quantize_dequantize(x.cuda(), scale.cuda(), inside.cuda(), 0, 255)
        y_out = B.quantize_dequantize(x.cuda(), scale.cuda(), outside.cuda(), 0, 255)
        tagged = outside.cuda()
        tagged[:] = 40.0
        tagged._b200_constant = 40.0
        y_tag = B.quantize_dequantize(x.cuda(), scale.cuda(), tagged, 0, 255)
    assert_same(y_in, O.fake_quantize(x, scale, inside, 0, 255), "zero points inside: fake-quantize arithmetic")
    assert_same(y_out, O.quantize_dequantize(x, scale, outside, 0, 255), "a zero point outside: division arithmetic")
    assert_same(y_tag, O.quantize_dequantize(x, scale, torch.full((12, 1), 40.0), 0, 255), "host-known constant")


def test_functional_call_forms():
    """``aimet_b200.quantize`` / ``quantize_dequantize`` / ``dequantize`` with the reference's three
    ways of naming the grid (backends/__init__.py:50-175, 215-369) give what the explicit
    ``qmin, qmax`` form gives, and that is the oracle's result."""
    import aimet_b200

    x = torch.arange(-0.3, 1.3, 0.05).cuda()
    scale, offset = torch.tensor(1 / 15).cuda(), torch.tensor(0.0).cuda()
    want_q = O.quantize(x.cpu(), scale.cpu(), offset.cpu(), 0, 15)
    for got in (aimet_b200.quantize(x, scale, offset, 0, 15), aimet_b200.quantize(x, scale, offset, bitwidth=4),
                aimet_b200.quantize(x, scale, offset, 4), aimet_b200.quantize(x, scale, offset, num_steps=15, signed=False),
                aimet_b200.quantize(x, scale, offset, qmin=0, qmax=15)):
        assert_same(got, want_q)
    want = O.fake_quantize(x.cpu(), scale.cpu(), offset.cpu(), -8, 7)  # no parameter gradient: the fast path
    for got in (aimet_b200.quantize_dequantize(x, scale, offset, -8, 7),
                aimet_b200.quantize_dequantize(x, scale, offset, 4, True),
                aimet_b200.quantize_dequantize(x, scale, offset, bitwidth=4, signed=True),
                aimet_b200.quantize_dequantize(x, scale, offset, num_steps=15, signed=True)):
        assert_same(got, want)
    assert_same(aimet_b200.dequantize(want_q.cuda(), scale, offset), O.dequantize(want_q, scale.cpu(), offset.cpu()))


PGS = load_golden("pgs_cases.pt")


@pytest.mark.parametrize("name", sorted(PGS))
def test_gradient_multiplier_near_rounding_boundaries(name):
    """The reference's experimental "pivot gradient spiking" (experimental/pgs.py): the input
    gradient of elements whose rounding error exceeds (1 - eps) / 2 is multiplied.  Bit-exact
    against the reference's own backward; the switch is read when the forward runs."""
    from aimet_b200 import pgs

    c = PGS[name]
    B = _backend()
    idt = O.internal_dtype(c["dtype"], c["qmin"], c["qmax"])
    xi = c["x"].clone().cuda().requires_grad_(True)
    s = c["scale"].clone().cuda().requires_grad_(c["param_grads"])
    o = c["offset"].clone().cuda().requires_grad_(c["param_grads"])
    pgs.enable_pgs(c["eps"], c["multiplier"])
    try:
        assert pgs.is_pgs_enabled() and pgs.get_pgs_eps() == c["eps"] and pgs.get_pgs_multiplier() == c["multiplier"]
        y = B.quantize_dequantize(xi, s, o, c["qmin"], c["qmax"], c["block_size"], c["zero_point_shift"])
    finally:
        pgs.disable_pgs()
    assert not pgs.is_pgs_enabled()
    y.backward(c["grad"].cuda())
    assert_same(y.detach(), c["y"], "y")
    assert_same(xi.grad, c["gx"], "grad_x")
    if c["param_grads"]:
        _check_param_grad(s.grad, c["gs"], idt, "grad_scale")
        _check_param_grad(o.grad, c["go"], idt, "grad_offset")
    with pytest.raises(ValueError):
        pgs.enable_pgs(0.0, 3.0)
    with pytest.raises(ValueError):
        pgs.enable_pgs(0.1, 1.0)


def test_gradient_multiplier_at_a_large_size():
    """The same against the oracle on a tensor that takes the vector kernels (bf16, blockwise)."""
    from aimet_b200 import pgs

    B = _backend()
    g = torch.Generator().manual_seed(77)
    shape, pshape, block, qmin, qmax = (512, 4096), (512, 64), (1, 64), -8, 7
    x = (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16)
    grad = torch.randn(shape, generator=g).to(torch.bfloat16)
    scale = (x.float().reshape(512, 64, 64).abs().amax(2) / 7).clamp_min(1e-6)
    offset = torch.zeros(pshape)
    xi = x.clone().cuda().requires_grad_(True)
    s = scale.clone().cuda().requires_grad_(True)
    pgs.enable_pgs(0.1, 3.0)
    try:
        y = B.quantize_dequantize(xi, s, offset.cuda(), qmin, qmax, block)
    finally:
        pgs.disable_pgs()
    y.backward(grad.cuda())
    ogx, ogs, _ = O.quantize_dequantize_backward(x, grad, scale, offset, qmin, qmax, block, 0.0, pgs_eps=0.1,
                                                 pgs_multiplier=3.0)
    assert_same(xi.grad, ogx, "grad_x")
    _check_param_grad(s.grad, ogs, O.internal_dtype(torch.bfloat16, qmin, qmax), "grad_scale")


def test_stack_of_parameter_sets_equals_separate_calls():
    """``quantize_dequantize_stack``: one output slice per leading index of the parameters, each what
    a separate call with that slice's parameters returns, in both arithmetics."""
    B = _backend()
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(96, 256, generator=g) * 0.05).to(torch.bfloat16).cuda()
    base = w.float().abs().amax(1, keepdim=True) / 7
    scale = torch.stack([base * f for f in (0.4, 0.7, 1.0)])            # [3, 96, 1]
    offset = torch.zeros_like(scale)
    for grads in (False, True):
        got = B.quantize_dequantize_stack(w, scale, offset, -8, 7, parameter_gradients=grads)
        assert got.shape == (3, 96, 256) and got.dtype == w.dtype
        for c in range(3):
            s = scale[c].clone().requires_grad_(grads)
            with torch.enable_grad() if grads else torch.no_grad():
                want = B.quantize_dequantize(w, s, offset[c], -8, 7)
            assert torch.equal(got[c], want.detach())
    # blockwise parameters: [candidates, rows, blocks]
    bscale = torch.stack([w.float().reshape(96, 4, 64).abs().amax(2) / 7 * f for f in (0.5, 1.0)])
    got = B.quantize_dequantize_stack(w, bscale, torch.zeros_like(bscale), -8, 7, block_size=(1, 64))
    for c in range(2):
        want = B.quantize_dequantize(w, bscale[c], torch.zeros_like(bscale[c]), -8, 7, block_size=(1, 64))
        assert torch.equal(got[c], want)
