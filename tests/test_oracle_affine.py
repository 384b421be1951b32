"""The CPU oracle of the affine functionals against fixtures produced by the reference itself."""

import pytest
import torch

from conftest import assert_same, load_golden
from oracle import affine as O

CASES = load_golden("affine_cases.pt")
VECTORS = load_golden("backend_vectors.pt")


@pytest.mark.parametrize("name", sorted(CASES))
def test_quantize_dequantize_matches_reference(name):
    c = CASES[name]
    args = (c["scale"], c["offset"], c["qmin"], c["qmax"], c["block_size"], c["zero_point_shift"])
    assert_same(O.quantize_dequantize(c["x"], *args), c["qdq"], "qdq")
    gx, gs, go = O.quantize_dequantize_backward(c["x"], c["grad"], *args)
    assert_same(gx, c["qdq_gx"], "grad_x")
    assert_same(gs, c["qdq_gs"], "grad_scale")
    assert_same(go, c["qdq_go"], "grad_offset")


@pytest.mark.parametrize("name", sorted(n for n, c in CASES.items() if "q" in c))
def test_quantize_and_dequantize_match_reference(name):
    c = CASES[name]
    q = O.quantize(c["x"], c["scale"], c["offset"], c["qmin"], c["qmax"], c["block_size"])
    assert_same(q, c["q"], "q")
    gx, gs, go = O.quantize_backward(c["x"], c["grad"], c["scale"], c["offset"], c["qmin"], c["qmax"], c["block_size"])
    assert_same(gx, c["q_gx"], "q grad_x")
    assert_same(gs, c["q_gs"], "q grad_scale")
    assert_same(go, c["q_go"], "q grad_offset")
    dq = O.dequantize(c["q"], c["scale"], c["offset"], c["block_size"])
    assert_same(dq, c["dq"], "dq")
    gx, gs, go = O.dequantize_backward(c["q"], c["grad"], c["scale"], c["offset"], c["block_size"])
    assert_same(gx, c["dq_gx"], "dq grad_x")
    assert_same(gs, c["dq_gs"], "dq grad_scale")
    assert_same(go, c["dq_go"], "dq grad_offset")


@pytest.mark.parametrize("name", sorted(VECTORS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_known_answer_vectors(name, dtype):
    """The hand-written vector sets of the reference's backend test: exact codes, exact
    dequantized values, exact quantize-dequantize output."""
    v = VECTORS[name]
    if dtype == torch.bfloat16 and not name.startswith("bfloat16_compat"):
        pytest.skip("inputs of this set are not exact in bfloat16")
    if dtype == torch.float16 and not name.startswith("bfloat16_compat"):
        pytest.skip("inputs of this set are not exact in float16")
    x = v["tensor"].to(dtype)
    scale, offset = v["delta"].to(dtype), v["offset"].to(dtype)
    q = O.quantize(x, scale, offset, v["qmin"], v["qmax"])
    assert torch.equal(q, v["tensor_q"].to(dtype))
    assert torch.equal(O.dequantize(q, scale, offset), v["tensor_qdq"].to(dtype))
    assert torch.equal(O.quantize_dequantize(x, scale, offset, v["qmin"], v["qmax"]), v["tensor_qdq"].to(dtype))
    gx, _, _ = O.quantize_dequantize_backward(x, torch.ones_like(x), scale, offset, v["qmin"], v["qmax"])
    assert torch.equal(gx, (~v["mask"]).to(dtype))


@pytest.mark.parametrize("name", sorted(CASES))
def test_fake_quantize_formula_is_what_aten_computes(name):
    """The float32 formula the CUDA kernel implements equals the ATen fake-quantize ops the
    reference calls when no parameter gradient is needed."""
    c = CASES[name]
    if c["dtype"] == torch.float64 or not O.takes_fake_quantize_path(c["x"], c["scale"], c["offset"], c["block_size"], c["zero_point_shift"]):
        pytest.skip("reference does not take the fake-quantize path here")
    a = O.fake_quantize(c["x"], c["scale"], c["offset"], c["qmin"], c["qmax"])
    assert_same(O.fake_quantize_formula(c["x"], c["scale"], c["offset"], c["qmin"], c["qmax"]), a, "formula")


PGS = load_golden("pgs_cases.pt")


@pytest.mark.parametrize("name", sorted(PGS))
def test_gradient_multiplier_near_rounding_boundaries_matches_reference(name):
    """quantize_dequantize backward with the reference's experimental "pivot gradient spiking" on."""
    c = PGS[name]
    args = (c["scale"], c["offset"], c["qmin"], c["qmax"], c["block_size"], c["zero_point_shift"])
    assert_same(O.quantize_dequantize(c["x"], *args), c["y"], "y")
    gx, gs, go = O.quantize_dequantize_backward(c["x"], c["grad"], *args, pgs_eps=c["eps"], pgs_multiplier=c["multiplier"])
    assert_same(gx, c["gx"], "grad_x")
    plain, _, _ = O.quantize_dequantize_backward(c["x"], c["grad"], *args)
    assert not torch.equal(plain, gx)  # the case does exercise the multiplier
    if c["param_grads"]:
        assert_same(gs, c["gs"], "grad_scale")
        assert_same(go, c["go"], "grad_offset")
