"""The drop-in boundary on the host: registration with the reference's own backend registry and the
behaviour under ``torch.compile``.  CPU only."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

from conftest import ROOT


def _reference_checkout():
    """The reference's source tree: $AIMET_REFERENCE_ROOT, else a directory ``reference`` beside this
    repository."""
    for cand in (os.environ.get("AIMET_REFERENCE_ROOT"), os.path.join(ROOT, os.pardir, "reference")):
        if cand and os.path.isdir(os.path.join(cand, "TrainingExtensions", "torch", "src", "python", "aimet_torch")):
            return os.path.abspath(cand)
    return None


def test_reference_dispatches_to_the_registered_backend():
    """``aimet_b200.register_backend`` + the reference's ``set_backend``: the reference's own
    QuantizeDequantize module and functionals then call this backend
    (quantization/affine/backends/utils.py:58-114, backends/__init__.py:173, 365, 403).  Run on CPU
    tensors, so what must surface is this backend's refusal of CPU tensors; the reference's stock
    backend would have computed a result instead."""
    ref = _reference_checkout()
    if ref is None:
        pytest.skip("no checkout of the reference available")
    script = textwrap.dedent(
        """
        import sys, torch
        sys.path.insert(0, {root!r}); sys.path.insert(0, {golden!r})
        import _reference_shim
        _reference_shim.install()
        import aimet_torch.quantization as Q
        from aimet_torch.quantization.affine.backends import utils as ref_backends
        import aimet_b200
        assert aimet_b200.register_backend("b200") is None
        assert "b200" in ref_backends._SUPPORTED_BACKENDS
        x = torch.linspace(-1, 1, 64).reshape(4, 16)
        q = Q.affine.QuantizeDequantize((), 8, False)
        with q.compute_encodings():
            q(x)
        stock = q(x)                                   # the reference's own backend computes on CPU
        assert stock.shape == x.shape
        with Q.set_backend("b200"):
            assert Q.get_backend().__name__ == "aimet_b200.backend"
            for call in (lambda: q(x),
                         lambda: Q.affine.quantize_dequantize(x, torch.tensor(0.01), torch.tensor(0.0), bitwidth=8, signed=True),
                         lambda: Q.affine.quantize(x, torch.tensor(0.01), torch.tensor(0.0), 0, 255),
                         lambda: Q.affine.dequantize(x, torch.tensor(0.01), torch.tensor(0.0))):
                try:
                    call()
                except RuntimeError as e:
                    assert "no CPU fallback" in str(e), e
                else:
                    raise AssertionError("the call did not reach the b200 backend")
        assert Q.get_backend().__name__ != "aimet_b200.backend"   # the context restored the previous one
        assert torch.equal(q(x), stock)
        ctx = aimet_b200.register_backend("b200", select=True)      # permanent selection
        assert Q.get_backend().__name__ == "aimet_b200.backend"
        print("DISPATCH-OK")
        """
    ).format(root=ROOT, golden=os.path.join(ROOT, "tests", "golden"))
    env = dict(os.environ, AIMET_REFERENCE_ROOT=ref)
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0 and "DISPATCH-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_behaviour_under_torch_compile(monkeypatch):
    """Inside a ``torch.compile`` region the reference never takes the ATen fake-quantize path
    (torch_builtins.py:456-491: ``_torch_compiler_is_compiling`` -> None -> QuantDequantFunc), and
    neither does this backend; the kernel call itself is opaque to the compiler and runs eagerly."""
    from aimet_b200 import backend as B

    seen = []

    def fake_forward(tensor, scale, offset, op, qmin, qmax, zps, block_size, internal_dtype):
        seen.append(op)
        return tensor * 1.0, tensor, scale, offset, None

    monkeypatch.setattr(B, "_run_forward", fake_forward)
    monkeypatch.setattr(B, "_validate", lambda *a, **k: None)
    x, s, o = torch.randn(4, 8), torch.tensor(0.1), torch.tensor(0.0)

    def fn(t):
        return B.quantize_dequantize(t, s, o, -128, 127) + 1.0

    with torch.no_grad():
        eager = fn(x)
        assert seen == ["fq"]
        compiled = torch.compile(fn, backend="eager")(x)
    assert seen == ["fq", "qdq"]
    assert torch.equal(eager, compiled)


# (args after (tensor, scale, offset), kwargs) -> (qmin, qmax, block_size, zero_point_shift)
_CALL_FORMS = [
    ((0, 255), {}, (0, 255, None, 0.0)),
    ((-8, 7, (1, 64)), {}, (-8, 7, (1, 64), 0.0)),
    ((-128, 127, None, 0.5), {}, (-128, 127, None, 0.5)),
    ((), {"qmin": -4, "qmax": 3}, (-4, 3, None, 0.0)),
    ((8,), {}, (0, 255, None, 0.0)),
    ((8, True), {}, (-128, 127, None, 0.0)),
    ((4, False, (1, 32)), {}, (0, 15, (1, 32), 0.0)),
    ((), {"bitwidth": 4, "signed": True}, (-8, 7, None, 0.0)),
    ((), {"bitwidth": 2}, (0, 3, None, 0.0)),
    ((), {"num_steps": 15, "signed": False}, (0, 15, None, 0.0)),
    ((), {"num_steps": 15, "signed": True}, (-8, 7, None, 0.0)),
    ((), {"num_steps": 254, "signed": True, "block_size": (2, 2)}, (-127, 127, (2, 2), 0.0)),
    ((), {"num_steps": 3, "signed": True, "zero_point_shift": 0.5}, (-2, 1, None, 0.5)),
    ((16, True), {"block_size": [1, -1]}, (-32768, 32767, [1, -1], 0.0)),
]


def test_call_forms_of_the_functionals():
    """(qmin, qmax) / (bitwidth, signed) / num_steps= resolve like the reference's ``_parse_args``
    (backends/__init__.py:408-445)."""
    from aimet_b200 import functional as F

    for args, kwargs, want in _CALL_FORMS:
        assert F.parse_grid_arguments(args, kwargs) == want, (args, kwargs)
    with pytest.raises(KeyError):
        F.parse_grid_arguments((), {"num_steps": 15})  # signed is required in this form, as in the reference
    with pytest.raises(RuntimeError, match="zero_point_shift"):
        F.quantize(torch.zeros(4), torch.tensor(1.0), torch.tensor(0.0), 0, 15, None, 0.5)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        F.quantize_dequantize(torch.zeros(4), torch.tensor(1.0), torch.tensor(0.0), bitwidth=8, signed=True)


def test_call_forms_agree_with_the_reference_parser():
    ref = _reference_checkout()
    if ref is None:
        pytest.skip("no checkout of the reference available")
    script = textwrap.dedent(
        """
        import sys
        sys.path.insert(0, {root!r}); sys.path.insert(0, {golden!r}); sys.path.insert(0, {tests!r})
        import _reference_shim
        _reference_shim.install()
        from aimet_torch.quantization.affine.backends import _parse_args
        from aimet_b200 import functional as F
        from test_boundary_cpu import _CALL_FORMS
        for args, kwargs, want in _CALL_FORMS:
            assert tuple(_parse_args(args, kwargs)) == F.parse_grid_arguments(args, kwargs) == want, (args, kwargs)
        print("PARSE-OK")
        """
    ).format(root=ROOT, golden=os.path.join(ROOT, "tests", "golden"), tests=os.path.join(ROOT, "tests"))
    env = dict(os.environ, AIMET_REFERENCE_ROOT=ref)
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0 and "PARSE-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_batched_derivation_of_encodings_host_arithmetic():
    """``derive_encodings`` (scale / offset of many quantizers from a handful of tensor operations)
    gives each quantizer what its own ``get_encodings()`` gives; the CUDA run of the same check is
    in test_quantizer_gpu.py."""
    from test_quantizer_gpu import check_batched_derivation

    check_batched_derivation("cpu")
