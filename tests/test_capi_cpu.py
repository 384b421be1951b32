"""CPU-only checks: the C-ABI library loads, exports what the header declares, and the host-side
logic (argument validation, dtype rules, layout planning) behaves like the reference's."""

import os
import re

import pytest
import torch

from conftest import ROOT
from oracle import affine as O


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "aimet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aimet_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from aimet_b200 import _lib

    names = _header_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names
    assert _lib.lib.aimet_b200_version() >= 1


def test_layout_errors_and_scratch_queries_without_a_gpu():
    from aimet_b200 import _lib

    lib = _lib.lib
    bad = _lib.make_layout([6, 8], [4, 8])  # 4 does not divide 6
    assert lib.aimet_b200_backward_scratch_bytes(bad, _lib.AB_F32) == _lib.AB_ERR_INVALID
    assert "does not divide" in _lib.last_error()
    # rows of 4096 and blocks of 64 are reduced inside the kernel: no partial sums
    assert lib.aimet_b200_backward_scratch_bytes(_lib.make_layout([14336, 4096], [1, 4096]), _lib.AB_BF16) == 0
    assert lib.aimet_b200_backward_scratch_bytes(_lib.make_layout([14336, 4096], [1, 64]), _lib.AB_BF16) == 0
    # longer rows are cut into chunks of at most 8192 elements (scalar kernel): one partial pair each
    assert lib.aimet_b200_backward_scratch_bytes(_lib.make_layout([16, 65536], [1, 65536]), _lib.AB_BF16) == 16 * 8 * 16
    # per-tensor: one partial pair (two doubles) per chunk; the chunk count is rounded to whole
    # waves of CTAs, so only its range is fixed
    n = lib.aimet_b200_backward_scratch_bytes(_lib.make_layout([4096, 4096], [4096, 4096]), _lib.AB_F32)
    assert n % 16 == 0 and 4096 * 4096 // 32768 * 16 <= n <= (4096 * 4096 // 2048) * 16
    assert lib.aimet_b200_backward_scratch_bytes(_lib.make_layout([0, 4], [1, 4]), _lib.AB_F32) == 0
    # two column halves per 256-token tile, up to two values per (candidate, channel, block)
    assert lib.aimet_b200_seqmse_scratch_bytes(8192, 4096, 4096, 20) == 2 * 32 * 20 * 4096 * 2 * 4
    assert lib.aimet_b200_seqmse_blocks_scratch_bytes(8192, 4096, 4096, 64, 20) == 64 * 2 * 32 * 20 * 4096 * 2 * 4
    assert lib.aimet_b200_fixed_scratch_capacity() == 1 << 20
    with pytest.raises(RuntimeError):
        _lib.make_layout([1] * 9, [1] * 9)


def test_argument_checks_that_need_no_gpu():
    """Entry points refuse what they do not cover before anything touches the device."""
    from aimet_b200 import _lib

    lib = _lib.lib
    one = 16  # any non-NULL value: the calls below return before a pointer is used
    per_channel = _lib.make_layout([8, 64], [1, 64])
    rc = lib.aimet_b200_histogram_update(one, per_channel, _lib.AB_BF16, 64, *([one] * 17), one, 0, None)
    assert rc == _lib.AB_ERR_UNSUPPORTED and "single" in _lib.last_error()
    per_tensor = _lib.make_layout([8, 64], [8, 64])
    rc = lib.aimet_b200_histogram_update(one, per_tensor, _lib.AB_F64, 64, *([one] * 17), one, 0, None)
    assert rc == _lib.AB_ERR_UNSUPPORTED
    rc = lib.aimet_b200_histogram_update(one, per_tensor, _lib.AB_BF16, 100000, *([one] * 17), one, 0, None)
    assert rc == _lib.AB_ERR_UNSUPPORTED and "num_bins" in _lib.last_error()
    rc = lib.aimet_b200_quantize_dequantize_backward_ex(one, one, one, one, per_tensor, _lib.AB_F32, _lib.AB_F32, 0, 0, 255,
                                                        0.0, 1.5, 3.0, one, None, None, None, 0, None)
    assert rc == _lib.AB_ERR_INVALID and "pgs_eps" in _lib.last_error()
    rc = lib.aimet_b200_sqnr_encodings(one, one, one, one, one, 19, 17, 0, _lib.AB_F32, 1, 64, 255.0, 3.0, 0.0, 1e-9,
                                       one, None, None, one, one, one, None)
    assert rc == _lib.AB_ERR_INVALID and "exponent" in _lib.last_error()
    rc = lib.aimet_b200_float_fake_cast(one * 16, one * 16, one * 16, per_tensor, _lib.AB_F32, _lib.AB_BF16, _lib.AB_BF16, 4, 3,
                                        7, 448.0, 0, None)
    assert rc == _lib.AB_ERR_UNSUPPORTED and "in_dtype" in _lib.last_error()


def test_cpu_tensors_are_refused():
    from aimet_b200 import backend as B
    from aimet_b200 import encoding_analyzer as EA

    x, s, o = torch.randn(4, 4), torch.tensor(0.1), torch.tensor(0.0)
    for fn, args in ((B.quantize, (0, 15)), (B.quantize_dequantize, (0, 15)), (B.dequantize, ())):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            fn(x, s, o, *args)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        EA.MinMaxEncodingAnalyzer(()).update_stats(x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("grid", [(0, 15), (-8, 7), (0, 255), (-128, 127), (0, 65535), (-(2**31), 2**31 - 1), (0, 31), (0, 63)])
def test_internal_dtype_rule_matches_oracle(dtype, grid):
    from aimet_b200 import backend as B

    assert B._internal_dtype(dtype, *grid) == O.internal_dtype(dtype, *grid)
    assert B._is_grid_representable(dtype, *grid) == O.grid_representable(dtype, *grid)


def test_param_blocks_and_fast_path_selection():
    from aimet_b200 import backend as B

    assert B._param_blocks((4, 6, 5, 7), (6, 1, 1), None) == (4, 1, 5, 7)
    assert B._param_blocks((8, 12), (4, 3), (2, 4)) == (2, 4)
    assert B._param_blocks((6, 2, 8, 10), (2, 2, 5), (1, -1, 2)) == (6, 1, 4, 2)
    assert B._param_blocks((3, 5), (), None) == (3, 5)
    x = torch.zeros(4, 6, 5)
    s1, s2 = torch.ones(6, 1), torch.ones(4, 1, 5)
    for scale, block, zps in ((torch.ones(()), None, 0.0), (s1, None, 0.0), (s2, None, 0.0), (s1, (1, 1), 0.0), (s1, None, 0.5)):
        assert B._takes_fake_quantize_path(x, scale, torch.zeros_like(scale), block, zps) == O.takes_fake_quantize_path(
            x, scale, torch.zeros_like(scale), block, zps)
    assert not B._takes_fake_quantize_path(x, s1.requires_grad_(True), torch.zeros(6, 1), None, 0.0)


def test_quantizer_constructor_contracts():
    from aimet_b200 import quantizer as Q

    q = Q.QuantizeDequantize((3, 1), 8, True)
    assert (q.qmin, q.qmax, q.bitwidth, q.signed, q.symmetric) == (-128, 127, 8, True, True)
    q = Q.QuantizeDequantize((), qmin=0, qmax=15, symmetric=False)
    assert q.bitwidth == 4 and not q.signed and not q.is_initialized()
    assert q.get_scale() is None and q.get_encodings() is None
    with pytest.raises(TypeError):
        Q.QuantizeDequantize((), 8, False, bogus=1)
    with pytest.raises(TypeError):
        Q.QuantizeDequantize(())
    with pytest.raises(RuntimeError):
        Q.QuantizeDequantize((3,), 8, False, encoding_analyzer=__import__("aimet_b200.encoding_analyzer", fromlist=["x"]).MinMaxEncodingAnalyzer((4,)))
    with pytest.raises(RuntimeError):
        q.allow_overwrite(scale=False)
