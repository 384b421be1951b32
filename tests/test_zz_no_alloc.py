"""The allocation-free backward entry point, called through the C ABI.

Some hosts of this library run where device memory is not theirs to allocate (an operator inside a
serving runtime that owns the allocator, a worker that has committed all memory to a pool), so they
cannot bring the scratch buffer the ordinary backward entry point asks for.
``aimet_b200_quantize_dequantize_backward_fixed_scratch`` keeps the partial sums in a fixed array
inside the library instead.  It must return exactly what the ordinary entry point returns, also on
a second call that finds the first call's leftovers in the array.  (Collected last on purpose.)
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_both(x, g, scale, offset, size, block, ct, qmin, qmax, want_offset_grad):
    from aimet_b200 import _lib

    lib = _lib.lib
    lay = _lib.make_layout(size, block)
    io = _lib.DTYPE_CODE[x.dtype]
    st = torch.cuda.current_stream().cuda_stream
    need = lib.aimet_b200_backward_scratch_bytes(lay, io)
    assert 0 <= need <= lib.aimet_b200_fixed_scratch_capacity()
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    outs = []
    for fixed in (False, True):
        gx = torch.empty_like(x)
        gs = torch.full_like(scale, float("nan"))
        go = torch.full_like(scale, float("nan")) if want_offset_grad else None
        common = (x.data_ptr(), g.data_ptr(), scale.data_ptr(), offset.data_ptr(), lay, io, ct, _lib.AB_F32, qmin, qmax,
                  0.0, gx.data_ptr(), gs.data_ptr(), None if go is None else go.data_ptr())
        if fixed:
            rc = lib.aimet_b200_quantize_dequantize_backward_fixed_scratch(*common, st)
        else:
            rc = lib.aimet_b200_quantize_dequantize_backward(*common, scratch.data_ptr(), scratch.numel(), st)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        outs.append((gx, gs, go))
    return outs


def test_fixed_scratch_matches_ordinary_entry_point_twice_in_a_row():
    from aimet_b200 import _lib

    g = torch.Generator().manual_seed(123)
    # per-tensor float32 (partials + finishing kernel), then per-channel NCHW bf16 (outer dim > 1):
    # both layouts go through the scratch array, and the second call starts from the first one's data
    calls = [
        (torch.float32, (384, 1024), (), [384, 1024], [384, 1024], _lib.AB_F32, 0, 255, True),
        (torch.bfloat16, (8, 48, 40, 40), (48, 1, 1), [8, 48, 40, 40], [8, 1, 40, 40], _lib.AB_F32, -128, 127, False),
    ]
    for dtype, shape, pshape, size, block, ct, qmin, qmax, want_go in calls:
        x = (torch.randn(shape, generator=g) * (1 + 6 * (torch.rand(shape, generator=g) < 0.02))).to(dtype).cuda()
        gy = torch.randn(shape, generator=g).to(dtype).cuda()
        scale = ((4.0 / (qmax - qmin)) * (0.5 + torch.rand(pshape, generator=g))).cuda().contiguous()
        offset = (torch.round(-(qmax - qmin) * 0.5 * torch.ones(pshape)) - qmin).cuda().contiguous()
        (gx0, gs0, go0), (gx1, gs1, go1) = _call_both(x, gy, scale, offset, size, block, ct, qmin, qmax, want_go)
        # same kernels, same reduction order: bit-identical (tolerance of the other tests: exact for
        # grad_x, 1e-5 relative for the parameter gradients)
        assert torch.equal(gx0, gx1)
        assert torch.equal(gs0, gs1) and not torch.isnan(gs1).any()
        if want_go:
            assert torch.equal(go0, go1) and not torch.isnan(go1).any()
        # and both agree with the CPU oracle of the reference's backward pass
        from oracle import affine as O

        ogx, ogs, ogo = O.quantize_dequantize_backward(x.cpu(), gy.cpu(), scale.cpu(), offset.cpu(), qmin, qmax)
        assert torch.equal(gx1.cpu(), ogx)
        # sums taken in another order than torch's: 1e-5 of the result, or, where the terms cancel
        # (a per-tensor sum of signed terms may land near zero), of the terms' root-sum-square
        gnorm = float(gy.float().norm())
        for got, want, rss in ((gs1, ogs, 0.5 * gnorm), (go1, ogo, float(scale.max()) * gnorm) if want_go else (None, None, 0)):
            if got is not None:
                want = want.reshape(got.shape).double()
                assert (got.cpu().double() - want).abs().max() <= 1e-5 * max(float(want.abs().max()), rss)


def test_fixed_scratch_refuses_oversized_layouts():
    from aimet_b200 import _lib

    lib = _lib.lib
    # column mode with a long row: partials = row tiles x row length, far beyond 1 MiB
    size, block = [4096, 65536], [4096, 1]
    lay = _lib.make_layout(size, block)
    assert lib.aimet_b200_backward_scratch_bytes(lay, _lib.AB_F32) > lib.aimet_b200_fixed_scratch_capacity()
    dummy = torch.zeros(16, device="cuda")
    rc = lib.aimet_b200_quantize_dequantize_backward_fixed_scratch(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), lay, _lib.AB_F32, _lib.AB_F32,
        _lib.AB_F32, 0, 255, 0.0, dummy.data_ptr(), dummy.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.AB_ERR_SCRATCH
    assert "built-in buffer" in _lib.last_error()
