"""ctypes binding of ``libaimet_b200.so``, the C-ABI kernel library (see ``include/aimet_b200.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libaimet_b200.so")

AB_OK = 0
AB_ERR_INVALID = -1
AB_ERR_UNSUPPORTED = -2
AB_ERR_CUDA = -3
AB_ERR_SCRATCH = -4
AB_ERR_DEVICE = -5

AB_F32, AB_F16, AB_BF16, AB_F64 = 0, 1, 2, 3
AB_MAX_DIMS = 8

DTYPE_CODE = {
    torch.float32: AB_F32,
    torch.float16: AB_F16,
    torch.bfloat16: AB_BF16,
    torch.float64: AB_F64,
}


class Layout(ctypes.Structure):
    """Mirror of ``ab_layout``."""

    _fields_ = [
        ("ndim", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("size", ctypes.c_int64 * AB_MAX_DIMS),
        ("block", ctypes.c_int64 * AB_MAX_DIMS),
    ]


def make_layout(size: Sequence[int], block: Sequence[int]) -> Layout:
    if len(size) != len(block):
        raise ValueError("size and block must have the same length")
    if len(size) > AB_MAX_DIMS:
        raise RuntimeError(f"aimet_b200 supports at most {AB_MAX_DIMS} tensor dimensions, got {len(size)}")
    lay = Layout()
    lay.ndim = len(size)
    for k, (s, b) in enumerate(zip(size, block)):
        lay.size[k] = int(s)
        lay.block[k] = int(b)
    return lay


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA kernels of aimet_b200 have not been built. "
            "Run `python -m aimet_b200.build` (needs nvcc); there is no CPU or PyTorch fallback."
        )
    return ctypes.CDLL(LIB_PATH)


lib = _load()

_vp = ctypes.c_void_p
_i32 = ctypes.c_int
_i64 = ctypes.c_int64
_f64 = ctypes.c_double
_lay = ctypes.POINTER(Layout)

# name -> (restype, argtypes); kept in one table so a test can check it against the header
SIGNATURES = {
    "aimet_b200_version": (_i32, []),
    "aimet_b200_last_error": (ctypes.c_char_p, []),
    "aimet_b200_launch_count": (_i64, []),
    "aimet_b200_quantize": (_i32, [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _vp]),
    "aimet_b200_dequantize": (_i32, [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _vp]),
    "aimet_b200_quantize_dequantize": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _f64, _vp],
    ),
    "aimet_b200_fake_quantize": (_i32, [_vp, _vp, _vp, _vp, _lay, _i32, _i64, _i64, _vp]),
    "aimet_b200_fake_quantize_backward": (_i32, [_vp, _vp, _vp, _vp, _lay, _i32, _i64, _i64, _vp, _vp]),
    "aimet_b200_backward_scratch_bytes": (_i64, [_lay, _i32]),
    "aimet_b200_quantize_dequantize_backward": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _f64, _vp, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_quantize_dequantize_backward_ex": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _f64, _f64, _f64, _vp, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_fixed_scratch_capacity": (_i64, []),
    "aimet_b200_quantize_dequantize_backward_fixed_scratch": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _f64, _vp, _vp, _vp, _vp],
    ),
    "aimet_b200_quantize_backward": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_dequantize_backward": (
        _i32,
        [_vp, _vp, _vp, _vp, _lay, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_float_fake_cast": (_i32, [_vp, _vp, _vp, _lay, _i32, _i32, _i32, _i32, _i32, _i32, _f64, _i32, _vp]),
    "aimet_b200_stats_scratch_bytes": (_i64, [_lay, _i32]),
    "aimet_b200_minmax": (_i32, [_vp, _lay, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "aimet_b200_minmax_running": (_i32, [_vp, _lay, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "aimet_b200_histogram_ex": (
        _i32,
        [_vp, _lay, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _vp],
    ),
    "aimet_b200_minmax_batches": (_i32, [_vp, _i32, _lay, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "aimet_b200_histogram_batches": (
        _i32,
        [_vp, _i32, _lay, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_histogram_edges": (_i32, [_vp, _vp, _i32, _i32, _i32, _f64, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "aimet_b200_histogram_merge_ex": (_i32, [_vp] * 7 + [_i32, _i32] + [_vp] * 6 + [_i32, _vp]),
    "aimet_b200_histogram_combine": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp]),
    "aimet_b200_histogram_update": (_i32, [_vp, _lay, _i32, _i32] + [_vp] * 17 + [_vp, _i64, _vp]),
    "aimet_b200_sqnr_encodings": (
        _i32,
        [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _f64, _f64, _f64, _f64, _vp, _vp, _vp, _vp, _vp,
         _vp, _vp],
    ),
    "aimet_b200_histogram": (
        _i32,
        [_vp, _lay, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_histogram_merge": (_i32, [_vp] * 7 + [_i32, _i32] + [_vp] * 5),
    "aimet_b200_sqnr_sweep": (
        _i32,
        [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f64, _f64, _f64, _vp, _vp, _vp],
    ),
    "aimet_b200_seqmse_blocks_scratch_bytes": (_i64, [_i64, _i64, _i64, _i32, _i32]),
    "aimet_b200_seqmse_linear_loss_blocks": (
        _i32,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _vp],
    ),
    "aimet_b200_seqmse_wait_selftest": (_i32, [_vp, _i64, _vp]),
    "aimet_b200_seqmse_scratch_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "aimet_b200_seqmse_linear_loss": (
        _i32,
        [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _vp],
    ),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    msg = lib.aimet_b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int) -> None:
    """Turn a C-ABI status into the exception the reference's Python path would raise."""
    if rc >= 0:
        return
    msg = last_error()
    if rc == AB_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"aimet_b200: {msg} (status {rc})")


def ptr_array(tensors) -> ctypes.Array:
    """A host array of the tensors' device pointers (``const void *const *`` on the C side)."""
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    """The raw handle of the device's current stream."""
    index = device.index
    if index is None:
        index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(index)  # pylint: disable=protected-access


class _Here:
    """Stands in for ``torch.cuda.device(d)`` when ``d`` already is the current device."""

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_HERE = _Here()


def on_device(device: torch.device):
    """Context in which ``device`` is the current CUDA device (kernels are launched on the current
    device): nothing to switch, and nothing to pay, in the usual case that it already is."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _HERE
    return torch.cuda.device(device)


class _Scratch:
    """One grow-only scratch tensor per (device, stream); kernels on one stream run in order,
    so sharing it between consecutive calls is safe."""

    def __init__(self):
        self._buf: dict[tuple[int, int], torch.Tensor] = {}

    def get(self, device: torch.device, nbytes: int) -> torch.Tensor | None:
        if nbytes <= 0:
            return None
        key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr(device))
        buf = self._buf.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self._buf[key] = buf
        return buf


scratch = _Scratch()
