"""aimet_b200 -- the quantization-simulation hot path of aimet_torch on B200 (sm_100a) kernels.

* :mod:`aimet_b200.backend` -- ``quantize`` / ``dequantize`` / ``quantize_dequantize`` functionals
  (aimet_torch's backend protocol); :func:`register_backend` plugs them into an installed aimet_torch.
* :mod:`aimet_b200.functional` -- the same three functions for stand-alone use, with the reference's
  ``(qmin, qmax)`` / ``(bitwidth, signed)`` / ``num_steps=`` call forms (``aimet_b200.quantize`` ...).
* :mod:`aimet_b200.quantizer` -- ``Quantize``, ``QuantizeDequantize``, ``Dequantize``,
  ``GroupedBlockQuantizeDequantize`` modules with learnable ranges.
* :mod:`aimet_b200.float_quantizer` -- ``FloatQuantizeDequantize`` (fp16 / bf16 / fp8 / fp4 fake-cast), MXFP4, NVFP4.
* :mod:`aimet_b200.encoding_analyzer` -- MinMax / Percentile / SQNR / TF-enhanced analyzers.
* :mod:`aimet_b200.seq_mse` -- SeqMSE candidate search for Linear layers.
* :mod:`aimet_b200.distributed` -- sharded calibration and output-channel sharding helpers.

Everything runs through ``libaimet_b200.so`` (``include/aimet_b200.h``); importing the package
fails if that library has not been built (``python -m aimet_b200.build``).
"""

import importlib

__all__ = [
    "backend", "functional", "quantizer", "float_quantizer", "encoding_analyzer", "seq_mse", "distributed", "nn",
    "quantize", "dequantize", "quantize_dequantize", "register_backend",
]

_SUBMODULES = ("_lib", "backend", "functional", "pgs", "quantizer", "float_quantizer", "encoding_analyzer", "seq_mse", "distributed", "nn",
               "build")
_FUNCTIONS = ("quantize", "dequantize", "quantize_dequantize")


def __getattr__(name):
    # Submodules load on first use so that ``python -m aimet_b200.build`` can run before the kernel
    # library exists.  Anything else needs ``_lib`` and raises ImportError if the library is missing.
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    if name in _FUNCTIONS:
        return getattr(importlib.import_module(f"{__name__}.functional"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def register_backend(name: str = "b200", select: bool = False):
    """Register this backend with an installed ``aimet_torch`` under ``name``
    (quantization/affine/backends/utils.py:110-114) and optionally make it the active one."""
    from aimet_torch.quantization.affine.backends import utils as _ref_backends  # pylint: disable=import-error

    backend = importlib.import_module(f"{__name__}.backend")
    _ref_backends.add_backend(name, backend)
    if select:
        return _ref_backends.set_backend(name)
    return None
