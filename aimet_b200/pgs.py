"""Pivot gradient spiking: a process-wide switch that multiplies the straight-through input
gradient of quantize-dequantize for elements close to a rounding boundary (the reference's
``aimet_torch.experimental.pgs``; consumed in QuantDequantFunc, torch_builtins.py:259, 759-760,
790-821).  Off by default."""

__all__ = ["enable_pgs", "disable_pgs", "is_pgs_enabled", "get_pgs_eps", "get_pgs_multiplier"]

_eps: float = 0.0
_multiplier: float = 1.0


def enable_pgs(eps: float = 0.05, multiplier: float = 3.0):
    """Elements whose rounding error exceeds ``(1 - eps) / 2`` get ``multiplier`` times the upstream
    gradient."""
    global _eps, _multiplier  # pylint: disable=global-statement
    if not 0.0 < eps <= 1.0:
        raise ValueError(f"eps must be ∈ (0, 1] to enable PGS. Got {eps}")
    if multiplier == 1.0:
        raise ValueError("multiplier must be ≠1 to enable PGS")
    _eps, _multiplier = eps, multiplier


def disable_pgs():
    global _eps, _multiplier  # pylint: disable=global-statement
    _eps, _multiplier = 0.0, 1.0


def is_pgs_enabled() -> bool:
    return _eps > 0.0 and _multiplier != 1.0


def get_pgs_eps() -> float:
    return _eps


def get_pgs_multiplier() -> float:
    return _multiplier
