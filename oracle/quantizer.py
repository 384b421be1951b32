"""Oracle for the parameter arithmetic of the affine quantizer modules (CPU, PyTorch tensor ops).

Restates quantization/affine/quantizer.py: get_scale (:319-342), _get_offset (:357-376),
_get_scale_offset (:869-900) and the grouped-block (LPBQ) scale derivation (:1363-1399).
Test infrastructure only.
"""

from __future__ import annotations

import torch

from . import affine as A
from .encoding_analyzer import minimum_scale


def scale_offset_from_min_max(mn, mx, qmin, qmax, symmetric):
    """Encodings a quantizer parametrised by min/max uses in forward (quantizer.py:319-376)."""
    steps = qmax - qmin
    scale = ((mx.to(torch.float32) - mn.to(torch.float32)) / steps).abs().clamp_min(minimum_scale(steps))
    if symmetric:
        offset = torch.full(mn.shape, float(-round((qmin + qmax) / 2)))
    else:
        offset = torch.clamp(torch.round(mn / scale) - qmin, -qmax, -qmin).to(torch.float32)
    return scale, offset


def dynamic_scale_offset(mn, mx, qmin, qmax, symmetric):
    """_get_scale_offset (quantizer.py:869-900): encodings used for the batch being observed."""
    steps = qmax - qmin
    mn, mx = mn.to(torch.float32), mx.to(torch.float32)
    scale = (mx - mn) / steps
    if symmetric:
        offset = torch.full_like(mn, float(-round((qmin + qmax) / 2)))
    else:
        offset = torch.round(mn / scale) - qmin
    return scale, offset


def lpbq_scale(raw_scale, bitwidth, decompressed_bw, block_grouping):
    """GroupedBlockQuantizeDequantize._get_scale (quantizer.py:1363-1399)."""
    pc_shape = [d // g if g != -1 else 1 for d, g in zip(raw_scale.shape, block_grouping)]
    grouping = A.concrete_blocks(raw_scale.shape, pc_shape, block_grouping)
    grouped = raw_scale.reshape(*A._interleave(pc_shape, grouping))
    per_channel = torch.amax(grouped, dim=tuple(range(1, grouped.dim(), 2))) / 2 ** (decompressed_bw - bitwidth)
    scale = A.quantize_dequantize(raw_scale, per_channel, torch.zeros_like(per_channel), 1,
                                  2 ** (decompressed_bw - bitwidth), block_grouping)
    return scale, per_channel
