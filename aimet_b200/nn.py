"""Quantized Conv2d / Linear wrappers and a model-level calibration context.

A small mirror of the part of aimet_torch's quantized-module layer that a QuantSim forward of a
convolutional model exercises (nn/base.py:258-325 ``_patch_quantized_parameters``, nn/true_quant.py:600-616
``_forward_no_dispatch``, nn/__init__.py:22-84 ``compute_encodings``): a wrapped layer quantizes its
weight with ``param_quantizers["weight"]`` on every forward, its input with ``input_quantizers[0]``
and its output with ``output_quantizers[0]``.  It is a caller of the hot path, not a QuantSim
replacement: no config files, no graph analysis, no supergroups.
"""

from __future__ import annotations

import contextlib
import math
from typing import Callable, Iterable, Optional

import torch
from torch import nn

from .encoding_analyzer import MinMaxEncodingAnalyzer
from .quantizer import QuantizeDequantize

__all__ = ["QuantizedLayer", "quantize_model", "compute_encodings", "quantized_layers", "precomputed"]


class QuantizedLayer(nn.Module):
    """``out = Q_out(layer(Q_in(x)))`` with the layer's weight replaced by ``Q_w(weight)``."""

    def __init__(self, layer: nn.Module, input_quantizer=None, output_quantizer=None, weight_quantizer=None):
        super().__init__()
        if not isinstance(layer, (nn.Conv2d, nn.Linear)):
            raise NotImplementedError(f"QuantizedLayer wraps Conv2d and Linear, got {type(layer).__name__}")
        self.layer = layer
        self.input_quantizers = nn.ModuleList([input_quantizer])
        self.output_quantizers = nn.ModuleList([output_quantizer])
        self.param_quantizers = nn.ModuleDict({"weight": weight_quantizer, "bias": None})

    @property
    def weight(self):
        return self.layer.weight

    def _quantized_weight(self, qw):
        """The quantize-dequantized weight: computed on every forward like the reference
        (nn/base.py:296-325), unless :func:`precomputed` holds it for the duration of a context."""
        held = self.__dict__.get("_held_weight")
        if held is not None and not torch.is_grad_enabled() and getattr(qw, "_observer_hook", None) is None:
            return held
        return qw(self.layer.weight)

    def forward(self, x):
        qi, qo, qw = self.input_quantizers[0], self.output_quantizers[0], self.param_quantizers["weight"]
        if qi is not None:
            x = qi(x)
        w = self.layer.weight if qw is None else self._quantized_weight(qw)
        if isinstance(self.layer, nn.Conv2d):
            out = self.layer._conv_forward(x, w, self.layer.bias)  # pylint: disable=protected-access
        else:
            out = nn.functional.linear(x, w, self.layer.bias)
        return out if qo is None else qo(out)


def _per_channel_shape(weight: torch.Tensor):
    return (weight.shape[0],) + (1,) * (weight.dim() - 1)


def quantize_model(model: nn.Module, *, param_bw: int = 8, act_bw: int = 8,
                   analyzer_factory: Optional[Callable] = None) -> nn.Module:
    """Replace every Conv2d / Linear of ``model`` in place by a :class:`QuantizedLayer` with a
    per-channel symmetric weight quantizer and per-tensor asymmetric input and output quantizers
    (every conv / linear input and output per-tensor, weights per-channel).  ``analyzer_factory(shape)`` builds the activation
    analyzers (default: min-max)."""
    factory = analyzer_factory or (lambda shape: MinMaxEncodingAnalyzer(shape))
    for name, child in list(model.named_children()):
        if isinstance(child, (nn.Conv2d, nn.Linear)):
            dev = child.weight.device
            wrapped = QuantizedLayer(
                child,
                QuantizeDequantize((), act_bw, False, encoding_analyzer=factory(())),
                QuantizeDequantize((), act_bw, False, encoding_analyzer=factory(())),
                QuantizeDequantize(_per_channel_shape(child.weight), param_bw, True),
            ).to(dev)
            setattr(model, name, wrapped)
        else:
            quantize_model(child, param_bw=param_bw, act_bw=act_bw, analyzer_factory=analyzer_factory)
    return model


def quantized_layers(model: nn.Module) -> Iterable[QuantizedLayer]:
    return (m for m in model.modules() if isinstance(m, QuantizedLayer))


@contextlib.contextmanager
def compute_encodings(model: nn.Module, group=None):
    """Calibrate every quantizer of the model from the forward passes run inside the context
    (nn/__init__.py:22-84, nn/base.py:331-427): weights are calibrated on entry, activation quantizers
    observe in pass-through mode and get their ranges on exit.

    The weights are quantized once on entry and held for the forwards inside the context (they are
    taken as fixed while calibration data runs through; forwards with gradients enabled quantize
    them afresh).  An observing quantizer costs two kernel launches per forward (the running min / max is updated
    on the device, nothing is allocated or copied; the reference clones every observed activation).
    ``group``: a ``torch.distributed`` process group whose ranks each run a share of the calibration
    batches through their replica of the model (data-parallel calibration): on exit the min / max
    statistics of all quantizers travel in one all-reduce, so every rank ends with the encodings of
    the whole calibration set."""
    from .quantizer import finish_calibration

    quantizers, weight_quantizers = [], []
    layers = list(quantized_layers(model))
    with torch.no_grad(), contextlib.ExitStack() as stack:  # weights: observed once, in pass-through mode
        for layer in layers:
            qw = layer.param_quantizers["weight"]
            if qw is not None and qw.is_overwrite_allowed():
                stack.enter_context(qw._compute_encodings(passthrough=True, clone=False, finish=False))  # pylint: disable=protected-access
                qw(layer.layer.weight.detach())
                weight_quantizers.append(qw)
    finish_calibration(weight_quantizers)
    with contextlib.ExitStack() as stack:
        for layer in layers:
            for q in (*layer.input_quantizers, *layer.output_quantizers):
                if q is not None and q.is_overwrite_allowed():
                    stack.enter_context(q._compute_encodings(passthrough=True, clone=False, finish=False))  # pylint: disable=protected-access
                    quantizers.append(q)
        # the weights do not change while the calibration data runs through: each is quantized once
        # here instead of on every forward inside the context (no-grad forwards only)
        _hold_quantized_weights(layers)
        try:
            yield
        finally:
            for layer in layers:
                layer.__dict__.pop("_held_weight", None)
    if group is not None:
        _allreduce_minmax_statistics(quantizers, group)
    finish_calibration(quantizers)


def _hold_quantized_weights(layers):
    """Quantize the weight of every layer once and keep it on the layer (popped by the caller).  The
    scales and offsets of all weight quantizers come from one batched derivation: one by one, the
    few small tensor operations per quantizer cost more than quantizing the weights."""
    from .quantizer import derive_encodings

    pairs = [(layer, layer.param_quantizers["weight"]) for layer in layers]
    pairs = [(layer, qw) for layer, qw in pairs if qw is not None and qw.is_initialized()]
    with torch.no_grad():
        for (layer, qw), enc in zip(pairs, derive_encodings([qw for _, qw in pairs])):
            with qw._set_encodings(enc):  # pylint: disable=protected-access
                layer.__dict__["_held_weight"] = qw(layer.layer.weight).detach()


def _allreduce_minmax_statistics(quantizers, group):
    """One MIN all-reduce over the concatenation of every quantizer's (min, -max)."""
    from . import distributed as D
    from .encoding_analyzer import _MinMaxObserver, _MinMaxRange

    obs = [q.encoding_analyzer.observer for q in quantizers]
    if not all(isinstance(o, _MinMaxObserver) for o in obs):
        raise NotImplementedError("data-parallel model calibration combines min-max statistics; histogram analyzers "
                                  "need their range before binning (see distributed.calibrate_histogram)")
    dev = next((o.get_stats().min.device for o in obs if o.get_stats().min is not None), None)
    if dev is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    parts = []
    for o in obs:
        st = o.get_stats()
        n = math.prod(o.shape)
        if st.min is None:  # this rank saw nothing for this quantizer
            parts += [torch.full((n,), float("inf"), device=dev), torch.full((n,), float("inf"), device=dev)]
        else:
            parts += [st.min.reshape(-1).float(), -st.max.reshape(-1).float()]
    packed = torch.cat(parts)
    D._collective(torch.distributed.all_reduce, packed, op=torch.distributed.ReduceOp.MIN, group=group)  # pylint: disable=protected-access
    at = 0
    for o in obs:
        st = o.get_stats()
        n = math.prod(o.shape)
        mn, mx = packed[at:at + n], -packed[at + n:at + 2 * n]
        at += 2 * n
        dtype = st.min.dtype if st.min is not None else torch.float32
        if bool(torch.isinf(mn).all()):
            continue  # no rank observed this quantizer
        o.stats = _MinMaxRange(mn.to(dtype).reshape(o.shape), mx.to(dtype).reshape(o.shape))

@contextlib.contextmanager
def precomputed(model: nn.Module):
    """Inference with frozen parameters: inside the context every quantizer derives its scale and
    offset once (the reference's ``_precompute_encodings``, quantizer.py:790-804, entered for a whole
    model as in aimet_torch/utils.py:1666) and every layer quantizes its weight once instead of on
    every forward (what the reference's ``fold_param_quantizers`` achieves, nn/base.py:1103-1155,
    without giving up the quantizers).  Nothing is cached outside the context, so weights and
    ranges may be edited freely (in place, through ``.data``, by re-assignment) between contexts."""
    from .quantizer import derive_encodings

    with contextlib.ExitStack() as stack, torch.no_grad():
        layers = list(quantized_layers(model))
        frozen = [q for layer in layers
                  for q in (*layer.input_quantizers, *layer.output_quantizers, layer.param_quantizers["weight"])
                  if q is not None and q.is_initialized()]
        for q, enc in zip(frozen, derive_encodings(frozen)):
            stack.enter_context(q._set_encodings(enc))  # pylint: disable=protected-access
        for layer in layers:
            qw = layer.param_quantizers["weight"]
            if qw is not None and qw.is_initialized():
                layer.__dict__["_held_weight"] = qw(layer.layer.weight).detach()
        try:
            yield model
        finally:
            for layer in layers:
                layer.__dict__.pop("_held_weight", None)
