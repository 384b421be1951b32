"""Quantized Conv2d / Linear wrappers (the config-4 harness): every quantizer in a small CNN
produces exactly what the oracle computes from the same input and encodings."""

import pytest
import torch
from torch import nn

from conftest import assert_same
from oracle import affine as O

pytestmark = pytest.mark.gpu


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 8, 7, stride=2, padding=3, bias=False)  # 147 weights per channel: scalar path
        self.conv2 = nn.Conv2d(8, 16, 3, padding=1)
        self.fc = nn.Linear(16, 10)

    def forward(self, x):
        x = torch.relu(self.conv1(x))
        x = torch.relu(self.conv2(x))
        return self.fc(x.mean((2, 3)))


def test_quantized_cnn_matches_oracle_layer_by_layer():
    from aimet_b200 import nn as qnn

    torch.manual_seed(0)
    model = qnn.quantize_model(_Net().cuda().eval())
    x = torch.randn(5, 3, 33, 33).cuda()
    with torch.no_grad(), qnn.compute_encodings(model):
        model(x)
    layers = list(qnn.quantized_layers(model))
    assert len(layers) == 3
    seen = []

    def spy(q):
        def hook(_m, inp, out):
            seen.append((q, inp[0].detach().clone(), out.detach().clone()))
        return q.register_forward_hook(hook)

    hooks = [spy(q) for layer in layers
             for q in (layer.input_quantizers[0], layer.output_quantizers[0], layer.param_quantizers["weight"])]
    with torch.no_grad():
        y = model(x)
        assert y.shape == (5, 10) and len(seen) == 9
        # like the reference, every forward quantizes every weight again ...
        y2 = model(x)
        assert len(seen) == 18 and torch.equal(y, y2)
        del seen[9:]
        # ... unless the caller opts in to frozen parameters for the duration of a context: then only
        # the 6 activation quantizers run per forward, with the same result
        with qnn.precomputed(model):
            y3 = model(x)
            y4 = model(x)
        assert len(seen) == 9 + 3 + 6 + 6 and torch.equal(y, y3) and torch.equal(y, y4)
        del seen[9:]
        # nothing outlives the context: edits that leave no trace in a tensor's version counter
        # (writes through .data, as batch-norm folding and cross-layer equalisation do) take effect
        layers[1].layer.weight.data.mul_(2.0)
        layers[0].input_quantizers[0].max.data.mul_(0.5)
        y5 = model(x)
        assert not torch.equal(y, y5)
        layers[1].layer.weight.data.mul_(0.5)
        layers[0].input_quantizers[0].max.data.mul_(2.0)
        assert torch.equal(model(x), y)
        del seen[9:]
    for h in hooks:
        h.remove()
    for q, inp, out in seen:
        assert q.is_initialized()
        scale, offset = q.get_scale().detach().cpu(), q.get_offset().detach().cpu()
        want = O.fake_quantize(inp.cpu(), scale, offset, q.qmin, q.qmax)  # no_grad: the fast-path arithmetic
        assert_same(out, want, f"quantizer of shape {q.shape}")
    # with gradients enabled the same modules take the QuantDequantFunc arithmetic and are trainable
    model.train()
    out = model(x)
    out.sum().backward()
    assert all(layer.param_quantizers["weight"].min.grad is not None for layer in layers)
