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
        for layer in layers:
            layer.layer.weight.add_(0)  # an in-place update: the kept quantized weight must be refreshed
        y = model(x)
        assert y.shape == (5, 10) and len(seen) == 9
        # a second forward reuses the quantized weights (6 activation quantizer calls only), same result
        y2 = model(x)
        assert len(seen) == 15 and torch.equal(y, y2)
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
