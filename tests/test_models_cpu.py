"""Every architecture of the zoo builds, runs a 32 x 32 batch and matches the upstream
definition's parameter names and shapes (when the upstream research code is available)."""
import os
import sys

import pytest
import torch

from powersgd_b200 import models as zoo

from conftest import ROOT

CIFAR_MODELS = [
    "ResNet18", "ResNet50", "PreActResNet18", "PreActResNet50", "SENet18", "vgg11", "vgg16_bn", "LeNet", "MobileNet",
    "MobileNetV2", "ResNeXt29_2x64d", "ResNeXt29_32x4d", "DPN26", "GoogLeNet", "densenet_cifar", "DenseNet121",
    "ShuffleNetG2", "ShuffleNetG3", "PNASNetA", "PNASNetB",
]


def _upstream(name):
    arch = os.path.join(ROOT, "baseline", "_ref", "paper_code", "tasks", "cifar_architectures")
    if not os.path.isdir(arch):
        return None
    sys.path.insert(0, os.path.dirname(arch))
    try:
        import cifar_architectures as up  # noqa: F401
    except Exception:
        return None
    finally:
        sys.path.pop(0)
    return getattr(up, name, None)


@pytest.mark.parametrize("name", CIFAR_MODELS)
def test_cifar_model_forward_and_parameter_parity(name):
    torch.manual_seed(0)
    model = getattr(zoo, name)()
    model.eval()
    with torch.no_grad():
        out = model(torch.randn(2, 3, 32, 32))
    assert out.shape == (2, 10) and torch.isfinite(out).all()
    ctor = _upstream(name)
    if ctor is None or name.startswith("ShuffleNet"):  # upstream ShuffleNet no longer constructs (float channel counts)
        return
    ref = ctor()
    ours = {k: tuple(v.shape) for k, v in model.named_parameters()}
    theirs = {k: tuple(v.shape) for k, v in ref.named_parameters()}
    assert ours == theirs


def test_lstm_and_gpt2():
    lm = zoo.RNNModel("LSTM", 50, 8, 8, 2, dropout=0.0, tie_weights=True)
    assert lm.decoder.weight is lm.encoder.weight
    h = lm.init_hidden(3)
    out, h2 = lm(torch.randint(0, 50, (5, 3)), h)
    assert out.shape == (5, 3, 50)
    assert all(not t.requires_grad for t in lm.repackage_hidden(h2))
    full = zoo.wikitext2_lstm()
    shapes = sorted(tuple(p.shape) for p in full.parameters() if p.dim() == 2)
    assert (33278, 650) in shapes and shapes.count((2600, 650)) == 6
    g = zoo.GPT2(zoo.GPT2Config.tiny())
    t = torch.randint(0, 512, (2, 16))
    loss = g.loss(t, t)
    loss.backward()
    assert torch.isfinite(loss)
    assert zoo.GPT2Config.medium().n_layer == 24 and zoo.GPT2Config.medium().n_embd == 1024
