import pytest
import torch

from eagersgd_b200.models import create_model
from eagersgd_b200.ops.lstm import lstm_layer_reference


def test_model_factory_shapes():
    assert create_model("simple_mnist")(torch.randn(2, 1, 28, 28)).shape == (2, 10)
    assert create_model("deep_mnist")(torch.randn(2, 1, 28, 28)).shape == (2, 10)
    assert create_model("wide_resnet", depth=10, widen=2)(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    assert create_model("resnet", dataset="cifar10", depth=8)(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    assert create_model("resnet", dataset="imagenet", depth=18, num_classes=7)(torch.randn(1, 3, 64, 64)).shape == (1, 7)


def test_lstm_reference_matches_torch_lstm():
    torch.manual_seed(0)
    T, B, I, H = 6, 3, 5, 7
    ref = torch.nn.LSTM(I, H)
    x = torch.randn(T, B, I)
    y_ref, _ = ref(x)
    y = lstm_layer_reference(x, ref.weight_ih_l0, ref.weight_hh_l0, ref.bias_ih_l0 + ref.bias_hh_l0)
    assert torch.allclose(y, y_ref, atol=1e-5)


def test_lstm_classifier_trains_on_cpu():
    torch.manual_seed(1)
    m = create_model("lstm", input_dim=8, hidden=16, layers=2, num_classes=3)
    opt = torch.optim.SGD(m.parameters(), lr=0.5)
    x = torch.randn(12, 5, 8)
    y = torch.randint(0, 3, (12,))
    first = None
    for _ in range(30):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(m(x), y)
        loss.backward()
        opt.step()
        first = first or loss.item()
    assert loss.item() < first
