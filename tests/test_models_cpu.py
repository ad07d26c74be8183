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


def test_model_factory_in_the_reference_call_form():
    """create_model(name, batch_size, classes=, shape=) as deep500.networks.create_model is called."""
    cnn = create_model("simple_cnn", 64, classes=7, shape=(3, 32, 32))
    assert cnn(torch.randn(2, 3, 32, 32)).shape == (2, 7) and cnn.side == 5
    assert create_model("simple_cnn")(torch.randn(2, 1, 28, 28)).shape == (2, 10)
    assert create_model("deep_mnist", 8, classes=5)(torch.randn(2, 1, 28, 28)).shape == (2, 5)
    small = create_model("resnet", 32, classes=10, shape=(3, 32, 32), depth=8)            # CIFAR-sized input: the 6n+2 family
    assert small(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    big = create_model("resnet", 32, classes=11, shape=(3, 224, 224), depth=18)
    assert big(torch.randn(1, 3, 64, 64)).shape == (1, 11)
    with pytest.raises(KeyError, match="unknown model"):
        create_model("alexnet")


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


@pytest.mark.parametrize("size,version,params", [
    (18, 1, 11_689_512 + 4_224), (34, 1, 21_797_672 + 4_224), (50, 1, 25_557_032), (101, 1, 44_549_160), (152, 1, 60_192_808),
    (200, 1, 64_673_832), (18, 2, None), (50, 2, None), (200, 2, None)])
def test_imagenet_resnets_of_every_size(size, version, params, tmp_path):
    """Every ImageNet ResNet size (the reference's imagenet_test.py runs all sizes and versions): the v1 models have
    the parameter counts of the published architectures (1000 classes; the two building-block sizes carry 4,224 more
    because the first block of EVERY stage has a projection shortcut here, as in resnet_model.py:block_layer, where
    the common PyTorch definition leaves the first stage's out), a forward pass gives [N, classes], the variable
    layout exports and imports without loss."""
    import torch
    from eagersgd_b200 import ckpt
    from eagersgd_b200.models.resnet import imagenet_resnet
    torch.manual_seed(0)
    m = imagenet_resnet(size, version, 1000).eval()
    if params is not None:
        assert sum(p.numel() for p in m.parameters()) == params
    with torch.no_grad():
        y = m(torch.randn(1, 3, 64, 64))
    assert y.shape == (1, 1000) and torch.isfinite(y).all()
    path = str(tmp_path / "m.npz")
    ckpt.export_tf_layout(m, path)
    m2 = imagenet_resnet(size, version, 1000).eval()
    assert ckpt.import_tf_layout(m2, path) == 0               # the global step the file carries
    with torch.no_grad():
        assert torch.equal(m2(torch.ones(1, 3, 64, 64)), m(torch.ones(1, 3, 64, 64)))


def test_export_network_in_the_reference_call_form(tmp_path, monkeypatch):
    """onnx_file = export_network(name, BATCH_SIZE, classes=, shape=) and load it back, as the reference's distributed
    sample does (deep500/samples/distributed_training.py:36-39)."""
    from eagersgd_b200.graph import GraphNetwork, load_onnx
    from eagersgd_b200.models import export_network
    monkeypatch.chdir(tmp_path)
    path = export_network("simple_cnn", 64, classes=10, shape=(1, 28, 28))
    assert path == "simple_cnn.onnx" and (tmp_path / path).exists()
    g = load_onnx(path)
    assert len(g.inputs) == 1 and len(g.outputs) == 1
    x = torch.randn(3, 1, 28, 28)
    out = GraphNetwork(g).eval()(x)
    out = out[0] if isinstance(out, (list, tuple)) else out
    assert out.shape == (3, 10)
    assert export_network("deep_mnist", 8, file_path=str(tmp_path / "d.onnx")) == str(tmp_path / "d.onnx")
