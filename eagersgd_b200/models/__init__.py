"""Model zoo: ResNets (CIFAR / ImageNet), LSTM classifier, hyperplane regressor, small nets."""
from .resnet import ResNet, cifar_resnet, imagenet_resnet, count_parameters  # noqa: F401
from .hyperplane import HyperplaneRegressor, HyperplaneData  # noqa: F401
from .lstm import LSTMClassifier  # noqa: F401
from .small import MnistNet, DeepMnistNet, WideResNet  # noqa: F401

_FACTORIES = {
    "simple_mnist": lambda **kw: MnistNet(**kw), "deep_mnist": lambda **kw: DeepMnistNet(**kw),
    "wide_resnet": lambda **kw: WideResNet(**kw), "lstm": lambda **kw: LSTMClassifier(**kw),
    "hyperplane": lambda **kw: HyperplaneRegressor(**kw),
}


def create_model(name: str, **kw):
    """``create_model('resnet', depth=50, dataset='imagenet')`` etc. (deep500/networks/__init__.py)."""
    if name == "resnet":
        dataset = kw.pop("dataset", "imagenet")
        depth = kw.pop("depth", 50 if dataset == "imagenet" else 32)
        return (imagenet_resnet if dataset == "imagenet" else cifar_resnet)(depth, **kw)
    return _FACTORIES[name](**kw)


def export_network(name: str, file_path: str, **kw) -> str:
    """Write a network of this zoo as an ``.onnx`` file and return the path (deep500/networks/__init__.py:6-21)."""
    from ..graph.from_torch import export_network as _export
    return _export(name, file_path, **kw)
