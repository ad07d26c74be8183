"""Model zoo: ResNets (CIFAR / ImageNet), LSTM classifier, hyperplane regressor, small nets."""
from .resnet import ResNet, cifar_resnet, imagenet_resnet, count_parameters  # noqa: F401
from .hyperplane import HyperplaneRegressor, HyperplaneData  # noqa: F401
from .lstm import LSTMClassifier  # noqa: F401
from .small import MnistNet, SimpleCNN, DeepMnistNet, WideResNet  # noqa: F401

_FACTORIES = {
    "simple_mnist": lambda **kw: MnistNet(**kw), "simple_cnn": lambda **kw: SimpleCNN(**kw), "deep_mnist": lambda **kw: DeepMnistNet(**kw),
    "wide_resnet": lambda **kw: WideResNet(**kw), "lstm": lambda **kw: LSTMClassifier(**kw),
    "hyperplane": lambda **kw: HyperplaneRegressor(**kw),
}


def create_model(name: str, *args, **kw):
    """``create_model('resnet', depth=50, dataset='imagenet')`` etc.  The reference's call form works too:
    ``create_model(name, batch_size, classes=..., shape=(C, H, W), **model_kwargs)`` — the batch size is not needed
    here, ``classes`` sizes the output layer, and for a ResNet the height of ``shape`` chooses between the CIFAR
    (6n+2) and the ImageNet architectures (deep500/networks/__init__.py:23-37)."""
    classes, shape = kw.pop("classes", None), kw.pop("shape", None)
    if name == "resnet":
        dataset = kw.pop("dataset", None) or ("imagenet" if shape is None or shape[-1] >= 64 else "cifar10")
        depth = kw.pop("depth", 50 if dataset == "imagenet" else 32)
        if classes is not None:
            kw.setdefault("num_classes", classes)
        return (imagenet_resnet if dataset == "imagenet" else cifar_resnet)(depth, **kw)
    if name not in _FACTORIES:
        raise KeyError("unknown model %r (known: resnet, %s)" % (name, ", ".join(sorted(_FACTORIES))))
    if classes is not None and name not in ("hyperplane",):
        kw.setdefault("num_classes" if name == "lstm" else "classes", classes)
    if shape is not None and name == "simple_cnn":
        kw.setdefault("in_channels", shape[0])
        kw.setdefault("size", shape[1])
    return _FACTORIES[name](**kw)


def export_network(name: str, path_or_batch_size=None, *, file_path=None, **kw) -> str:
    """Write a network of this zoo as an ``.onnx`` file and return the path: ``export_network(name, path, **model_kwargs)``,
    or in the reference's call form ``export_network(name, batch_size, classes=, shape=, file_path=...)``, where the file
    defaults to ``<name>.onnx`` in the working directory (deep500/networks/__init__.py:6-21)."""
    from ..graph.from_torch import export_network as _export
    if isinstance(path_or_batch_size, str) and file_path is None:
        file_path = path_or_batch_size
    return _export(name, file_path, **kw)
