"""Training: the step API, trainer and events, metrics, schedules, injectors, loggers, mains."""
from .step import TrainStep, prepare_model  # noqa: F401
from .trainer import Trainer, test_training  # noqa: F401
from .executor import GraphExecutor, Network, classification_loss, mse_loss  # noqa: F401
