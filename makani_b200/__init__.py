"""B200-native training and inference framework for spherical machine-learning weather models."""

__version__ = "0.1.0"


def __getattr__(name):
    # heavy drivers are imported on first use so that `import makani_b200` stays cheap
    if name == "Trainer":
        from .utils.trainer import Trainer
        return Trainer
    if name == "Inferencer":
        from .utils.inferencer import Inferencer
        return Inferencer
    raise AttributeError(name)
