"""`modulus.Module.from_torch(torch_class, meta)`: returns a subclass of the torch module that carries the metadata."""

import torch.nn as nn


class Module(nn.Module):
    def __init__(self, meta=None):
        super().__init__()
        self.meta = meta

    @staticmethod
    def from_torch(torch_model_class, meta=None):
        class ModulusModel(torch_model_class):
            def __init__(self, *args, **kwargs):
                super().__init__(*args, **kwargs)
                self.meta = meta

        ModulusModel.__name__ = torch_model_class.__name__ + "ModulusModel"
        return ModulusModel
