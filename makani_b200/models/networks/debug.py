"""Identity-like network used by the autoregression self test (`--mode test`): y = factor * x."""

import torch
import torch.nn as nn


class DebugNet(nn.Module):
    def __init__(self, inp_shape=(16, 16), out_shape=(16, 16), inp_chans=2, out_chans=2, **kwargs):
        super().__init__()
        self.factor = nn.Parameter(torch.ones(1))

    def forward(self, x):
        return self.factor * x
