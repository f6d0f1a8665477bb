"""Image helpers (behaviour of makani/utils/img_utils.py:34-110): periodic padding in longitude."""

import torch
import torch.nn as nn
import torch.nn.functional as F


class PeriodicPad2d(nn.Module):
    """Circular padding in the last (longitude) dimension, zero padding in latitude."""

    def __init__(self, pad_width):
        super().__init__()
        self.pad_width = pad_width

    def forward(self, x):
        out = F.pad(x, (self.pad_width, self.pad_width, 0, 0), mode="circular")
        return F.pad(out, (0, 0, self.pad_width, self.pad_width), mode="constant", value=0)
