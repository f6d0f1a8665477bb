"""Building blocks shared by the networks: stochastic depth, patch embedding, pointwise encoder/decoder and
MLP stacks, and the planar FFT wrappers used by the FNO variants.

Module and parameter names follow the reference (makani/models/common/layers.py:35-287) so that its
checkpoints load: `EncoderDecoder.fwd.{0,2}`, `MLP.fwd.{0,3}`.  On CUDA bf16 inputs the two-layer stacks run
as fused tcgen05 GEMM chains (`makani_b200.ops.conv.mlp2`); otherwise as plain torch modules.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ...ops import conv as conv_ops
from ...ops import linear as linear_ops


def drop_path(x: torch.Tensor, drop_prob: float = 0.0, training: bool = False) -> torch.Tensor:
    """Per-sample stochastic depth."""
    if drop_prob == 0.0 or not training:
        return x
    keep = 1.0 - drop_prob
    shape = (x.shape[0],) + (1,) * (x.ndim - 1)
    mask = keep + torch.rand(shape, dtype=x.dtype, device=x.device)
    mask.floor_()
    return x.div(keep) * mask


class DropPath(nn.Module):
    def __init__(self, drop_prob=None):
        super().__init__()
        self.drop_prob = drop_prob

    def forward(self, x):
        return drop_path(x, self.drop_prob, self.training)


class PatchEmbed(nn.Module):
    def __init__(self, img_size=(224, 224), patch_size=(16, 16), in_chans=3, embed_dim=768):
        super().__init__()
        self.img_size = img_size
        self.patch_size = patch_size
        self.red_img_size = (img_size[0] // patch_size[0], img_size[1] // patch_size[1])
        self.num_patches = self.red_img_size[0] * self.red_img_size[1]
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.proj.weight.is_shared_mp = ["spatial"]
        self.proj.bias.is_shared_mp = ["spatial"]

    def forward(self, x):
        B, C, H, W = x.shape
        assert H == self.img_size[0] and W == self.img_size[1], f"Input image size ({H}*{W}) doesn't match model ({self.img_size[0]}*{self.img_size[1]})."
        # [B, C, H, W] -> [B, embed, H/p * W/p]
        return self.proj(x).flatten(2)


def _is_gelu(act_layer) -> bool:
    return act_layer is nn.GELU


class EncoderDecoder(nn.Module):
    """`num_layers` x (pointwise linear + bias + activation) followed by a bias-free pointwise linear."""

    def __init__(self, num_layers, input_dim, output_dim, hidden_dim, act_layer, gain=1.0, input_format="nchw"):
        super().__init__()
        mods = []
        cur = input_dim
        for _ in range(num_layers):
            lin = nn.Conv2d(cur, hidden_dim, 1, bias=True) if input_format == "nchw" else nn.Linear(cur, hidden_dim, bias=True)
            nn.init.normal_(lin.weight, mean=0.0, std=math.sqrt(2.0 / cur))
            nn.init.constant_(lin.bias, 0.0)
            lin.weight.is_shared_mp = ["spatial"]
            lin.bias.is_shared_mp = ["spatial"]
            mods += [lin, act_layer()]
            cur = hidden_dim
        out = nn.Conv2d(cur, output_dim, 1, bias=False) if input_format == "nchw" else nn.Linear(cur, output_dim, bias=False)
        nn.init.normal_(out.weight, mean=0.0, std=math.sqrt(gain / cur))
        out.weight.is_shared_mp = ["spatial"]
        mods.append(out)
        self.fwd = nn.Sequential(*mods)
        self._fusable = (num_layers == 1 and input_format == "nchw" and _is_gelu(act_layer))

    def forward(self, x):
        if self._fusable and x.is_cuda and conv_ops.fast_path_ok(x):
            return conv_ops.mlp2(x, self.fwd[0].weight, self.fwd[0].bias, self.fwd[2].weight, None)
        return self.fwd(x)


class MLP(nn.Module):
    """fc1 -> act -> drop -> fc2 -> drop, pointwise over NCHW (1x1 convs) or the last dim ("traditional")."""

    def __init__(self, in_features, hidden_features=None, out_features=None, act_layer=nn.GELU, output_bias=True,
                 input_format="nchw", drop_rate=0.0, drop_type="iid", checkpointing=0, gain=1.0, **kwargs):
        super().__init__()
        self.checkpointing = checkpointing
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        if input_format == "nchw":
            fc1 = nn.Conv2d(in_features, hidden_features, 1, bias=True)
            fc2 = nn.Conv2d(hidden_features, out_features, 1, bias=output_bias)
            for p in list(fc1.parameters()) + list(fc2.parameters()):
                p.is_shared_mp = ["spatial"]
        elif input_format == "traditional":
            if drop_type == "features":
                raise NotImplementedError("feature dropout needs the nchw format")
            fc1 = nn.Linear(in_features, hidden_features, bias=True)
            fc2 = nn.Linear(hidden_features, out_features, bias=output_bias)
        else:
            raise NotImplementedError(f"input format {input_format} not supported")
        nn.init.normal_(fc1.weight, mean=0.0, std=math.sqrt(2.0 / in_features))
        nn.init.constant_(fc1.bias, 0.0)
        nn.init.normal_(fc2.weight, mean=0.0, std=math.sqrt(gain / hidden_features))
        if fc2.bias is not None:
            nn.init.constant_(fc2.bias, 0.0)
        if drop_rate > 0.0:
            drop = nn.Dropout(drop_rate) if drop_type == "iid" else nn.Dropout2d(drop_rate)
        else:
            drop = nn.Identity()
        self.fwd = nn.Sequential(fc1, act_layer(), drop, fc2, drop)
        self._fusable = (input_format == "nchw" and _is_gelu(act_layer) and drop_rate == 0.0)
        self._fusable_tokens = (input_format == "traditional" and _is_gelu(act_layer) and drop_rate == 0.0)

    def _run(self, x):
        if self._fusable and x.is_cuda and conv_ops.fast_path_ok(x):
            return conv_ops.mlp2(x, self.fwd[0].weight, self.fwd[0].bias, self.fwd[3].weight, self.fwd[3].bias)
        if self._fusable_tokens and linear_ops.fast_path_ok(x):
            return linear_ops.mlp2_lastdim(x, self.fwd[0].weight, self.fwd[0].bias, self.fwd[3].weight, self.fwd[3].bias)
        return self.fwd(x)

    def checkpoint_forward(self, x):
        """The forward pass with its activations recomputed in backward (makani/models/common/layers.py `MLP`)."""
        return checkpoint(self._run, x, use_reentrant=False)

    def forward(self, x):
        if self.checkpointing >= 2 and self.training:
            return self.checkpoint_forward(x)
        return self._run(x)


class RealFFT2(nn.Module):
    """rfft2 (ortho) truncated to the `lmax` lowest |k_lat| rows and first `mmax` columns."""

    def __init__(self, nlat, nlon, lmax=None, mmax=None):
        super().__init__()
        self.nlat, self.nlon = nlat, nlon
        self.lmax = min(lmax or nlat, nlat)
        self.mmax = min(mmax or nlon // 2 + 1, nlon // 2 + 1)
        self.truncate = not (self.lmax == nlat and self.mmax == nlon // 2 + 1)
        self.lmax_high = math.ceil(self.lmax / 2)
        self.lmax_low = math.floor(self.lmax / 2)

    def forward(self, x):
        y = torch.fft.rfft2(x, s=(self.nlat, self.nlon), dim=(-2, -1), norm="ortho")
        if self.truncate:
            parts = [y[..., : self.lmax_high, : self.mmax]]
            if self.lmax_low > 0:
                parts.append(y[..., -self.lmax_low:, : self.mmax])
            y = torch.cat(parts, dim=-2)
        return y


class InverseRealFFT2(nn.Module):
    """Inverse of `RealFFT2`: zero-pads the discarded middle rows, then irfft2 (ortho)."""

    def __init__(self, nlat, nlon, lmax=None, mmax=None):
        super().__init__()
        self.nlat, self.nlon = nlat, nlon
        self.lmax = min(lmax or nlat, nlat)
        self.mmax = min(mmax or nlon // 2 + 1, nlon // 2 + 1)
        self.truncate = not (self.lmax == nlat and self.mmax == nlon // 2 + 1)
        self.lmax_high = math.ceil(self.lmax / 2)
        self.lmax_low = math.floor(self.lmax / 2)

    def forward(self, x):
        xt = x[..., : self.mmax]
        if self.truncate:
            hi = F.pad(xt[..., : self.lmax_high, :], (0, 0, 0, self.nlat - self.lmax))
            parts = [hi]
            if self.lmax_low > 0:
                parts.append(xt[..., -self.lmax_low:, :])
            xt = torch.cat(parts, dim=-2)
        return torch.fft.irfft2(xt, s=(self.nlat, self.nlon), dim=(-2, -1), norm="ortho")
