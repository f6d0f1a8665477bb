"""Adaptive Fourier Neural Operator, NCHW variant with complex block-diagonal kernels, instance/layer norm and
an optional (linear / identity) skip around the spectral filter.  Architecture and parameter names follow
makani/models/networks/afnonet_v2.py:34-314."""

from __future__ import annotations

from functools import partial

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..common.activations import ComplexReLU
from ..common.layers import MLP, DropPath, PatchEmbed


def compl_mul_add_fwd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Real-arithmetic complex product: a [b,k,i,x,y,2], b [k,i,o,2] -> [b,k,o,x,y,2]."""
    tmp = torch.einsum("bkixys,kior->srbkoxy", a, b)
    return torch.stack([tmp[0, 0] - tmp[1, 1], tmp[1, 0] + tmp[0, 1]], dim=-1)


def compl_mul_add_fwd_c(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.view_as_real(torch.einsum("bkixy,kio->bkoxy", torch.view_as_complex(a), torch.view_as_complex(b)))


class AFNO2D(nn.Module):
    def __init__(self, hidden_size, num_blocks=8, sparsity_threshold=0.0, hard_thresholding_fraction=1, hidden_size_factor=1,
                 use_complex_kernels=False):
        super().__init__()
        assert hidden_size % num_blocks == 0, f"hidden_size {hidden_size} should be divisble by num_blocks {num_blocks}"
        self.hidden_size, self.num_blocks = hidden_size, num_blocks
        self.sparsity_threshold = sparsity_threshold
        self.block_size = hidden_size // num_blocks
        self.hard_thresholding_fraction = hard_thresholding_fraction
        self.hidden_size_factor = hidden_size_factor
        self.scale = 0.02
        self.mult_handle = compl_mul_add_fwd_c if use_complex_kernels else compl_mul_add_fwd
        bs, f = self.block_size, hidden_size_factor
        self.w1 = nn.Parameter(self.scale * torch.randn(num_blocks, bs, bs * f, 2))
        self.b1 = nn.Parameter(self.scale * torch.randn(1, num_blocks * bs, 1, 1))
        self.w2 = nn.Parameter(self.scale * torch.randn(num_blocks, bs * f, bs, 2))
        self.act = ComplexReLU(negative_slope=0.0, mode="cartesian")

    def forward(self, x):
        bias = x
        dtype = x.dtype
        x = x.float()
        B, C, H, W = x.shape
        tot_h, tot_w = H // 2 + 1, W // 2 + 1
        kept_h = int(tot_h * self.hard_thresholding_fraction)
        kept_w = int(tot_w * self.hard_thresholding_fraction)
        xf = torch.fft.rfft2(x, dim=(-2, -1), norm="ortho").view(B, self.num_blocks, self.block_size, H, W // 2 + 1)
        xr = torch.view_as_real(xf)
        out = torch.zeros_like(xr)

        def mlp(z):
            o = torch.view_as_real(self.act(torch.view_as_complex(self.mult_handle(z.contiguous(), self.w1).contiguous())))
            return self.mult_handle(o.contiguous(), self.w2)

        if kept_h == tot_h:
            out[:, :, :, :, :kept_w] = mlp(xr[:, :, :, :, :kept_w])
        else:
            out[:, :, :, :kept_h, :kept_w] = mlp(xr[:, :, :, :kept_h, :kept_w])
            out[:, :, :, -kept_h:, :kept_w] = mlp(xr[:, :, :, -kept_h:, :kept_w])
        out = F.softshrink(out, lambd=self.sparsity_threshold)
        out = torch.view_as_complex(out).reshape(B, C, H, W // 2 + 1)
        y = torch.fft.irfft2(out, s=(H, W), dim=(-2, -1), norm="ortho").to(dtype)
        return y + self.b1.to(dtype) + bias


class Block(nn.Module):
    def __init__(self, h, w, dim, mlp_ratio=4.0, drop=0.0, drop_path=0.0, act_layer=nn.GELU, norm_layer=nn.LayerNorm,
                 num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1.0, use_complex_kernels=True,
                 skip_fno="linear", nested_skip_fno=True, checkpointing=False, verbose=True):
        super().__init__()
        self.norm1 = norm_layer()
        if skip_fno == "linear":
            self.skip_layer = nn.Conv2d(dim, dim, 1, 1)
        elif skip_fno == "identity":
            self.skip_layer = nn.Identity()
        else:
            skip_fno = None
        self.skip_fno, self.nested_skip_fno = skip_fno, nested_skip_fno
        self.filter = AFNO2D(dim, num_blocks, sparsity_threshold, hard_thresholding_fraction, use_complex_kernels=use_complex_kernels)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = norm_layer()
        self.mlp = MLP(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop_rate=drop,
                       checkpointing=2 if checkpointing else 0)

    def forward(self, x):
        residual = x
        x = self.filter(self.norm1(x))
        if self.skip_fno is not None:
            x = x + self.skip_layer(residual)
            if not self.nested_skip_fno:
                residual = x
        x = self.mlp(self.norm2(x))
        return self.drop_path(x) + residual


class AdaptiveFourierNeuralOperatorNet(nn.Module):
    def __init__(self, inp_shape=(720, 1440), patch_size=(16, 16), inp_chans=2, out_chans=2, embed_dim=768, num_layers=12,
                 mlp_ratio=4.0, drop_rate=0.0, drop_path_rate=0.0, num_blocks=16, sparsity_threshold=0.01,
                 normalization_layer="instance_norm", skip_fno="linear", nested_skip_fno=True, hard_thresholding_fraction=1.0,
                 checkpointing=False, use_complex_kernels=True, verbose=False, **kwargs):
        super().__init__()
        self.img_size, self.patch_size = tuple(inp_shape), tuple(patch_size)
        self.inp_chans, self.out_chans, self.embed_dim = inp_chans, out_chans, embed_dim
        assert len(patch_size) == 2, f"Expected patch_size to have two entries but got {patch_size} instead"
        assert self.img_size[0] % self.patch_size[0] == 0 and self.img_size[1] % self.patch_size[1] == 0, \
            f"the patch size {self.patch_size} does not divide the image dimensions {self.img_size} evenly"
        self.patch_embed = PatchEmbed(img_size=self.img_size, patch_size=self.patch_size, in_chans=inp_chans, embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, embed_dim, self.patch_embed.num_patches))
        self.pos_drop = nn.Dropout(p=drop_rate) if drop_rate > 0.0 else nn.Identity()
        dpr = [x.item() for x in torch.linspace(0, drop_path_rate, num_layers)]
        self.h = self.img_size[0] // self.patch_size[0]
        self.w = self.img_size[1] // self.patch_size[1]
        if normalization_layer == "layer_norm":
            norm_layer = partial(nn.LayerNorm, normalized_shape=(self.h, self.w), eps=1e-6)
        elif normalization_layer == "instance_norm":
            norm_layer = partial(nn.InstanceNorm2d, num_features=embed_dim, eps=1e-6, affine=True, track_running_stats=False)
        else:
            raise NotImplementedError(f"normalization {normalization_layer} not implemented")
        self.blocks = nn.ModuleList([
            Block(h=self.h, w=self.w, dim=embed_dim, mlp_ratio=mlp_ratio, drop=drop_rate, drop_path=dpr[i], norm_layer=norm_layer,
                  num_blocks=num_blocks, sparsity_threshold=sparsity_threshold, hard_thresholding_fraction=hard_thresholding_fraction,
                  use_complex_kernels=use_complex_kernels, skip_fno=skip_fno, nested_skip_fno=nested_skip_fno,
                  checkpointing=checkpointing, verbose=verbose) for i in range(num_layers)])
        self.head = nn.Conv2d(embed_dim, out_chans * self.patch_size[0] * self.patch_size[1], 1, bias=False)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    def _init_weights(self, m):
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    @torch.jit.ignore
    def no_weight_decay(self):
        return {"pos_embed", "cls_token"}

    def forward_features(self, x):
        B = x.shape[0]
        x = self.patch_embed(x)
        x = self.pos_drop(x + self.pos_embed.to(x.dtype))
        x = x.reshape(B, self.embed_dim, self.h, self.w)
        for blk in self.blocks:
            x = blk(x)
        return x

    def forward(self, x):
        x = self.head(self.forward_features(x))
        b = x.shape[0]
        xv = x.view(b, self.patch_size[0], self.patch_size[1], -1, self.h, self.w)
        xvt = torch.permute(xv, (0, 3, 4, 1, 5, 2)).contiguous()
        return xvt.view(b, -1, self.h * self.patch_size[0], self.w * self.patch_size[1])
