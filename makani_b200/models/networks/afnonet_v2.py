"""AFNO, second generation ("AFNO" in the registry): patch tokens on an [embed, h, w] grid, per block

    x -> norm1 -> spectral filter (+ its input, + a per-channel bias) -> + skip(x) -> norm2 -> MLP -> + x

Checkpoint contract (parameter names and shapes of makani/models/networks/afnonet_v2.py:52-314):
`patch_embed.proj`, `pos_embed [1, E, h*w]`, `blocks.{i}.{norm1, norm2, skip_layer, filter.{w1 [nb,bs,bs*f,2],
b1 [1,E,1,1], w2 [nb,bs*f,bs,2]}, mlp}`, `head` (1x1 convolution without bias).

Execution is laid out for B200: activations are NCHW tensors in channels-last memory (a token's channels are one
contiguous line, which is what the TMA tiles of the GEMM engine want), and a block is five fused launches groups:

  * instance norm: two streaming kernels (`ops/norm.py`);
  * spectral filter: the GEMM chain of `ops/afno.py` (both FFTs restricted to the kept modes, block-diagonal complex MLP
    with ReLU and soft shrinkage in the epilogues), which also adds its input in its last epilogue;
  * skip: the 1x1 convolution of the block input is a GEMM whose epilogue adds the filter output; the filter's bias `b1` is
    folded into that convolution's bias, so no elementwise pass is left;
  * MLP: two GEMMs with bias + GELU and bias + residual epilogues (`ops/conv.py`).

On CPU, or for dtypes / shapes the kernels do not take, each piece falls back to its plain torch formulation.
"""

from __future__ import annotations

from functools import partial

import torch
import torch.nn as nn

from ...ops import afno as afno_ops
from ...ops import conv as conv_ops
from ...ops import norm as norm_ops
from ..common.layers import MLP, DropPath, PatchEmbed


def _cl(x: torch.Tensor) -> torch.Tensor:
    """Channels-last memory for a 4-D NCHW-shaped activation (no copy when it already is)."""
    return x.contiguous(memory_format=torch.channels_last)


class AFNO2D(nn.Module):
    """Spectral token mixer.  `forward` returns filter(x) + x + b1 unless `fold_bias` asks the caller to add `b1`."""

    def __init__(self, hidden_size, num_blocks=8, sparsity_threshold=0.0, hard_thresholding_fraction=1, hidden_size_factor=1,
                 use_complex_kernels=False):
        super().__init__()
        if hidden_size % num_blocks != 0:
            raise ValueError(f"hidden_size {hidden_size} is not a multiple of num_blocks {num_blocks}")
        self.hidden_size, self.num_blocks = hidden_size, num_blocks
        self.block_size = hidden_size // num_blocks
        self.hidden_size_factor = hidden_size_factor
        self.sparsity_threshold = float(sparsity_threshold)
        self.hard_thresholding_fraction = hard_thresholding_fraction
        bs, hid, std = self.block_size, self.block_size * hidden_size_factor, 0.02
        self.w1 = nn.Parameter(std * torch.randn(num_blocks, bs, hid, 2))
        self.b1 = nn.Parameter(std * torch.randn(1, hidden_size, 1, 1))
        self.w2 = nn.Parameter(std * torch.randn(num_blocks, hid, bs, 2))

    def forward(self, x: torch.Tensor, fold_bias: bool = False) -> torch.Tensor:
        B, C, H, W = x.shape
        kx, ncols = afno_ops.mode_window_v2(H, W, self.hard_thresholding_fraction)
        tok = _cl(x).permute(0, 2, 3, 1)                       # [B, H, W, C] view of the channels-last storage
        hid = self.block_size * self.hidden_size_factor
        fn = afno_ops.afno_filter if afno_ops.fast_path_ok(tok, self.num_blocks, hid) else afno_ops.afno_filter_reference
        y = fn(tok, self.w1[..., 0], self.w1[..., 1], None, None, self.w2[..., 0], self.w2[..., 1], None, None,
               kx, ncols, self.sparsity_threshold, skip=tok)
        y = y.permute(0, 3, 1, 2)                               # back to an NCHW-shaped channels-last tensor
        return y if fold_bias else y + self.b1.to(y.dtype)


class _Norm(nn.Module):
    """Instance norm with affine parameters (fused kernels on the channels-last path) or layer norm over (h, w); either
    way the parameters are `weight` / `bias`, as in the checkpoints."""

    def __init__(self, kind: str, channels: int, hw):
        super().__init__()
        self.kind, self.eps, self.hw = kind, 1e-6, tuple(hw)
        if kind == "instance_norm":
            shape = (channels,)
        elif kind == "layer_norm":
            shape = self.hw
        else:
            raise NotImplementedError(f"normalization {kind} not implemented")
        self.weight = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape))

    def forward(self, x):
        if self.kind == "instance_norm":
            return norm_ops.instance_norm(x, self.weight, self.bias, self.eps, "none")
        return torch.nn.functional.layer_norm(x, self.hw, self.weight.to(x.dtype), self.bias.to(x.dtype), self.eps)


class Block(nn.Module):
    def __init__(self, h, w, dim, mlp_ratio=4.0, drop=0.0, drop_path=0.0, act_layer=nn.GELU, norm_kind="instance_norm",
                 num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1.0, use_complex_kernels=True,
                 skip_fno="linear", nested_skip_fno=True, checkpointing=False):
        super().__init__()
        self.norm1 = _Norm(norm_kind, dim, (h, w))
        self.norm2 = _Norm(norm_kind, dim, (h, w))
        self.filter = AFNO2D(dim, num_blocks, sparsity_threshold, hard_thresholding_fraction, use_complex_kernels=use_complex_kernels)
        self.skip_fno = skip_fno if skip_fno in ("linear", "identity") else None
        self.nested_skip_fno = nested_skip_fno
        if self.skip_fno == "linear":
            self.skip_layer = nn.Conv2d(dim, dim, 1, 1)
        elif self.skip_fno == "identity":
            self.skip_layer = nn.Identity()
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.mlp = MLP(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop_rate=drop,
                       checkpointing=2 if checkpointing else 0)

    def forward(self, x):
        residual = x
        if self.skip_fno == "linear":
            # filter output enters the skip convolution as its epilogue residual; b1 rides on the convolution's bias
            f = self.filter(self.norm1(x), fold_bias=True)
            bias = self.skip_layer.bias + self.filter.b1.reshape(-1)
            x = conv_ops.conv1x1(_cl(residual), self.skip_layer.weight, bias, resid=_cl(f))
        else:
            x = self.filter(self.norm1(x))
            if self.skip_fno == "identity":
                x = x + residual
        if self.skip_fno is not None and not self.nested_skip_fno:
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
        if len(self.patch_size) != 2:
            raise ValueError(f"patch_size needs two entries, got {patch_size}")
        if self.img_size[0] % self.patch_size[0] or self.img_size[1] % self.patch_size[1]:
            raise ValueError(f"patch size {self.patch_size} does not divide the image {self.img_size}")
        self.inp_chans, self.out_chans, self.embed_dim = inp_chans, out_chans, embed_dim
        self.h, self.w = self.img_size[0] // self.patch_size[0], self.img_size[1] // self.patch_size[1]
        self.patch_embed = PatchEmbed(img_size=self.img_size, patch_size=self.patch_size, in_chans=inp_chans, embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, embed_dim, self.h * self.w))
        self.pos_drop = nn.Dropout(p=drop_rate) if drop_rate > 0.0 else nn.Identity()
        rates = torch.linspace(0, drop_path_rate, num_layers).tolist()
        self.blocks = nn.ModuleList([
            Block(self.h, self.w, embed_dim, mlp_ratio=mlp_ratio, drop=drop_rate, drop_path=rates[i],
                  norm_kind=normalization_layer, num_blocks=num_blocks, sparsity_threshold=sparsity_threshold,
                  hard_thresholding_fraction=hard_thresholding_fraction, use_complex_kernels=use_complex_kernels,
                  skip_fno=skip_fno, nested_skip_fno=nested_skip_fno, checkpointing=checkpointing)
            for i in range(num_layers)])
        self.head = nn.Conv2d(embed_dim, out_chans * self.patch_size[0] * self.patch_size[1], 1, bias=False)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Conv2d)):
                nn.init.trunc_normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    @torch.jit.ignore
    def no_weight_decay(self):
        return {"pos_embed", "cls_token"}

    def forward_features(self, x):
        tokens = self.patch_embed(x)                                           # [B, E, h*w]
        tokens = self.pos_drop(tokens + self.pos_embed.to(tokens.dtype))
        x = _cl(tokens.reshape(tokens.shape[0], self.embed_dim, self.h, self.w))
        for blk in self.blocks:
            x = blk(x)
        return x

    def forward(self, x):
        feat = self.forward_features(x)
        y = conv_ops.conv1x1(feat, self.head.weight, None)                      # [B, out*p0*p1, h, w]
        B, (p0, p1) = y.shape[0], self.patch_size
        # un-patchify: channel index (p0, p1, c) of token (i, j) -> pixel (i*p0 + a, j*p1 + b) of channel c
        y = y.reshape(B, p0, p1, self.out_chans, self.h, self.w).permute(0, 3, 4, 1, 5, 2)
        return y.reshape(B, self.out_chans, self.h * p0, self.w * p1)
