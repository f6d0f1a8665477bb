"""Adaptive Fourier Neural Operator, version 1 (FourCastNet): token mixing by a block-diagonal complex MLP in
2-D Fourier space on NHWC patch tokens.

Architecture, parameter names and initialisation follow makani/models/networks/afnonet.py:26-268
(`patch_embed.proj`, `pos_embed`, `blocks.{i}.{norm1,filter.{w1,b1,w2,b2},norm2,mlp.{fc1,fc2}}`, `head`).
Beyond the reference, this network is channel parallel: with `fin * fout > 1` the MLP runs as a
`DistributedMLP` over ("fin", "fout") and the spectral blocks are sharded over the whole `matmul` group
(semantics of makani/mpu/layers.py:352-359,573-603); the reference's AFNO nets are serial only.
"""

from __future__ import annotations

from functools import partial

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import afno as afno_ops
from ...ops import linear as linear_ops
from ...parallel.helpers import compute_split_shapes
from ...parallel.layers import DistributedMLP
from ...parallel.mappings import gather_from_parallel_region, scatter_to_parallel_region
from ...utils import comm
from ...utils.img_utils import PeriodicPad2d
from ..common.layers import DropPath, PatchEmbed


class Mlp(nn.Module):
    def __init__(self, in_features, hidden_features=None, out_features=None, act_layer=nn.GELU, drop=0.0):
        super().__init__()
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.fc1 = nn.Linear(in_features, hidden_features)
        self.act = act_layer()
        self.fc2 = nn.Linear(hidden_features, out_features)
        self.drop = nn.Dropout(drop)
        self._fusable = act_layer is nn.GELU and drop == 0.0

    def forward(self, x):
        if self._fusable and linear_ops.fast_path_ok(x):
            return linear_ops.mlp2_lastdim(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias)
        return self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))


class AFNO2D(nn.Module):
    """rfft2 -> per-block complex (linear, ReLU, linear) -> softshrink -> irfft2, plus the input as skip
    (makani/models/networks/afnonet.py:45-112), evaluated as one chain of tensor-core GEMMs."""

    def __init__(self, hidden_size, num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1, hidden_size_factor=1):
        super().__init__()
        assert hidden_size % num_blocks == 0, f"hidden_size {hidden_size} should be divisble by num_blocks {num_blocks}"
        self.hidden_size, self.num_blocks = hidden_size, num_blocks
        self.sparsity_threshold = sparsity_threshold
        self.block_size = hidden_size // num_blocks
        self.hard_thresholding_fraction = hard_thresholding_fraction
        self.hidden_size_factor = hidden_size_factor
        self.scale = 0.02
        msize = comm.get_size("matmul")
        assert num_blocks % msize == 0, "spectral blocks must divide over the matmul group"
        self.num_blocks_local = num_blocks // msize
        self.chan_shapes = compute_split_shapes(hidden_size, msize)
        nb, bs, f = self.num_blocks_local, self.block_size, hidden_size_factor
        self.w1 = nn.Parameter(self.scale * torch.randn(2, nb, bs, bs * f))
        self.b1 = nn.Parameter(self.scale * torch.randn(2, nb, bs * f))
        self.w2 = nn.Parameter(self.scale * torch.randn(2, nb, bs * f, bs))
        self.b2 = nn.Parameter(self.scale * torch.randn(2, nb, bs))
        for p in (self.w1, self.b1, self.w2, self.b2):
            p.is_shared_mp = ["spatial"]
            p.sharded_dims_mp = [None, "matmul"] + [None] * (p.dim() - 2)

    def forward(self, x):
        """x [B, H, W, C_local-or-full] NHWC tokens.  The whole filter (both FFTs, the block MLP, the skip) is the GEMM
        chain of `ops/afno.py`; tensors it does not take (odd block sizes, fp32 on CUDA) go through its torch.fft twin."""
        msize = comm.get_size("matmul")
        if msize > 1:
            x = scatter_to_parallel_region(x, 3, "matmul")
        B, H, W, C = x.shape
        kx, ncols = afno_ops.mode_window_v1(H, W, self.hard_thresholding_fraction)
        hid = self.block_size * self.hidden_size_factor
        xc = x.contiguous()
        if xc.is_cuda and xc.dtype == torch.float32 and torch.is_autocast_enabled():
            xc = xc.to(torch.get_autocast_gpu_dtype())     # layer norm hands fp32 on under autocast; the GEMM chain runs in bf16
        fn = afno_ops.afno_filter if afno_ops.fast_path_ok(xc, self.num_blocks_local, hid) else afno_ops.afno_filter_reference
        y = fn(xc, self.w1[0], self.w1[1], self.b1[0], self.b1[1], self.w2[0], self.w2[1], self.b2[0], self.b2[1],
               kx, ncols, self.sparsity_threshold, skip=xc)
        if msize > 1:
            y = gather_from_parallel_region(y, 3, self.chan_shapes, "matmul")
        return y


class Block(nn.Module):
    def __init__(self, dim, mlp_ratio=4.0, drop=0.0, drop_path=0.0, act_layer=nn.GELU, norm_layer=nn.LayerNorm,
                 double_skip=True, num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1.0):
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.filter = AFNO2D(dim, num_blocks, sparsity_threshold, hard_thresholding_fraction)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = norm_layer(dim)
        hidden = int(dim * mlp_ratio)
        self.channel_parallel = comm.get_size("matmul") > 1
        if self.channel_parallel:
            self.mlp = DistributedMLP(in_features=dim, hidden_features=hidden, out_features=dim, act_layer=act_layer,
                                      drop_rate=drop, input_format="traditional", comm_inp_name="fin", comm_hidden_name="fout")
            self.fin_shapes = compute_split_shapes(dim, comm.get_size("fin"))
        else:
            self.mlp = Mlp(in_features=dim, hidden_features=hidden, act_layer=act_layer, drop=drop)
        self.double_skip = double_skip

    def forward(self, x):
        residual = x
        x = self.filter(self.norm1(x))
        if self.double_skip:
            x = x + residual
            residual = x
        x = self.norm2(x)
        if self.channel_parallel:
            # the MLP input is sharded over fin, its output is sharded the same way
            x = scatter_to_parallel_region(x, 3, "fin")
            x = self.mlp(x)
            x = gather_from_parallel_region(x, 3, self.fin_shapes, "fin")
        else:
            x = self.mlp(x)
        return self.drop_path(x) + residual


class PrecipNet(nn.Module):
    def __init__(self, backbone, patch_size=(16, 16), inp_chans=2, out_chans=2, **kwargs):
        super().__init__()
        self.patch_size, self.inp_chans, self.out_chans = patch_size, inp_chans, out_chans
        self.backbone = backbone
        self.ppad = PeriodicPad2d(1)
        self.conv = nn.Conv2d(out_chans, out_chans, kernel_size=3, stride=1, padding=0, bias=True)
        self.act = nn.ReLU()

    def forward(self, x):
        return self.act(self.conv(self.ppad(self.backbone(x))))


class AdaptiveFourierNeuralOperatorNet(nn.Module):
    def __init__(self, inp_shape=(720, 1440), patch_size=(16, 16), inp_chans=2, out_chans=2, embed_dim=768, num_layers=12,
                 mlp_ratio=4.0, drop_rate=0.0, drop_path_rate=0.0, num_blocks=16, sparsity_threshold=0.01,
                 hard_thresholding_fraction=1.0, **kwargs):
        super().__init__()
        self.img_size, self.patch_size = tuple(inp_shape), tuple(patch_size)
        self.inp_chans, self.out_chans, self.embed_dim = inp_chans, out_chans, embed_dim
        self.compute_dtype = None
        norm_layer = partial(nn.LayerNorm, eps=1e-6)
        self.patch_embed = PatchEmbed(img_size=self.img_size, patch_size=self.patch_size, in_chans=inp_chans, embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.pos_drop = nn.Dropout(p=drop_rate)
        dpr = [x.item() for x in torch.linspace(0, drop_path_rate, num_layers)]
        self.h = self.img_size[0] // self.patch_size[0]
        self.w = self.img_size[1] // self.patch_size[1]
        self.blocks = nn.ModuleList([
            Block(dim=embed_dim, mlp_ratio=mlp_ratio, drop=drop_rate, drop_path=dpr[i], norm_layer=norm_layer,
                  num_blocks=num_blocks, sparsity_threshold=sparsity_threshold,
                  hard_thresholding_fraction=hard_thresholding_fraction) for i in range(num_layers)])
        self.head = nn.Linear(embed_dim, out_chans * self.patch_size[0] * self.patch_size[1], bias=False)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    def _init_weights(self, m):
        if isinstance(m, nn.Linear):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def set_compute_dtype(self, dtype):
        self.compute_dtype = dtype

    @torch.jit.ignore
    def no_weight_decay(self):
        return {"pos_embed", "cls_token"}

    def forward_features(self, x):
        B = x.shape[0]
        x = self.patch_embed(x).transpose(1, 2)
        x = self.pos_drop(x + self.pos_embed.to(x.dtype))
        x = x.reshape(B, self.h, self.w, self.embed_dim)
        for blk in self.blocks:
            x = blk(x)
        return x

    def forward(self, x):
        if self.compute_dtype is not None:
            # parameters stay fp32; convolutions / linears run in the compute dtype whatever dtype the input has
            with torch.autocast(device_type=x.device.type, dtype=self.compute_dtype):
                return self._forward(x)
        return self._forward(x)

    def _forward(self, x):
        x = self.head(self.forward_features(x))
        b = x.shape[0]
        xv = x.view(b, self.h, self.w, self.patch_size[0], self.patch_size[1], -1)
        xvt = torch.permute(xv, (0, 5, 1, 3, 2, 4)).contiguous()
        return xvt.view(b, -1, self.h * self.patch_size[0], self.w * self.patch_size[1])
