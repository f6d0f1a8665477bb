"""Model-parallel layers: 2-D sharded pointwise matmuls (channel parallelism over the `fin` / `fout` groups),
encoder/decoder and MLP stacks built from them, tensor-parallel attention, and the spatially distributed 2-D
FFT pair.  Behavioural contract: makani/mpu/layers.py:37-642.

Channel parallelism: a weight [out, in] is stored as the block [out / |G_out|, in / |G_in|].  The input arrives
sharded over G_in; the local product is a partial sum that is all-reduced over G_in (forward) and whose data
gradient is all-reduced over G_out (backward).  Consecutive layers swap the roles of the two groups so
activations never need re-sharding.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..utils import comm
from .helpers import compute_split_shapes
from .mappings import (copy_to_parallel_region, gather_from_parallel_region, reduce_from_parallel_region,
                       scatter_to_parallel_region)
from .transpose import distributed_transpose_azimuth, distributed_transpose_polar


class DistributedRealFFT2(nn.Module):
    """rfft2 with truncation on [B, C, H_loc, W_loc] data sharded over ("h", "w")."""

    def __init__(self, nlat, nlon, lmax=None, mmax=None):
        super().__init__()
        self.comm_size_h, self.comm_size_w = comm.get_size("h"), comm.get_size("w")
        self.comm_rank_w = comm.get_rank("w")
        self.nlat, self.nlon = nlat, nlon
        self.lmax = min(lmax or nlat, nlat)
        self.mmax = min(mmax or nlon // 2 + 1, nlon // 2 + 1)
        self.lmax_high, self.lmax_low = math.ceil(self.lmax / 2), math.floor(self.lmax / 2)
        self.lat_shapes = compute_split_shapes(nlat, self.comm_size_h)
        self.lon_shapes = compute_split_shapes(nlon, self.comm_size_w)
        self.l_shapes = compute_split_shapes(self.lmax, self.comm_size_h)
        self.m_shapes = compute_split_shapes(self.mmax, self.comm_size_w)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.lon_shapes)
        x = torch.fft.rfft(x, n=self.nlon, dim=-1, norm="ortho")[..., : self.mmax]
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), compute_split_shapes(num_chans, self.comm_size_w))
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x, (1, -2), self.lat_shapes)
        x = torch.fft.fft(x, n=self.nlat, dim=-2, norm="ortho")
        parts = [x[..., : self.lmax_high, :]]
        if self.lmax_low > 0:
            parts.append(x[..., -self.lmax_low:, :])
        x = torch.cat(parts, dim=-2)
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), compute_split_shapes(num_chans, self.comm_size_h))
        return x


class DistributedInverseRealFFT2(nn.Module):
    def __init__(self, nlat, nlon, lmax=None, mmax=None):
        super().__init__()
        self.comm_size_h, self.comm_size_w = comm.get_size("h"), comm.get_size("w")
        self.nlat, self.nlon = nlat, nlon
        self.lmax = min(lmax or nlat, nlat)
        self.mmax = min(mmax or nlon // 2 + 1, nlon // 2 + 1)
        self.lmax_high, self.lmax_low = math.ceil(self.lmax / 2), math.floor(self.lmax / 2)
        self.lat_shapes = compute_split_shapes(nlat, self.comm_size_h)
        self.lon_shapes = compute_split_shapes(nlon, self.comm_size_w)
        self.l_shapes = compute_split_shapes(self.lmax, self.comm_size_h)
        self.m_shapes = compute_split_shapes(self.mmax, self.comm_size_w)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x, (1, -2), self.l_shapes)
        hi = F.pad(x[..., : self.lmax_high, :], (0, 0, 0, self.nlat - self.lmax))
        parts = [hi]
        if self.lmax_low > 0:
            parts.append(x[..., -self.lmax_low:, :])
        x = torch.cat(parts, dim=-2)
        x = torch.fft.ifft(x, n=self.nlat, dim=-2, norm="ortho")
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), compute_split_shapes(num_chans, self.comm_size_h))
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.m_shapes)
        x = torch.fft.irfft(x, n=self.nlon, dim=-1, norm="ortho")
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), compute_split_shapes(num_chans, self.comm_size_w))
        return x


class DistributedMatmul(nn.Module):
    """Pointwise linear map with the weight sharded [out over comm_out, in over comm_inp]."""

    def __init__(self, inp_dim, out_dim, input_format="nchw", comm_inp_name="fin", comm_out_name="fout", bias=True):
        super().__init__()
        self.comm_inp_name, self.comm_out_name = comm_inp_name, comm_out_name
        self.input_format = input_format
        inp_loc = compute_split_shapes(inp_dim, comm.get_size(comm_inp_name))[comm.get_rank(comm_inp_name)]
        out_loc = compute_split_shapes(out_dim, comm.get_size(comm_out_name))[comm.get_rank(comm_out_name)]
        if input_format == "nchw":
            self.weight = nn.Parameter(torch.ones(out_loc, inp_loc, 1, 1))
            self.weight.sharded_dims_mp = [comm_out_name, comm_inp_name, None, None]
            self.matmul_handle = F.conv2d
        elif input_format == "traditional":
            self.weight = nn.Parameter(torch.ones(out_loc, inp_loc))
            self.weight.sharded_dims_mp = [comm_out_name, comm_inp_name]
            self.matmul_handle = F.linear
        else:
            raise NotImplementedError(f"input format {input_format} not supported")
        self.weight.is_shared_mp = ["spatial"]
        if bias:
            if input_format == "nchw":
                self.bias = nn.Parameter(torch.zeros(1, out_loc, 1, 1))
                self.bias.sharded_dims_mp = [None, comm_out_name, None, None]
            else:
                self.bias = nn.Parameter(torch.zeros(out_loc))
                self.bias.sharded_dims_mp = [comm_out_name]
            self.bias.is_shared_mp = ["spatial", comm_inp_name]

    def forward(self, x):
        if self.input_format == "nchw":
            from ..ops import matmul_dist
            w2 = self.weight.reshape(self.weight.shape[0], self.weight.shape[1])
            if matmul_dist.supported(x, w2, self.comm_inp_name, self.comm_out_name):
                # tcgen05 GEMM whose epilogue delivers the partial products to the group (no NCCL on this path)
                return matmul_dist.fused_dist_matmul(x, w2, getattr(self, "bias", None), self.comm_inp_name, self.comm_out_name)
        elif self.input_format == "traditional" and x.dim() == 4 and x.is_contiguous():
            # token-major [B, h, w, C] is the channels-last memory layout of a [B, C, h, w] activation
            from ..ops import matmul_dist
            xv = x.permute(0, 3, 1, 2)
            if matmul_dist.supported(xv, self.weight, self.comm_inp_name, self.comm_out_name):
                y = matmul_dist.fused_dist_matmul(xv, self.weight, getattr(self, "bias", None), self.comm_inp_name,
                                                  self.comm_out_name)
                return y.permute(0, 2, 3, 1)
        x_cp = copy_to_parallel_region(x, self.comm_out_name)
        x_loc = self.matmul_handle(x_cp, self.weight.to(x_cp.dtype), bias=None)
        x_out = reduce_from_parallel_region(x_loc, self.comm_inp_name)
        if hasattr(self, "bias"):
            x_out = x_out + self.bias.to(x_out.dtype)
        return x_out


class DistributedPatchEmbed(nn.Module):
    """Patch embedding (strided convolution) whose output channels may be sharded over the `matmul` group; the input
    is gathered first when it arrives channel-sharded.  Interface of makani/mpu/layers.py:403-450 (no network of the
    reference uses it); the width must divide evenly over the spatial group."""

    def __init__(self, img_size=(224, 224), patch_size=(16, 16), in_chans=3, embed_dim=768, input_is_matmul_parallel=False,
                 output_is_matmul_parallel=True):
        super().__init__()
        self.input_parallel, self.output_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        msize, ssize = comm.get_size("matmul"), comm.get_size("spatial")
        assert (img_size[1] // patch_size[1]) % ssize == 0, "the spatial group size must divide the number of patches along W"
        self.img_size = (img_size[0], img_size[1] // ssize)
        self.patch_size = patch_size
        self.num_patches = ((img_size[1] // patch_size[1]) // ssize) * (img_size[0] // patch_size[0])
        if self.output_parallel:
            assert embed_dim % msize == 0, "embed_dim must be divisible by the matmul group size"
            out_local = embed_dim // msize
        else:
            out_local = embed_dim
        self.proj = nn.Conv2d(in_chans, out_local, kernel_size=patch_size, stride=patch_size)
        self.proj.weight.is_shared_mp = ["spatial"]
        self.proj.bias.is_shared_mp = ["spatial"]
        if self.output_parallel:
            self.proj.weight.sharded_dims_mp = ["matmul", None, None, None]
            self.proj.bias.sharded_dims_mp = ["matmul"]
        self.gather_shapes = compute_split_shapes(in_chans, msize)

    def forward(self, x):
        if self.input_parallel:
            x = gather_from_parallel_region(x, 1, self.gather_shapes, "matmul")
        if self.output_parallel:
            x = copy_to_parallel_region(x, "matmul")
        B, C, H, W = x.shape
        assert H == self.img_size[0] and W == self.img_size[1], f"input size ({H}x{W}) does not match the model ({self.img_size})"
        return self.proj(x).flatten(2)


class DistributedEncoderDecoder(nn.Module):
    """Channel-parallel pointwise encoder/decoder; the in/out group names alternate from layer to layer."""

    def __init__(self, num_layers, input_dim, output_dim, hidden_dim, act_layer, gain=1.0, input_format="nchw",
                 comm_inp_name="fin", comm_out_name="fout"):
        super().__init__()
        mods = []
        cur = input_dim
        cin, cout = comm_inp_name, comm_out_name
        for _ in range(num_layers):
            lin = DistributedMatmul(cur, hidden_dim, input_format, cin, cout, bias=True)
            nn.init.normal_(lin.weight, mean=0.0, std=math.sqrt(2.0 / cur))
            nn.init.constant_(lin.bias, 0.0)
            mods += [lin, act_layer()]
            cur = hidden_dim
            cin, cout = cout, cin
        out = DistributedMatmul(cur, output_dim, input_format, cin, cout, bias=False)
        nn.init.normal_(out.weight, mean=0.0, std=math.sqrt(gain / cur))
        mods.append(out)
        self.fwd = nn.Sequential(*mods)
        self.comm_inp_name, self.comm_out_name = comm_inp_name, cout

    def forward(self, x):
        return self.fwd(x)


class DistributedMLP(nn.Module):
    def __init__(self, in_features, hidden_features=None, out_features=None, output_bias=True, input_format="nchw",
                 comm_inp_name="fin", comm_hidden_name="fout", act_layer=nn.GELU, drop_rate=0.0, drop_type="iid",
                 checkpointing=0, gain=1.0, **kwargs):
        super().__init__()
        self.checkpointing = checkpointing
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.fc1 = DistributedMatmul(in_features, hidden_features, input_format, comm_inp_name, comm_hidden_name, bias=True)
        nn.init.normal_(self.fc1.weight, mean=0.0, std=math.sqrt(2.0 / in_features))
        nn.init.constant_(self.fc1.bias, 0.0)
        self.fc2 = DistributedMatmul(hidden_features, out_features, input_format, comm_hidden_name, comm_inp_name, bias=output_bias)
        nn.init.normal_(self.fc2.weight, mean=0.0, std=math.sqrt(gain / hidden_features))
        if hasattr(self.fc2, "bias"):
            nn.init.constant_(self.fc2.bias, 0.0)
        self.act = act_layer()
        if drop_rate > 0.0:
            self.drop = nn.Dropout(drop_rate) if drop_type == "iid" else nn.Dropout2d(drop_rate)
        else:
            self.drop = nn.Identity()

    def fwd(self, x):
        return self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))

    def forward(self, x):
        if self.checkpointing >= 2 and self.training:
            return checkpoint(self.fwd, x, use_reentrant=False)
        return self.fwd(x)


class DistributedAttention(nn.Module):
    """Multi-head self attention with heads split over `comm_hidden_name` (sequence stays whole)."""

    def __init__(self, dim, input_format="traditional", comm_inp_name="fin", comm_hidden_name="fout", num_heads=8,
                 qkv_bias=False, qk_norm=False, attn_drop_rate=0.0, proj_drop_rate=0.0, norm_layer=nn.LayerNorm):
        super().__init__()
        assert dim % num_heads == 0
        assert num_heads % comm.get_size(comm_hidden_name) == 0, "heads must divide over the hidden group"
        self.num_heads = num_heads
        self.num_heads_local = num_heads // comm.get_size(comm_hidden_name)
        self.head_dim = dim // num_heads
        self.comm_inp_name, self.comm_hidden_name = comm_inp_name, comm_hidden_name
        self.qkv = DistributedMatmul(dim, dim * 3, input_format, comm_inp_name, comm_hidden_name, bias=qkv_bias)
        self.proj = DistributedMatmul(dim, dim, input_format, comm_hidden_name, comm_inp_name, bias=False)
        nn.init.trunc_normal_(self.qkv.weight, std=0.02)
        nn.init.trunc_normal_(self.proj.weight, std=0.02)
        self.attn_drop_rate = attn_drop_rate
        self.proj_drop = nn.Dropout(proj_drop_rate)
        # per-head normalisation of queries and keys only on request (makani/mpu/layers.py:464,482-483); each rank holds
        # whole heads, so these small parameters are private to it
        self.q_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.k_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        for norm in (self.q_norm, self.k_norm):
            for prm in norm.parameters():
                prm.is_shared_mp = []

    def forward(self, x):
        B, N, C = x.shape
        # local rows of the qkv projection are ordered (q | k | v, local head, head_dim), as in makani/mpu/layers.py:507:
        # at one rank that is the serial layout, and a rank's rows are the q, k and v rows of its own heads
        qkv = self.qkv(x).reshape(B, N, 3, self.num_heads_local, self.head_dim).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        q, k = self.q_norm(q), self.k_norm(k)
        y = F.scaled_dot_product_attention(q, k, v, dropout_p=self.attn_drop_rate if self.training else 0.0)
        y = y.transpose(1, 2).reshape(B, N, self.num_heads_local * self.head_dim)
        return self.proj_drop(self.proj(y))


class DistributedAFNO2Dv2(nn.Module):
    """AFNO spectral filter (NCHW) with its channel blocks sharded over the `matmul` group: every rank runs the GEMM-chain
    filter of `ops/afno.py` on its own blocks; the input is scattered / the output gathered along the channels unless
    the caller already works on channel shards.  Interface and sharding tags of makani/mpu/layers.py:532-645
    (`w1 [nb_local, bs, bs*f, 2]`, `b1`, `w2`, `b2` complex pairs; shared over `spatial`, sharded over `matmul`)."""

    def __init__(self, hidden_size, num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1,
                 hidden_size_factor=1, input_is_matmul_parallel=False, output_is_matmul_parallel=False, use_complex_kernels=False):
        super().__init__()
        msize = comm.get_size("matmul")
        if hidden_size % num_blocks or num_blocks % msize:
            raise ValueError(f"hidden_size {hidden_size} / num_blocks {num_blocks} / matmul group {msize} do not divide")
        self.hidden_size, self.num_blocks = hidden_size, num_blocks
        self.num_blocks_local = num_blocks // msize
        self.block_size = hidden_size // num_blocks
        self.sparsity_threshold = float(sparsity_threshold)
        self.hard_thresholding_fraction = hard_thresholding_fraction
        self.hidden_size_factor = hidden_size_factor
        self.input_parallel, self.output_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        self.chan_shapes = compute_split_shapes(hidden_size, msize)
        bs, hid, nb, std = self.block_size, self.block_size * hidden_size_factor, self.num_blocks_local, 0.02
        self.w1 = nn.Parameter(std * torch.randn(nb, bs, hid, 2))
        self.b1 = nn.Parameter(std * torch.randn(nb, hid, 1, 1, 2))
        self.w2 = nn.Parameter(std * torch.randn(nb, hid, bs, 2))
        self.b2 = nn.Parameter(std * torch.randn(nb, bs, 1, 1, 2))
        for p in (self.w1, self.b1, self.w2, self.b2):
            p.is_shared_mp = ["spatial"]
            p.sharded_dims_mp = ["matmul"] + [None] * (p.dim() - 1)

    def forward(self, x):
        from ..ops import afno as afno_ops
        if not self.input_parallel:
            x = scatter_to_parallel_region(x, 1, "matmul")
        B, C, H, W = x.shape
        kx, ncols = afno_ops.mode_window_v2(H, W, self.hard_thresholding_fraction)
        tok = x.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1)
        hid = self.block_size * self.hidden_size_factor
        fn = afno_ops.afno_filter if afno_ops.fast_path_ok(tok, self.num_blocks_local, hid) else afno_ops.afno_filter_reference
        b1, b2 = self.b1[:, :, 0, 0], self.b2[:, :, 0, 0]
        y = fn(tok, self.w1[..., 0], self.w1[..., 1], b1[..., 0], b1[..., 1], self.w2[..., 0], self.w2[..., 1], b2[..., 0], b2[..., 1],
               kx, ncols, self.sparsity_threshold, skip=tok).permute(0, 3, 1, 2)
        if not self.output_parallel:
            y = gather_from_parallel_region(y, 1, self.chan_shapes, "matmul")
        return y
