"""Spherical Fourier Neural Operator (SFNO) and its planar FFT twin (FNO).

Architecture, constructor arguments, parameter names and initialisation follow
makani/models/networks/sfnonet.py:51-673: pointwise encoder -> `num_layers` blocks of
(spectral filter -> norm -> [inner skip] -> activation -> MLP -> norm -> drop path -> [outer skip]) -> pointwise
decoder (+ "big skip" from the input).  The first block analyses on the data grid and synthesises on the
internal (scale_factor-times coarser) grid, the last block goes back up.

B200 execution: with CUDA input and `bf16` compute (autocast bf16 active, bf16 input, or
`model.set_compute_dtype(torch.bfloat16)`) activations stay bf16 NCHW end to end and every layer is a
hand-written sm_100a kernel: tcgen05 GEMM chains for the spectral filter, the MLPs, encoder/decoder and
skips (bias/GELU/residual fused in the epilogues), fused instance-norm(+GELU) kernels.  Everything else (CPU,
fp32, exotic options) runs the same modules through plain torch ops.
"""

from __future__ import annotations

import math
from functools import partial

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ...ops import conv as conv_ops
from ...ops import norm as norm_ops
from ...parallel.helpers import compute_split_shapes
from ...parallel.layer_norm import DistributedInstanceNorm2d, DistributedLayerNorm
from ...parallel.layers import (DistributedEncoderDecoder, DistributedInverseRealFFT2, DistributedMLP,
                                DistributedRealFFT2)
from ...parallel.mappings import gather_from_parallel_region, scatter_to_parallel_region
from ...sht import DistributedInverseRealSHT, DistributedRealSHT, InverseRealSHT, RealSHT
from ...utils import comm
from ..common import (MLP, DropPath, EncoderDecoder, FactorizedSpectralConv, InverseRealFFT2, RealFFT2,
                      SpectralAttention, SpectralConv)


class InstanceNorm2d(nn.InstanceNorm2d):
    """nn.InstanceNorm2d whose CUDA bf16 path is the fused statistics+normalise(+GELU) kernel."""

    def forward(self, x, act: str = "none"):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4:
            return norm_ops.instance_norm(x, self.weight, self.bias, self.eps, act)
        y = super().forward(x)
        if act == "gelu":
            y = torch.nn.functional.gelu(y)
        return y


class SpectralFilterLayer(nn.Module):
    def __init__(self, forward_transform, inverse_transform, embed_dim, filter_type="linear", operator_type="diagonal",
                 hidden_size_factor=1, factorization=None, rank=1.0, separable=False, complex_activation="real",
                 spectral_layers=1, bias=False, drop_rate=0.0, gain=1.0):
        super().__init__()
        if filter_type == "non-linear":
            self.filter = SpectralAttention(forward_transform, inverse_transform, embed_dim, embed_dim,
                                            operator_type=operator_type, hidden_size_factor=hidden_size_factor,
                                            complex_activation=complex_activation, spectral_layers=spectral_layers,
                                            drop_rate=drop_rate, bias=bias, gain=gain)
        elif filter_type == "linear" and factorization is None:
            self.filter = SpectralConv(forward_transform, inverse_transform, embed_dim, embed_dim,
                                       operator_type=operator_type, separable=separable, bias=bias, gain=gain)
        elif filter_type == "linear":
            self.filter = FactorizedSpectralConv(forward_transform, inverse_transform, embed_dim, embed_dim,
                                                 operator_type=operator_type, rank=rank, factorization=factorization,
                                                 separable=separable, bias=bias, gain=gain)
        else:
            raise NotImplementedError(f"filter type {filter_type}")

    def forward(self, x):
        return self.filter(x)


class FourierNeuralOperatorBlock(nn.Module):
    def __init__(self, forward_transform, inverse_transform, embed_dim, filter_type="linear", operator_type="diagonal",
                 mlp_ratio=2.0, mlp_drop_rate=0.0, path_drop_rate=0.0, act_layer=nn.GELU,
                 norm_layer=(nn.Identity, nn.Identity), rank=1.0, factorization=None, separable=False,
                 inner_skip="linear", outer_skip=None, use_mlp=False, comm_feature_inp_name=None,
                 comm_feature_hidden_name=None, complex_activation="real", spectral_layers=1, bias=False,
                 final_activation=False, checkpointing=0):
        super().__init__()
        self.norm0 = norm_layer[0]()
        gain = 1.0 if act_layer == nn.Identity else 2.0
        if inner_skip == "linear":
            self.inner_skip = nn.Conv2d(embed_dim, embed_dim, 1, 1, bias=False)
            gain /= 2.0
            nn.init.normal_(self.inner_skip.weight, std=math.sqrt(gain / embed_dim))
            self.inner_skip.weight.is_shared_mp = ["spatial"]
        elif inner_skip == "identity":
            self.inner_skip = nn.Identity()
            gain /= 2.0
        elif inner_skip not in ("none", None):
            raise ValueError(f"Unknown skip connection type {inner_skip}")

        self.filter = SpectralFilterLayer(forward_transform, inverse_transform, embed_dim, filter_type, operator_type,
                                          hidden_size_factor=mlp_ratio, factorization=factorization, rank=rank,
                                          separable=separable, complex_activation=complex_activation,
                                          spectral_layers=spectral_layers, bias=bias, drop_rate=path_drop_rate, gain=gain)
        self.act_layer0 = act_layer()
        self._act0_is_gelu = act_layer is nn.GELU
        self.norm1 = norm_layer[1]()

        gain = 2.0 if (final_activation and act_layer != nn.Identity) else 1.0
        if outer_skip == "linear":
            self.outer_skip = nn.Conv2d(embed_dim, embed_dim, 1, 1, bias=False)
            gain /= 2.0
            nn.init.normal_(self.outer_skip.weight, std=math.sqrt(gain / embed_dim))
            self.outer_skip.weight.is_shared_mp = ["spatial"]
        elif outer_skip == "identity":
            self.outer_skip = nn.Identity()
            gain /= 2.0
        elif outer_skip not in ("none", None):
            raise ValueError(f"Unknown skip connection type {outer_skip}")

        if use_mlp:
            mlp_cls = DistributedMLP if comm.get_size("matmul") > 1 else MLP
            self.mlp = mlp_cls(in_features=embed_dim, hidden_features=int(embed_dim * mlp_ratio), act_layer=act_layer,
                               drop_rate=mlp_drop_rate, drop_type="features", comm_inp_name=comm_feature_inp_name,
                               comm_hidden_name=comm_feature_hidden_name, checkpointing=checkpointing, gain=gain)
        self.drop_path = DropPath(path_drop_rate) if path_drop_rate > 0.0 else nn.Identity()
        if final_activation:
            self.act_layer1 = act_layer()

    def forward(self, x):
        x, residual = self.filter(x)

        fuse_act = (isinstance(self.norm0, InstanceNorm2d) and self._act0_is_gelu and not hasattr(self, "inner_skip")
                    and x.is_cuda and x.dtype == torch.bfloat16)
        if fuse_act:
            x = self.norm0(x, act="gelu")
        else:
            x = self.norm0(x)
            if hasattr(self, "inner_skip"):
                x = x + self.inner_skip(residual)
            x = self.act_layer0(x)

        if hasattr(self, "mlp"):
            x = self.mlp(x)
        x = self.norm1(x)
        x = self.drop_path(x)

        if hasattr(self, "outer_skip"):
            if isinstance(self.outer_skip, nn.Conv2d) and x.is_cuda and conv_ops.fast_path_ok(x) and conv_ops.fast_path_ok(residual):
                # x + W r with the addition fused into the GEMM epilogue
                x = conv_ops.conv1x1(residual, self.outer_skip.weight, None, resid=x)
            else:
                x = x + self.outer_skip(residual)
        if hasattr(self, "act_layer1"):
            x = self.act_layer1(x)
        return x


class SphericalFourierNeuralOperatorNet(nn.Module):
    def __init__(self, spectral_transform="sht", model_grid_type="equiangular", sht_grid_type="legendre-gauss",
                 filter_type="linear", operator_type="dhconv", inp_shape=(721, 1440), out_shape=(721, 1440), scale_factor=8,
                 inp_chans=2, out_chans=2, embed_dim=32, num_layers=4, repeat_layers=1, use_mlp=True, mlp_ratio=2.0,
                 encoder_ratio=1, decoder_ratio=1, activation_function="gelu", encoder_layers=1, pos_embed="none",
                 pos_drop_rate=0.0, path_drop_rate=0.0, mlp_drop_rate=0.0, normalization_layer="instance_norm",
                 max_modes=None, hard_thresholding_fraction=1.0, big_skip=True, rank=1.0, factorization=None,
                 separable=False, complex_activation="real", spectral_layers=3, bias=False, checkpointing=0, **kwargs):
        super().__init__()
        self.inp_shape, self.out_shape = tuple(inp_shape), tuple(out_shape)
        self.inp_chans, self.out_chans = inp_chans, out_chans
        self.embed_dim, self.repeat_layers = embed_dim, repeat_layers
        self.big_skip, self.checkpointing = big_skip, checkpointing
        self.compute_dtype = None
        self.h = int(self.inp_shape[0] // scale_factor)
        self.w = int(self.inp_shape[1] // scale_factor)
        self._init_spectral_transforms(spectral_transform, model_grid_type, sht_grid_type, hard_thresholding_fraction, max_modes)

        acts = {"relu": nn.ReLU, "gelu": nn.GELU, "silu": nn.SiLU}
        if activation_function not in acts:
            raise ValueError(f"Unknown activation function {activation_function}")
        act = acts[activation_function]

        if comm.get_size("matmul") > 1:
            self.encoder = DistributedEncoderDecoder(num_layers=encoder_layers, input_dim=inp_chans, output_dim=embed_dim,
                                                     hidden_dim=int(encoder_ratio * embed_dim), act_layer=act,
                                                     input_format="nchw", comm_inp_name="fin", comm_out_name="fout")
            mlp_inp = self.encoder.comm_out_name
            mlp_hid = "fout" if mlp_inp == "fin" else "fin"
        else:
            self.encoder = EncoderDecoder(num_layers=encoder_layers, input_dim=inp_chans, output_dim=embed_dim,
                                          hidden_dim=int(encoder_ratio * embed_dim), act_layer=act, input_format="nchw")
            mlp_inp, mlp_hid = "fin", "fout"

        self.pos_drop = nn.Dropout(p=pos_drop_rate) if pos_drop_rate > 0.0 else nn.Identity()
        dpr = [x.item() for x in torch.linspace(0, path_drop_rate, num_layers)]

        if normalization_layer == "layer_norm":
            norm = partial(DistributedLayerNorm, normalized_shape=(embed_dim), elementwise_affine=True, eps=1e-6)
        elif normalization_layer == "instance_norm":
            if comm.get_size("spatial") > 1:
                norm = partial(DistributedInstanceNorm2d, num_features=embed_dim, eps=1e-6, affine=True)
            else:
                norm = partial(InstanceNorm2d, num_features=embed_dim, eps=1e-6, affine=True, track_running_stats=False)
        elif normalization_layer == "none":
            norm = nn.Identity
        else:
            raise NotImplementedError(f"normalization {normalization_layer} not implemented")

        self.blocks = nn.ModuleList()
        for i in range(num_layers):
            first, last = i == 0, i == num_layers - 1
            self.blocks.append(FourierNeuralOperatorBlock(
                self.trans_down if first else self.trans, self.itrans_up if last else self.itrans, embed_dim,
                filter_type=filter_type, operator_type=operator_type, mlp_ratio=mlp_ratio, mlp_drop_rate=mlp_drop_rate,
                path_drop_rate=dpr[i], act_layer=act, norm_layer=(norm, norm), inner_skip="none", outer_skip="linear",
                use_mlp=use_mlp, comm_feature_inp_name=mlp_inp, comm_feature_hidden_name=mlp_hid, rank=rank,
                factorization=factorization, separable=separable, complex_activation=complex_activation,
                spectral_layers=spectral_layers, bias=bias, checkpointing=checkpointing))

        if comm.get_size("matmul") > 1:
            self.decoder = DistributedEncoderDecoder(num_layers=encoder_layers, input_dim=embed_dim, output_dim=out_chans,
                                                     hidden_dim=int(decoder_ratio * embed_dim), act_layer=act,
                                                     gain=0.5 if big_skip else 1.0, comm_inp_name=mlp_inp,
                                                     comm_out_name=mlp_hid, input_format="nchw")
            self.gather_shapes = compute_split_shapes(out_chans, comm.get_size(self.decoder.comm_out_name))
        else:
            self.decoder = EncoderDecoder(num_layers=encoder_layers, input_dim=embed_dim, output_dim=out_chans,
                                          hidden_dim=int(decoder_ratio * embed_dim), act_layer=act,
                                          gain=0.5 if big_skip else 1.0, input_format="nchw")

        if big_skip:
            self.residual_transform = nn.Conv2d(inp_chans, out_chans, 1, bias=False)
            self.residual_transform.weight.is_shared_mp = ["spatial"]
            self.residual_transform.weight.sharded_dims_mp = [None, None, None, None]
            nn.init.normal_(self.residual_transform.weight, mean=0.0, std=math.sqrt(0.5 / inp_chans))

        if pos_embed == "direct":
            self.pos_embed = nn.Parameter(torch.zeros(1, embed_dim, self.inp_shape_loc[0], self.inp_shape_loc[1]))
            self.pos_embed.is_shared_mp = []
            self.pos_embed.sharded_dims_mp = [None, None, "h", "w"]
            self.pos_embed.type = "direct"
            nn.init.trunc_normal_(self.pos_embed, std=0.02)
        elif pos_embed == "frequency":
            if comm.get_size("spatial") > 1:
                lmax_loc = self.itrans_up.l_shapes[comm.get_rank("h")]
                mmax_loc = self.itrans_up.m_shapes[comm.get_rank("w")]
            else:
                lmax_loc, mmax_loc = self.itrans_up.lmax, self.itrans_up.mmax
            rc = nn.Parameter(torch.tril(torch.randn(1, embed_dim, lmax_loc, mmax_loc), diagonal=0))
            cc = nn.Parameter(torch.tril(torch.randn(1, embed_dim, lmax_loc, mmax_loc - 1), diagonal=-1))
            nn.init.trunc_normal_(rc, std=0.02)
            nn.init.trunc_normal_(cc, std=0.02)
            self.pos_embed = nn.ParameterList([rc, cc])
            self.pos_embed.type = "frequency"
            for p in self.pos_embed:
                p.is_shared_mp = []
                p.sharded_dims_mp = [None, None, "h", "w"]
        elif pos_embed not in ("none", "None", None):
            raise ValueError("Unknown position embedding type")

    # -----------------------------------------------------------------------------------------------
    def _init_spectral_transforms(self, spectral_transform, model_grid_type, sht_grid_type, hard_thresholding_fraction, max_modes):
        if max_modes is not None:
            modes_lat, modes_lon = max_modes
        else:
            modes_lat = int(self.h * hard_thresholding_fraction)
            modes_lon = int((self.w // 2 + 1) * hard_thresholding_fraction)
        dist_spatial = comm.get_size("spatial") > 1
        if spectral_transform == "sht":
            fwd = DistributedRealSHT if dist_spatial else RealSHT
            inv = DistributedInverseRealSHT if dist_spatial else InverseRealSHT
            self.trans_down = fwd(*self.inp_shape, lmax=modes_lat, mmax=modes_lon, grid=model_grid_type)
            self.itrans_up = inv(*self.out_shape, lmax=modes_lat, mmax=modes_lon, grid=model_grid_type)
            self.trans = fwd(self.h, self.w, lmax=modes_lat, mmax=modes_lon, grid=sht_grid_type)
            self.itrans = inv(self.h, self.w, lmax=modes_lat, mmax=modes_lon, grid=sht_grid_type)
        elif spectral_transform == "fft":
            fwd = DistributedRealFFT2 if dist_spatial else RealFFT2
            inv = DistributedInverseRealFFT2 if dist_spatial else InverseRealFFT2
            self.trans_down = fwd(*self.inp_shape, lmax=modes_lat, mmax=modes_lon)
            self.itrans_up = inv(*self.out_shape, lmax=modes_lat, mmax=modes_lon)
            self.trans = fwd(self.h, self.w, lmax=modes_lat, mmax=modes_lon)
            self.itrans = inv(self.h, self.w, lmax=modes_lat, mmax=modes_lon)
        else:
            raise ValueError("Unknown spectral transform")
        if dist_spatial:
            rh, rw = comm.get_rank("h"), comm.get_rank("w")
            self.inp_shape_loc = (self.trans_down.lat_shapes[rh], self.trans_down.lon_shapes[rw])
            self.out_shape_loc = (self.itrans_up.lat_shapes[rh], self.itrans_up.lon_shapes[rw])
            self.h_loc, self.w_loc = self.itrans.lat_shapes[rh], self.itrans.lon_shapes[rw]
        else:
            self.inp_shape_loc = (self.trans_down.nlat, self.trans_down.nlon)
            self.out_shape_loc = (self.itrans_up.nlat, self.itrans_up.nlon)
            self.h_loc, self.w_loc = self.itrans.nlat, self.itrans.nlon

    def set_compute_dtype(self, dtype) -> None:
        """Force the activation dtype of the forward pass (torch.bfloat16 selects the sm_100a kernels on CUDA)."""
        self.compute_dtype = dtype

    @torch.jit.ignore
    def no_weight_decay(self):
        return {"pos_embed", "cls_token"}

    def _forward_features(self, x):
        for _ in range(self.repeat_layers):
            for blk in self.blocks:
                if self.checkpointing >= 3 and self.training:
                    x = checkpoint(blk, x, use_reentrant=False)
                else:
                    x = blk(x)
        return x

    def _working_dtype(self, x):
        if self.compute_dtype is not None:
            return self.compute_dtype
        if x.is_cuda and torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.bfloat16:
            return torch.bfloat16
        return x.dtype

    def forward(self, x):
        wd = self._working_dtype(x)
        if x.dtype != wd:
            x = x.to(wd)
        if conv_ops.layout_of(x) is None:
            x = x.contiguous()

        if self.big_skip:
            if self.out_shape != self.inp_shape:
                with torch.autocast(device_type=x.device.type, enabled=False):
                    residual = self.itrans_up(self.trans_down(x.float()).contiguous()).to(x.dtype)
            else:
                residual = x

        if comm.get_size("fin") > 1:
            x = scatter_to_parallel_region(x, 1, "fin")

        if self.checkpointing >= 1 and self.training:
            x = checkpoint(self.encoder, x, use_reentrant=False)
        else:
            x = self.encoder(x)

        if hasattr(self, "pos_embed"):
            if self.pos_embed.type == "frequency":
                pe = torch.stack([self.pos_embed[0], nn.functional.pad(self.pos_embed[1], (1, 0), "constant", 0)], dim=-1)
                with torch.autocast(device_type=x.device.type, enabled=False):
                    pe = self.itrans_up(torch.view_as_complex(pe.float().contiguous()))
            else:
                pe = self.pos_embed
            x = x + pe.to(x.dtype)
        x = self.pos_drop(x)

        x = self._forward_features(x)

        if self.checkpointing >= 1 and self.training:
            x = checkpoint(self.decoder, x, use_reentrant=False)
        else:
            x = self.decoder(x)
        if hasattr(self.decoder, "comm_out_name") and comm.get_size(self.decoder.comm_out_name) > 1:
            x = gather_from_parallel_region(x, 1, self.gather_shapes, self.decoder.comm_out_name)

        if self.big_skip:
            rt = self.residual_transform
            if x.is_cuda and conv_ops.fast_path_ok(x) and conv_ops.fast_path_ok(residual):
                x = conv_ops.conv1x1(residual, rt.weight, None, resid=x)
            else:
                x = x + rt(residual)
        return x


class FourierNeuralOperatorNet(SphericalFourierNeuralOperatorNet):
    """Planar FNO: the same network with 2-D real FFTs as the spectral transform."""

    def __init__(self, *args, **kwargs):
        kwargs["spectral_transform"] = "fft"
        super().__init__(*args, **kwargs)


# names under which the reference exports these through modulus (makani/models/networks/sfnonet.py:652-673)
SFNO = SphericalFourierNeuralOperatorNet
FNO = FourierNeuralOperatorNet
