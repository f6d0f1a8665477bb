"""Vision transformer on lat/lon patch tokens.

Checkpoint contract (names and shapes of makani/models/networks/vit.py:29-231): `patch_embed.proj`,
`pos_embed [1, tokens, E]`, `blocks.{i}.{norm1, norm2, attn.{qkv, proj, q_norm, k_norm}, mlp.fwd.{0,3}}`, `norm`, `head`
(linear without bias); with `fin * fout > 1` the attention heads and the MLP hidden features are split over the
channel-parallel groups (makani/mpu/layers.py:352-359,453-529).

Execution: tokens stay in one [B, tokens, E] bf16 matrix.  Every projection (qkv, attention output, both MLP layers with
bias + GELU / bias epilogues, head) is a GEMM of the in-tree tensor-core engine (`ops/linear.py`); the softmax
attention itself is `scaled_dot_product_attention` (a library kernel: attention is not among this framework's own
kernels).  Layer norms are torch's.  On CPU / fp32 every piece is the plain torch op.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import linear as linear_ops
from ...parallel.layers import DistributedAttention, DistributedMLP
from ...utils import comm
from ..common.layers import MLP, DropPath, PatchEmbed


class _Proj(nn.Linear):
    """nn.Linear whose forward runs on the GEMM engine when the tokens qualify (bf16, CUDA, features % 8 == 0)."""

    def forward(self, x):
        return linear_ops.linear_lastdim(x, self.weight, self.bias)


class Attention(nn.Module):
    """Multi-head self attention over all tokens; q / k may be layer-normalised per head."""

    def __init__(self, dim, input_format="traditional", num_heads=8, qkv_bias=False, qk_norm=False, attn_drop_rate=0.0,
                 proj_drop_rate=0.0, norm_layer=nn.LayerNorm):
        super().__init__()
        if dim % num_heads:
            raise ValueError(f"dim {dim} is not a multiple of num_heads {num_heads}")
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.qkv = _Proj(dim, 3 * dim, bias=qkv_bias)
        self.proj = _Proj(dim, dim)
        self.q_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.k_norm = norm_layer(self.head_dim) if qk_norm else nn.Identity()
        self.attn_drop_rate = attn_drop_rate
        self.proj_drop = nn.Dropout(proj_drop_rate) if proj_drop_rate > 0 else nn.Identity()

    def forward(self, x):
        B, N, C = x.shape
        # [B, N, (3, heads, head_dim)] -> three [B, heads, N, head_dim] views, no copies before the attention kernel
        q, k, v = self.qkv(x).view(B, N, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4).unbind(0)
        ctx = F.scaled_dot_product_attention(self.q_norm(q), self.k_norm(k), v,
                                             dropout_p=self.attn_drop_rate if self.training else 0.0)
        return self.proj_drop(self.proj(ctx.transpose(1, 2).reshape(B, N, C)))


class Block(nn.Module):
    """x + attn(norm1(x)), then z = norm2(.), z + mlp(z) (the second residual starts after the norm, as upstream)."""

    def __init__(self, dim, num_heads, mlp_ratio=4.0, qkv_bias=False, mlp_drop_rate=0.0, attn_drop_rate=0.0,
                 path_drop_rate=0.0, act_layer=nn.GELU, norm_layer=nn.LayerNorm, comm_inp_name="fin", comm_hidden_name="fout"):
        super().__init__()
        hidden = int(dim * mlp_ratio)
        self.norm1, self.norm2 = norm_layer(dim), norm_layer(dim)
        if comm.get_size(comm_inp_name) * comm.get_size(comm_hidden_name) > 1:
            self.attn = DistributedAttention(dim, input_format="traditional", comm_inp_name=comm_inp_name,
                                             comm_hidden_name=comm_hidden_name, num_heads=num_heads, qkv_bias=qkv_bias,
                                             attn_drop_rate=attn_drop_rate, proj_drop_rate=mlp_drop_rate, norm_layer=None)
            self.mlp = DistributedMLP(in_features=dim, hidden_features=hidden, out_features=dim, act_layer=act_layer,
                                      drop_rate=mlp_drop_rate, input_format="traditional", comm_inp_name=comm_inp_name,
                                      comm_hidden_name=comm_hidden_name)
        else:
            self.attn = Attention(dim, num_heads=num_heads, qkv_bias=qkv_bias, attn_drop_rate=attn_drop_rate,
                                  proj_drop_rate=mlp_drop_rate, norm_layer=norm_layer)
            self.mlp = MLP(in_features=dim, hidden_features=hidden, out_features=dim, act_layer=act_layer,
                           drop_rate=mlp_drop_rate, input_format="traditional")      # fused token MLP (ops/linear.py)
        self.drop_path = DropPath(path_drop_rate) if path_drop_rate > 0.0 else nn.Identity()

    def forward(self, x):
        x = x + self.drop_path(self.attn(self.norm1(x)))
        z = self.norm2(x)
        return z + self.drop_path(self.mlp(z))


class VisionTransformer(nn.Module):
    def __init__(self, inp_shape=(224, 224), patch_size=(16, 16), inp_chans=3, out_chans=3, embed_dim=768, depth=12,
                 num_heads=12, mlp_ratio=4.0, qkv_bias=True, mlp_drop_rate=0.0, attn_drop_rate=0.0, path_drop_rate=0.0,
                 norm_layer="layer_norm", comm_inp_name="fin", comm_hidden_name="fout", **kwargs):
        super().__init__()
        if norm_layer != "layer_norm":
            raise NotImplementedError(f"normalization layer type {norm_layer} not implemented for ViT")
        self.img_size, self.patch_size = tuple(inp_shape), tuple(patch_size)
        self.embed_dim = self.num_features = embed_dim
        self.out_ch = out_chans
        self.comm_inp_name, self.comm_hidden_name = comm_inp_name, comm_hidden_name
        self.patch_embed = PatchEmbed(img_size=self.img_size, patch_size=self.patch_size, in_chans=inp_chans, embed_dim=embed_dim)
        self.grid = tuple(self.patch_embed.red_img_size)                       # tokens along latitude / longitude
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.pos_embed.is_shared_mp = []
        self.pos_drop = nn.Dropout(p=path_drop_rate)
        rates = torch.linspace(0, path_drop_rate, depth).tolist()
        self.blocks = nn.ModuleList([
            Block(embed_dim, num_heads, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, mlp_drop_rate=mlp_drop_rate,
                  attn_drop_rate=attn_drop_rate, path_drop_rate=rates[i], norm_layer=nn.LayerNorm,
                  comm_inp_name=comm_inp_name, comm_hidden_name=comm_hidden_name) for i in range(depth)])
        self.norm = nn.LayerNorm(embed_dim)
        self.out_size = out_chans * self.patch_size[0] * self.patch_size[1]
        self.head = _Proj(embed_dim, self.out_size, bias=False)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.LayerNorm):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)

    def prepare_tokens(self, x):
        tokens = self.patch_embed(x).transpose(1, 2)                            # [B, tokens, E]
        return self.pos_drop(tokens + self.pos_embed.to(tokens.dtype))

    def forward_head(self, tokens):
        B = tokens.shape[0]
        (h, w), (p, q) = self.grid, self.patch_size
        y = self.head(tokens)                                                   # [B, h*w, p*q*out]
        # token (i, j), feature (a, b, c) -> pixel (i*p + a, j*q + b) of channel c
        y = y.view(B, h, w, p, q, self.out_ch).permute(0, 5, 1, 3, 2, 4)
        return y.reshape(B, self.out_ch, h * p, w * q)

    def forward(self, x):
        tokens = self.prepare_tokens(x)
        for blk in self.blocks:
            tokens = blk(tokens)
        return self.forward_head(self.norm(tokens))
