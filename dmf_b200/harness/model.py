"""DMFT (Decoupled MeanFlow Transformer) with the reference's module and parameter
names, so that state dicts are interchangeable with models/dmft.py.

Structure (models/dmft.py:27-151, models/layers.py): patch embedding + fixed 2-D
sin-cos positions; ``dmf_depth`` encoder DiT blocks conditioned on (t, y), the
remaining decoder blocks and the final layer conditioned on (r, y); optional
log-variance head.  Attention goes through ``attn_op`` with the reference's
selector strings: 'fa2' / 'fa3' -> dmf_b200.flash_attn_func, 'base' -> naive
softmax attention, 'torch_sdpa' -> F.scaled_dot_product_attention.
"""

from __future__ import annotations

import math
from functools import partial

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..flash_attn_jvp import flash_attn_func, flash_attn_qkvpacked_func
from .. import adaln
from ..rms_norm import rms_norm


def attn_op(q, k, v, op: str = "base"):
    """Selector of models/layers.py:86-115; q, k, v and the result are (B, L, H, D)."""
    if op in ("fa2", "fa3"):
        return flash_attn_func(q, k, v)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if op == "torch_sdpa":
        x = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=False)
    elif op == "base":
        attn = (q * q.shape[-1] ** -0.5) @ k.transpose(-2, -1)
        x = attn.softmax(dim=-1) @ v
    else:
        raise ValueError(f"unknown attention op {op!r}")
    return x.transpose(1, 2)


class RMSNorm(nn.Module):
    """models/layers.py:33-42.  With ``fused`` the per-head norm of a 16-bit (B, L, H, D) CUDA tensor runs as
    the single-pass kernel of dmf_b200.rms_norm (tangent included under forward-mode AD); anything else takes
    the reference's elementwise form below."""

    def __init__(self, dim: int, eps: float = 1e-6, fused: bool = False):
        super().__init__()
        self.eps = eps
        self.fused = fused
        self.scale = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        if (self.fused and x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16)
                and x.shape[-1] % 8 == 0 and x.shape[-1] <= 128):
            return rms_norm(x, self.scale, self.eps)
        norm_x = torch.rsqrt(x.pow(2).mean(-1, keepdim=True, dtype=torch.float32) + self.eps)
        return x * norm_x.to(dtype=x.dtype) * self.scale.to(dtype=x.dtype)


def timestep_embedding(t, dim: int, max_period: int = 10000):
    """models/layers.py:46-55: [cos | sin] of t * geometric frequencies."""
    half = dim // 2
    # built on t's device (the reference builds it on the host and copies, models/layers.py:50-51: a host-to-device
    # copy per call, which also cannot be captured in a CUDA graph)
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[..., None].float() * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb


class TimestepEmbedder(nn.Module):
    def __init__(self, hidden_size: int, emb_size: int = 256):
        super().__init__()
        self.emb_size = emb_size
        self.mlp = nn.Sequential(nn.Linear(emb_size, hidden_size), nn.SiLU(), nn.Linear(hidden_size, hidden_size))

    def forward(self, t):
        return self.mlp(timestep_embedding(t, self.emb_size).to(t.dtype))


class LabelEmbedder(nn.Module):
    def __init__(self, num_classes: int, hidden_size: int, use_cfg_embedding: bool = True):
        super().__init__()
        self.embedding_table = nn.Embedding(num_classes + int(use_cfg_embedding), hidden_size)

    def forward(self, labels):
        return self.embedding_table(labels)


class PatchEmbed(nn.Module):
    """The part of timm's PatchEmbed the model uses (models/dmft.py:54-60, 91-93): a strided
    convolution ``proj`` and ``num_patches``; output (B, L, C)."""

    def __init__(self, img_size: int, patch_size: int, in_chans: int, embed_dim: int, bias: bool = True):
        super().__init__()
        self.num_patches = (img_size // patch_size) ** 2
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size, bias=bias)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class Attention(nn.Module):
    """models/layers.py:119-154: packed qkv projection, optional per-head RMSNorm of q and k,
    attention on (B, L, H, D) views of the packed buffer, output projection."""

    def __init__(self, dim: int, num_heads: int, qkv_bias: bool = False, qk_norm: bool = False,
                 proj_bias: bool = True, attn_func: str = "torch_sdpa"):
        super().__init__()
        assert dim % num_heads == 0
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        fused = attn_func in ("fa2", "fa3")   # the B200 ops travel together
        self.q_norm = RMSNorm(self.head_dim, fused=fused) if qk_norm else nn.Identity()
        self.k_norm = RMSNorm(self.head_dim, fused=fused) if qk_norm else nn.Identity()
        self.proj = nn.Linear(dim, dim, bias=proj_bias)
        self.attn = partial(attn_op, op=attn_func)
        self.packed = fused and not qk_norm

    def forward(self, x):
        B, L, C = x.shape
        if self.packed and x.is_cuda:
            # same computation on the packed projection: its gradient is written packed, not copied together
            qkv = self.qkv(x).reshape(B, L, 3, self.num_heads, self.head_dim)
            return self.proj(flash_attn_qkvpacked_func(qkv).reshape(B, L, C))
        q, k, v = self.qkv(x).reshape(B, L, 3, self.num_heads, self.head_dim).permute(2, 0, 1, 3, 4).unbind(0)
        q, k = self.q_norm(q), self.k_norm(k)
        return self.proj(self.attn(q, k, v).reshape(B, L, C))


class Mlp(nn.Module):
    def __init__(self, in_features: int, hidden_features: int):
        super().__init__()
        self.fc1 = nn.Linear(in_features, hidden_features)
        self.act = nn.GELU(approximate="tanh")
        self.fc2 = nn.Linear(hidden_features, in_features)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


def modulate(x, shift, scale):
    return x * (1 + scale) + shift


class DiTBlock(nn.Module):
    """adaLN-Zero block, models/layers.py:170-201."""

    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0, **block_kwargs):
        super().__init__()
        self.norm1 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.attn = Attention(hidden_size, num_heads=num_heads, qkv_bias=True,
                              qk_norm=block_kwargs.get("qk_norm", False),
                              attn_func=block_kwargs.get("attn_func", "base"))
        self.norm2 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.mlp = Mlp(hidden_size, int(hidden_size * mlp_ratio))
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 6 * hidden_size))
        self.fused = block_kwargs.get("attn_func", "base") in ("fa2", "fa3")   # the B200 ops travel together

    def forward(self, x, c):
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = self.adaLN_modulation(c).chunk(6, dim=-1)
        if self.fused and adaln.usable(x):
            # one kernel each (primal + tangent under forward-mode AD) instead of the elementwise forms below
            x = adaln.gate_residual(x, g_a, self.attn(adaln.ln_modulate(x, sh_a, sc_a, self.norm1.eps)))
            return adaln.gate_residual(x, g_m, self.mlp(adaln.ln_modulate(x, sh_m, sc_m, self.norm2.eps)))
        x = x + g_a * self.attn(modulate(self.norm1(x), sh_a, sc_a))
        x = x + g_m * self.mlp(modulate(self.norm2(x), sh_m, sc_m))
        return x


class FinalLayer(nn.Module):
    def __init__(self, hidden_size: int, patch_size: int, out_channels: int):
        super().__init__()
        self.norm_final = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.linear = nn.Linear(hidden_size, patch_size * patch_size * out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size))
        self.fused = False   # set by DMFT when the blocks use the B200 ops

    def forward(self, x, c):
        shift, scale = self.adaLN_modulation(c).chunk(2, dim=-1)
        if self.fused and adaln.usable(x):
            return self.linear(adaln.ln_modulate(x, shift, scale, self.norm_final.eps))
        return self.linear(modulate(self.norm_final(x), shift, scale))


def sincos_pos_embed_2d(embed_dim: int, grid_size: int) -> np.ndarray:
    """models/layers.py:224-271: [sin | cos] of the w coordinate in the first half of the
    channels, of the h coordinate in the second half (the meshgrid puts w first)."""
    def one_dim(dim, pos):
        omega = 1.0 / 10000 ** (np.arange(dim // 2, dtype=np.float64) / (dim / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)

    coords = np.arange(grid_size, dtype=np.float32)
    gw, gh = np.meshgrid(coords, coords)  # gw varies along the fast axis
    return np.concatenate([one_dim(embed_dim // 2, gw), one_dim(embed_dim // 2, gh)], axis=1)


class DMFT(nn.Module):
    def __init__(self, input_size: int = 32, patch_size: int = 2, in_channels: int = 4, hidden_size: int = 1152,
                 depth: int = 28, num_heads: int = 16, mlp_ratio: float = 4.0, use_cfg_embedding: bool = True,
                 num_classes: int = 1000, dmf_depth: int = 8, use_logvar: bool = False, **block_kwargs):
        super().__init__()
        self.input_size, self.patch_size = input_size, patch_size
        self.in_channels = self.out_channels = in_channels
        self.num_heads, self.num_classes = num_heads, num_classes
        self.dmf_depth, self.use_logvar = dmf_depth, use_logvar
        self.x_embedder = PatchEmbed(input_size, patch_size, in_channels, hidden_size, bias=True)
        self.t_embedder = TimestepEmbedder(hidden_size)
        self.y_embedder = LabelEmbedder(num_classes, hidden_size, use_cfg_embedding)
        self.num_patches = self.x_embedder.num_patches
        self.pos_embed = nn.Parameter(torch.zeros(1, self.num_patches, hidden_size), requires_grad=False)
        self.blocks = nn.ModuleList([DiTBlock(hidden_size, num_heads, mlp_ratio=mlp_ratio, **block_kwargs)
                                     for _ in range(depth)])
        self.final_layer = FinalLayer(hidden_size, patch_size, self.out_channels)
        self.final_layer.fused = block_kwargs.get("attn_func", "base") in ("fa2", "fa3")
        if use_logvar:
            self.logvar_linear = nn.Linear(256, 1)
        self.initialize_weights()

    def initialize_weights(self, zero_init: bool = True):
        """models/dmft.py:74-115.  ``zero_init=False`` replaces the zero initialisation of the
        adaLN / output layers by N(0, 0.02): with literal zeros every attention output is
        multiplied by a zero gate, so model-level parity tests could not see an attention bug."""
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)
        grid = int(self.num_patches ** 0.5)
        self.pos_embed.data.copy_(torch.from_numpy(sincos_pos_embed_2d(self.pos_embed.shape[-1], grid)).float()[None])
        w = self.x_embedder.proj.weight.data
        nn.init.xavier_uniform_(w.view(w.shape[0], -1))
        nn.init.constant_(self.x_embedder.proj.bias, 0)
        nn.init.normal_(self.y_embedder.embedding_table.weight, std=0.02)
        nn.init.normal_(self.t_embedder.mlp[0].weight, std=0.02)
        nn.init.normal_(self.t_embedder.mlp[2].weight, std=0.02)
        last = [b.adaLN_modulation[-1] for b in self.blocks] + [self.final_layer.adaLN_modulation[-1],
                                                                  self.final_layer.linear]
        if self.use_logvar:
            last.append(self.logvar_linear)
        for lin in last:
            if zero_init:
                nn.init.constant_(lin.weight, 0)
            else:
                nn.init.normal_(lin.weight, std=0.02)
            nn.init.constant_(lin.bias, 0)

    def unpatchify(self, x):
        c, p = self.out_channels, self.patch_size
        h = w = int(x.shape[1] ** 0.5)
        x = x.reshape(x.shape[0], h, w, p, p, c)
        return torch.einsum("nhwpqc->nchpwq", x).reshape(x.shape[0], c, h * p, w * p)

    def forward(self, x, t, r, y, return_logvar: bool = False):
        t, r = t.reshape(-1), r.reshape(-1)
        x = self.x_embedder(x) + self.pos_embed
        B, L, D = x.shape
        y_embed = self.y_embedder(y).reshape(B, -1, D)
        c_t = self.t_embedder(t).reshape(B, -1, D) + y_embed
        for block in self.blocks[:self.dmf_depth]:
            x = block(x, c_t)
        c_r = self.t_embedder(r).reshape(B, -1, D) + y_embed
        for block in self.blocks[self.dmf_depth:]:
            x = block(x, c_r)
        x = self.unpatchify(self.final_layer(x, c_r))
        if return_logvar:
            emb = torch.cat([timestep_embedding(t, 128), timestep_embedding(r, 128)], dim=1)
            logvar = self.logvar_linear(emb).view(-1, *[1] * (x.ndim - 1))
            return x, logvar
        return x


DMFT_CONFIGS = {
    "DMFT-XL/2": dict(depth=28, hidden_size=1152, patch_size=2, num_heads=16),
    "DMFT-L/2": dict(depth=24, hidden_size=1024, patch_size=2, num_heads=16),
    "DMFT-B/2": dict(depth=12, hidden_size=768, patch_size=2, num_heads=12),
    "DMFT-S/2": dict(depth=12, hidden_size=384, patch_size=2, num_heads=6),
}


def build_dmft(name: str = "DMFT-XL/2", **kwargs) -> DMFT:
    return DMFT(**DMFT_CONFIGS[name], **kwargs)
