"""The three callers of the attention module, restated in plain PyTorch with random weights.

The reference swaps its ``MonarchAttention`` into HuggingFace / diffusers models
(reference: experiments/vit/model.py:60-125, experiments/roberta/model.py:63-166,
experiments/dit/attention_processor.py:59-165).  Those wrappers need checkpoints,
datasets and library versions that are not available offline, so the architectures are
restated here - same shapes, same attention call site - with seeded random weights:
what is exercised is the op inside its callers, not model quality.

Every builder takes ``attn_factory``, a zero-argument callable returning the attention
module of one layer (``MonarchAttention(...)``, a dense-attention stand-in, or a test
double that calls the CPU oracle), and calls it exactly as the reference adapters do:
``attn_module(q, k, v)`` / ``attn_module(q, k, v, attention_mask)`` on (E, H, N, D) views of
the projection outputs, followed by ``permute(0, 2, 1, 3)`` back to token-major.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def _init(model: nn.Module, seed: int) -> nn.Module:
    """Seeded weights: matrices truncated-normal(0.02), biases uniform in +-0.02, norm scales left at one.
    Nothing is taken from the global generator, so two builds with one seed are identical."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() > 1:
                p.copy_(torch.empty_like(p, dtype=torch.float32).normal_(0.0, 0.02, generator=g).clamp_(-0.04, 0.04))
            elif name.endswith("bias"):
                p.copy_((torch.rand(p.shape, generator=g) - 0.5) * 0.04)
    return model


def _heads(x: torch.Tensor, n_heads: int) -> torch.Tensor:
    """(E, N, H*D) -> (E, H, N, D) view, as ``transpose_for_scores`` does (reference: experiments/vit/model.py:73-79)."""
    E, N, W = x.shape
    return x.view(E, N, n_heads, W // n_heads).permute(0, 2, 1, 3)


def _merge(ctx: torch.Tensor) -> torch.Tensor:
    """(E, H, N, D) -> (E, N, H*D) (reference: experiments/vit/model.py:99-101)."""
    E, H, N, D = ctx.shape
    return ctx.permute(0, 2, 1, 3).contiguous().view(E, N, H * D)


# ---------------------------------------------------------------------------------------------
# ViT-B/16: 224x224x3 input, 196 patches + CLS, 12 pre-LN layers, hidden 768, 12 heads of 64, MLP 3072
# ---------------------------------------------------------------------------------------------
class _ViTBlock(nn.Module):
    def __init__(self, attn_factory):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(768, eps=1e-12), nn.LayerNorm(768, eps=1e-12)
        self.q, self.k, self.v, self.o = (nn.Linear(768, 768) for _ in range(4))
        self.fc1, self.fc2 = nn.Linear(768, 3072), nn.Linear(3072, 768)
        self.attn = attn_factory()

    def forward(self, x):
        hdn = self.ln1(x)
        q, k, v = (_heads(p(hdn), 12) for p in (self.q, self.k, self.v))
        x = x + self.o(_merge(self.attn(q, k, v)))          # reference: experiments/vit/model.py:93-103
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class ViT(nn.Module):
    def __init__(self, attn_factory, depth=12):
        super().__init__()
        self.patch = nn.Conv2d(3, 768, 16, 16)
        self.cls = nn.Parameter(torch.zeros(1, 1, 768))
        self.pos = nn.Parameter(torch.zeros(1, 197, 768))
        self.blocks = nn.ModuleList(_ViTBlock(attn_factory) for _ in range(depth))
        self.ln = nn.LayerNorm(768, eps=1e-12)
        self.head = nn.Linear(768, 1000)

    def forward(self, img):
        x = self.patch(img).flatten(2).transpose(1, 2)
        x = torch.cat((self.cls.expand(x.shape[0], -1, -1), x), dim=1) + self.pos
        for b in self.blocks:
            x = b(x)
        return self.head(self.ln(x)[:, 0])


def build_vit_b16(attn_factory, dtype=torch.bfloat16, device="cuda", depth=12, seed=0):
    return _init(ViT(attn_factory, depth), seed).to(device=device, dtype=dtype).eval()


# ---------------------------------------------------------------------------------------------
# RoBERTa-base encoder: 12 post-LN layers, hidden 768, 12 heads of 64, FFN 3072, vocabulary 50265
# ---------------------------------------------------------------------------------------------
class _RobertaLayer(nn.Module):
    def __init__(self, attn_factory):
        super().__init__()
        self.q, self.k, self.v, self.o = (nn.Linear(768, 768) for _ in range(4))
        self.ln1, self.ln2 = nn.LayerNorm(768, eps=1e-5), nn.LayerNorm(768, eps=1e-5)
        self.fc1, self.fc2 = nn.Linear(768, 3072), nn.Linear(3072, 768)
        self.attn = attn_factory()

    def forward(self, x, attention_mask):
        q, k, v = (_heads(p(x), 12) for p in (self.q, self.k, self.v))
        # the raw (E, N) mask goes to the module unchanged (reference: experiments/roberta/model.py:104-106, :155-159)
        x = self.ln1(x + self.o(_merge(self.attn(q, k, v, attention_mask))))
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))


class RobertaEncoder(nn.Module):
    def __init__(self, attn_factory, depth=12, vocab=50265, max_pos=514):
        super().__init__()
        self.word = nn.Embedding(vocab, 768, padding_idx=1)
        self.position = nn.Embedding(max_pos, 768, padding_idx=1)
        self.token_type = nn.Embedding(1, 768)
        self.ln = nn.LayerNorm(768, eps=1e-5)
        self.layers = nn.ModuleList(_RobertaLayer(attn_factory) for _ in range(depth))

    def forward(self, input_ids, attention_mask=None):
        E, N = input_ids.shape
        if attention_mask is None:
            attention_mask = torch.ones(E, N, dtype=torch.long, device=input_ids.device)
        pos = (torch.cumsum(attention_mask, dim=1) * attention_mask + 1).long()   # RoBERTa: positions start at 2, pad = 1
        x = self.ln(self.word(input_ids) + self.position(pos) + self.token_type.weight[0])
        for layer in self.layers:
            x = layer(x, attention_mask)
        return x


def build_roberta_base(attn_factory, dtype=torch.bfloat16, device="cuda", depth=12, seed=0):
    return _init(RobertaEncoder(attn_factory, depth), seed).to(device=device, dtype=dtype).eval()


# ---------------------------------------------------------------------------------------------
# DiT-XL/2: 4x64x64 latents, patch 2 -> 1024 tokens, 28 layers, hidden 1152, 16 heads of 72, adaLN-Zero
# ---------------------------------------------------------------------------------------------
def _sincos(n: int, dim: int, device=None, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=device) / half)
    args = torch.arange(n, dtype=torch.float32, device=device)[:, None] * freqs[None]
    return torch.cat((torch.cos(args), torch.sin(args)), dim=-1)


class _DiTBlock(nn.Module):
    def __init__(self, attn_factory, hidden=1152, heads=16):
        super().__init__()
        self.heads = heads
        self.norm1 = nn.LayerNorm(hidden, elementwise_affine=False, eps=1e-6)
        self.norm2 = nn.LayerNorm(hidden, elementwise_affine=False, eps=1e-6)
        self.to_q, self.to_k, self.to_v, self.to_out = (nn.Linear(hidden, hidden) for _ in range(4))
        self.fc1, self.fc2 = nn.Linear(hidden, 4 * hidden), nn.Linear(4 * hidden, hidden)
        self.ada = nn.Linear(hidden, 6 * hidden)
        self.attn = attn_factory()

    def forward(self, x, c):
        sh1, sc1, g1, sh2, sc2, g2 = self.ada(F.silu(c)).unsqueeze(1).chunk(6, dim=-1)
        h = self.norm1(x) * (1 + sc1) + sh1
        # reference: experiments/dit/attention_processor.py:131-147 (view(E, -1, heads, head_dim).transpose(1, 2),
        # attn_module(q, k, v, attention_mask) with no mask for the class-conditional model)
        q, k, v = (_heads(p(h), self.heads) for p in (self.to_q, self.to_k, self.to_v))
        x = x + g1 * self.to_out(_merge(self.attn(q, k, v, None)))
        h = self.norm2(x) * (1 + sc2) + sh2
        return x + g2 * self.fc2(F.gelu(self.fc1(h), approximate="tanh"))


class DiT(nn.Module):
    def __init__(self, attn_factory, depth=28, hidden=1152, heads=16, in_ch=4, patch=2, grid=32, classes=1000):
        super().__init__()
        self.patch, self.grid, self.in_ch = patch, grid, in_ch
        self.embed = nn.Conv2d(in_ch, hidden, patch, patch)
        self.register_buffer("pos", _sincos(grid * grid, hidden).unsqueeze(0), persistent=False)
        self.t_mlp = nn.Sequential(nn.Linear(256, hidden), nn.SiLU(), nn.Linear(hidden, hidden))
        self.y_embed = nn.Embedding(classes + 1, hidden)
        self.blocks = nn.ModuleList(_DiTBlock(attn_factory, hidden, heads) for _ in range(depth))
        self.final_norm = nn.LayerNorm(hidden, elementwise_affine=False, eps=1e-6)
        self.final_ada = nn.Linear(hidden, 2 * hidden)
        self.final = nn.Linear(hidden, patch * patch * 2 * in_ch)

    def forward(self, latents, t, labels):
        E = latents.shape[0]
        x = self.embed(latents).flatten(2).transpose(1, 2) + self.pos.to(latents.dtype)
        freqs = torch.exp(-math.log(10000.0) * torch.arange(128, dtype=torch.float32, device=latents.device) / 128)
        args = t.float()[:, None] * freqs[None]   # sinusoidal timestep embedding, 256 wide
        c = self.t_mlp(torch.cat((torch.cos(args), torch.sin(args)), dim=-1).to(latents.dtype)) + self.y_embed(labels)
        for b in self.blocks:
            x = b(x, c)
        sh, sc = self.final_ada(F.silu(c)).unsqueeze(1).chunk(2, dim=-1)
        x = self.final(self.final_norm(x) * (1 + sc) + sh)
        p, gsz = self.patch, self.grid
        x = x.view(E, gsz, gsz, p, p, 2 * self.in_ch).permute(0, 5, 1, 3, 2, 4)
        return x.reshape(E, 2 * self.in_ch, gsz * p, gsz * p)


def build_dit_xl2(attn_factory, dtype=torch.bfloat16, device="cuda", depth=28, seed=0):
    return _init(DiT(attn_factory, depth), seed).to(device=device, dtype=dtype).eval()


class DenseAttention(nn.Module):
    """Dense softmax attention with the attention module's call signature (timing context)."""

    def forward(self, q, k, v, attention_mask=None):
        m = None
        if attention_mask is not None:
            m = attention_mask.to(torch.bool)[:, None, None, :]
        return F.scaled_dot_product_attention(q, k, v, attn_mask=m)
