"""EAGLE draft head (one decoder block over [target feature ; token embedding]) in plain PyTorch.

Same computation as the reference's `DraftHead` (reference: train/draft_model.py:24-64): x = merge(cat(feat, emb)),
pre-norm multi-head attention with half-split RoPE, SwiGLU, `fout` back to the feature width. It runs as PyTorch
bf16 modules exactly as the reference runs it (reference: spec_mega.py:39-44); the target model's verify step is
where this repository's kernels are. The state-dict keys equal the reference's, so its checkpoints load unchanged.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def rmsnorm(x, w, eps: float = 1e-5):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(positions, head_dim, base, device, dtype):
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(positions.float(), inv)
    emb = torch.cat([ang, ang], -1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def _rotate(x, cos, sin):
    a, b = x.chunk(2, dim=-1)
    return x * cos + torch.cat([-b, a], -1) * sin


class DraftHead(nn.Module):
    def __init__(self, dim: int, nh: int, inter: int, fuse: int = 1, rope_base: float = 1e7):
        super().__init__()
        self.nh, self.hd, self.rope_base = nh, dim // nh, rope_base
        self.dim, self.fuse, self.fdim = dim, fuse, fuse * dim
        self.merge = nn.Linear(self.fdim + dim, dim, bias=False)
        self.n1 = nn.Parameter(torch.ones(dim))
        self.n2 = nn.Parameter(torch.ones(dim))
        self.q = nn.Linear(dim, dim, bias=False)
        self.k = nn.Linear(dim, dim, bias=False)
        self.v = nn.Linear(dim, dim, bias=False)
        self.o = nn.Linear(dim, dim, bias=False)
        self.gate = nn.Linear(dim, inter, bias=False)
        self.up = nn.Linear(dim, inter, bias=False)
        self.down = nn.Linear(inter, dim, bias=False)
        self.fout = nn.Linear(dim, self.fdim, bias=False)

    def setup_cache(self, max_roll: int, device, dtype=torch.bfloat16):
        self.kc = torch.zeros(1, self.nh, max_roll, self.hd, device=device, dtype=dtype)
        self.vc = torch.zeros(1, self.nh, max_roll, self.hd, device=device, dtype=dtype)
        self.cmask = torch.tril(torch.ones(max_roll, max_roll, dtype=torch.bool, device=device))

    def forward(self, feat, emb, positions=None, input_pos=None):
        B, T, _ = feat.shape
        if positions is None:
            positions = torch.arange(T, device=feat.device)
        x = self.merge(torch.cat([feat, emb], -1))
        h = rmsnorm(x, self.n1)
        split = lambda t: t.view(B, T, self.nh, self.hd).transpose(1, 2)
        q, k, v = split(self.q(h)), split(self.k(h)), split(self.v(h))
        cos, sin = _rope(positions, self.hd, self.rope_base, feat.device, feat.dtype)
        q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        if input_pos is not None:
            self.kc[:, :, input_pos] = k
            self.vc[:, :, input_pos] = v
            att = F.scaled_dot_product_attention(q, self.kc, self.vc, attn_mask=self.cmask[input_pos])
        else:
            att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o(att.transpose(1, 2).reshape(B, T, self.dim))
        h = rmsnorm(x, self.n2)
        h = x + self.down(F.silu(self.gate(h)) * self.up(h))
        return self.fout(h)


def seeded_draft(dim: int, nh: int, inter: int, seed: int = 0, rope_base: float = 10000.0, device="cpu") -> DraftHead:
    """Draft head with seeded N(0, 0.02) weights (stand-in for a trained EAGLE checkpoint, which needs the training
    kit and datasets the reference used)."""
    g = torch.Generator().manual_seed(seed)
    m = DraftHead(dim, nh, inter, fuse=1, rope_base=rope_base)
    for p in m.parameters():
        if p.dim() == 2:
            p.data = torch.randn(p.shape, generator=g) * 0.02
    return m.to(torch.bfloat16).to(device).eval()
