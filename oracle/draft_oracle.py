"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference's EAGLE draft head and its token head.

Follows the reference line by line (paths inside the reference project):
  rmsnorm            train/draft_model.py:9-10
  rope / rotate      train/draft_model.py:12-22     cos / sin tables cast to the activation dtype (bf16)
  DraftHead.forward  train/draft_model.py:45-64     both modes: plain causal (input_pos None) and fixed-slot cache
  head_tok / tlog    spec_mega.py:43-44, spec_tree.py:38
  sample             engine/generate.py:37-55       softmax(logits / T) with top-k masking (the distribution only)

Arithmetic: fp32 with a bf16 rounding wherever a bf16 PyTorch module produces a tensor (every Linear, every elementwise
result). Pinned by tests/golden/draft_tiny.npz, which the reference's own DraftHead produced. Nothing in the product
package may import this module.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from .oracle import bf16_round, bf16_to_f32


def rb(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 precision (kept as fp32)."""
    return bf16_to_f32(bf16_round(np.asarray(x, dtype=np.float32)))


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    ms = rb(rb(x * x).astype(np.float32).mean(-1, keepdims=True))
    r = rb(1.0 / np.sqrt(rb(ms + np.float32(eps))))
    return rb(rb(x * r) * w)


def linear(x: np.ndarray, W: np.ndarray) -> np.ndarray:
    return rb(x.astype(np.float32) @ W.astype(np.float32).T)


class DraftOracle:
    """sd: state dict of the reference's DraftHead as fp32 arrays holding bf16 values (keys merge.weight, q.weight, ...)."""

    def __init__(self, sd: Dict[str, np.ndarray], nh: int, rope_base: float, max_roll: int = 64, n_kv: Optional[int] = None):
        self.sd = sd
        self.dim = sd["q.weight"].shape[0]
        self.nh, self.nkv = nh, n_kv or nh
        self.hd = self.dim // nh
        self.rope_base = float(rope_base)
        self.kc = np.zeros((max_roll, self.nkv, self.hd), np.float32)
        self.vc = np.zeros((max_roll, self.nkv, self.hd), np.float32)

    def _rope(self, x, positions):
        half = self.hd // 2
        inv = (1.0 / (np.float32(self.rope_base) ** (np.arange(0, self.hd, 2, dtype=np.float32) / np.float32(self.hd)))).astype(np.float32)
        ang = np.outer(positions.astype(np.float32), inv).astype(np.float32)
        c, s = rb(np.cos(ang))[:, None, :], rb(np.sin(ang))[:, None, :]
        a, b = x[..., :half], x[..., half:]
        return np.concatenate([rb(rb(a * c) + rb(-b * s)), rb(rb(b * c) + rb(a * s))], -1)

    def forward(self, feat, emb, positions, slots=None):
        """feat [T, fdim], emb [T, dim] (fp32 holding bf16 values) -> predicted next features [T, fdim]."""
        sd, T = self.sd, feat.shape[0]
        x = linear(np.concatenate([feat, emb], -1), sd["merge.weight"])
        h = rmsnorm(x, sd["n1"])
        q = linear(h, sd["q.weight"]).reshape(T, self.nh, self.hd)
        k = linear(h, sd["k.weight"]).reshape(T, self.nkv, self.hd)
        v = linear(h, sd["v.weight"]).reshape(T, self.nkv, self.hd)
        q, k = self._rope(q, positions), self._rope(k, positions)
        sl = np.arange(T) if slots is None else np.asarray(slots)
        if slots is None:
            kc, vc = k, v
        else:
            self.kc[sl], self.vc[sl] = k, v
            kc, vc = self.kc, self.vc
        att = np.zeros((T, self.nh, self.hd), np.float32)
        rep = self.nh // self.nkv
        for t in range(T):
            last = int(sl[t])
            for hh in range(self.nh):
                sc = (kc[:last + 1, hh // rep] @ q[t, hh]) * np.float32(self.hd ** -0.5)
                p = np.exp(sc - sc.max())
                att[t, hh] = (p[:, None] * vc[:last + 1, hh // rep]).sum(0) / p.sum()
        att = rb(att).reshape(T, self.dim)
        x2 = rb(x + linear(att, sd["o.weight"]))
        h = rmsnorm(x2, sd["n2"])
        g, u = linear(h, sd["gate.weight"]), linear(h, sd["up.weight"])
        act = rb(rb(g / (1.0 + np.exp(-g))) * u)
        hh_ = rb(x2 + linear(act, sd["down.weight"]))
        return linear(hh_, sd["fout.weight"])

    def head_logits(self, f, nf, embed, logits_scaling: float = 1.0):
        """bf16 logits of the token head over the high slice of the (fused) feature."""
        return rb(linear(rmsnorm(f[..., -self.dim:], nf), embed) / np.float32(logits_scaling))


def sample_probs(logits: np.ndarray, temperature: float, top_k: int = 0) -> np.ndarray:
    """The distribution the reference's sample() draws from (reference: engine/generate.py:41-47)."""
    lg = logits.astype(np.float64) / max(temperature, 1e-5)
    if top_k and top_k < lg.size:
        kth = np.sort(lg)[-top_k]
        lg = np.where(lg < kth, -np.inf, lg)
    p = np.exp(lg - lg.max())
    return p / p.sum()
