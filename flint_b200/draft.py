"""EAGLE draft head on the extension's kernels (`fb_draft_*` in include/flint_b200.h).

The object keeps the reference's surface (reference: train/draft_model.py:24-64): constructor arguments, the state-dict
keys of its checkpoints (`merge.weight`, `n1`, `q.weight` ... `fout.weight`), `setup_cache`, and a call
`draft(feat, emb, positions, input_pos=None)` returning the predicted next (fused) features. There is no PyTorch
arithmetic here: tensors are device memory handed to the C ABI. The token head (final norm of the target + tied
embedding, reference: spec_mega.py:43-44) is `head()`; it returns token ids on the device.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import _lib

_KEYS = {"merge": "merge.weight", "n1": "n1", "n2": "n2", "q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight",
         "gate": "gate.weight", "up": "up.weight", "down": "down.weight", "fout": "fout.weight"}


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class DraftHead:
    def __init__(self, dim: int, nh: int, inter: int, fuse: int = 1, rope_base: float = 1e7, n_kv: Optional[int] = None,
                 norm_eps: float = 1e-5):
        self.dim, self.nh, self.nkv, self.inter, self.fuse = dim, nh, n_kv or nh, inter, fuse
        self.hd, self.fdim, self.rope_base, self.eps = dim // nh, fuse * dim, float(rope_base), float(norm_eps)
        self.lib = _lib.load()
        self._h = ctypes.c_void_p()
        self._w: Dict[str, torch.Tensor] = {}
        self._target = None
        self.max_roll = 0
        self.max_tokens = 64

    # ---- weights ----
    def state_shapes(self) -> Dict[str, tuple]:
        d, kv, f, i = self.dim, self.nkv * self.hd, self.fdim, self.inter
        return {"merge.weight": (d, f + d), "n1": (d,), "n2": (d,), "q.weight": (d, d), "k.weight": (kv, d),
                "v.weight": (kv, d), "o.weight": (d, d), "gate.weight": (i, d), "up.weight": (i, d), "down.weight": (d, i),
                "fout.weight": (f, d)}

    def load_state_dict(self, sd: Dict[str, torch.Tensor], device="cuda") -> "DraftHead":
        shapes = self.state_shapes()
        missing = [k for k in shapes if k not in sd]
        if missing:
            raise KeyError(f"draft checkpoint lacks {missing}")
        for k, shp in shapes.items():
            t = sd[k]
            if tuple(t.shape) != shp:
                raise ValueError(f"{k}: shape {tuple(t.shape)}, expected {shp}")
            self._w[k] = t.detach().to(device=device, dtype=torch.bfloat16).contiguous()
        self._bind()
        return self

    def bind_target(self, embed: torch.Tensor, nf: torch.Tensor, logits_scaling: float = 1.0) -> "DraftHead":
        """The target's embedding table (bf16 [vocab, dim], raw: no multiplier, reference: spec_mega.py:68,78) and final
        norm weight: the draft's token head and its on-device embedding lookup use them."""
        self._target = (embed.contiguous(), nf.contiguous(), float(logits_scaling))
        self._bind()
        return self

    def setup_cache(self, max_roll: int, device=None, dtype=torch.bfloat16) -> None:
        self.max_roll = int(max_roll)
        self._bind()

    def _bind(self):
        if not self._w or self._target is None or self.max_roll <= 0:
            return
        embed, nf, ls = self._target
        if self._h.value:
            self.lib.fb_draft_destroy(self._h)
            self._h = ctypes.c_void_p()
        dev = embed.device
        d = _lib.DraftDesc(self.dim, self.nh, self.nkv, self.inter, self.fuse, embed.shape[0], self.max_roll, self.max_tokens,
                           self.rope_base, self.eps, ls)
        _lib.check(self.lib.fb_draft_create(ctypes.byref(d), dev.index or 0, ctypes.byref(self._h)), "fb_draft_create")
        w = _lib.DraftWeights()
        for f, k in _KEYS.items():
            setattr(w, f, self._w[k].data_ptr())
        w.nf, w.embed = nf.data_ptr(), embed.data_ptr()
        _lib.check(self.lib.fb_draft_bind(self._h, ctypes.byref(w)), "fb_draft_bind")
        self.device = dev

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.fb_draft_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- launches (asynchronous on the current stream) ----
    def forward(self, feat: torch.Tensor, emb: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
                input_pos: Optional[torch.Tensor] = None, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """feat [1, T, fdim] or [T, fdim]; the embeddings either as `emb` (same leading shape, dim wide) or as `tokens`
        (int32 [T] on the device, a negative id = zero row) looked up on the device. input_pos = cache slots."""
        if not self._h.value:
            raise RuntimeError("load_state_dict, bind_target and setup_cache first")
        lead = feat.shape[:-1]
        f2 = feat.reshape(-1, self.fdim).contiguous()
        T = f2.shape[0]
        dev = f2.device
        pos = (torch.arange(T, device=dev) if positions is None else positions).to(device=dev, dtype=torch.int32).contiguous()
        slots = None if input_pos is None else input_pos.to(device=dev, dtype=torch.int32).contiguous()
        e2 = None if emb is None else emb.reshape(-1, self.dim).to(torch.bfloat16).contiguous()
        tk = None if tokens is None else tokens.to(device=dev, dtype=torch.int32).contiguous()
        out = torch.empty(T, self.fdim, dtype=torch.bfloat16, device=dev)
        st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(self.lib.fb_draft_forward(self._h, _p(f2), _p(e2), _p(tk), _p(pos), _p(slots), T, _p(out), st),
                   "fb_draft_forward")
        self._keep = (f2, e2, tk, pos, slots)
        return out.view(*lead, self.fdim)

    __call__ = forward

    def head(self, f_rows: torch.Tensor, top_b: int = 1, want_scores: bool = False):
        """Feature rows [n, fdim] -> token ids int32 [n, top_b] on the device (best first) (and their bf16-rounded logits)."""
        f2 = f_rows.reshape(-1, self.fdim).contiguous()
        n = f2.shape[0]
        toks = torch.empty(n, top_b, dtype=torch.int32, device=f2.device)
        sc = torch.empty(n, top_b, dtype=torch.float32, device=f2.device) if want_scores else None
        st = ctypes.c_void_p(torch.cuda.current_stream(f2.device).cuda_stream)
        _lib.check(self.lib.fb_draft_head(self._h, _p(f2), n, top_b, _p(toks), _p(sc), st), "fb_draft_head")
        self._keep_h = f2
        return (toks, sc) if want_scores else toks


def seeded_draft(dim: int, nh: int, inter: int, seed: int = 0, rope_base: float = 10000.0, device="cuda",
                 n_kv: Optional[int] = None, fuse: int = 1) -> DraftHead:
    """Draft head with seeded N(0, 0.02) weights (stand-in for a trained EAGLE checkpoint, which needs the training
    kit and datasets the reference used)."""
    g = torch.Generator().manual_seed(seed)
    m = DraftHead(dim, nh, inter, fuse=fuse, rope_base=rope_base, n_kv=n_kv)
    sd = {k: (torch.randn(shp, generator=g) * 0.02 if len(shp) == 2 else torch.ones(shp)) for k, shp in m.state_shapes().items()}
    return m.load_state_dict(sd, device=device)
