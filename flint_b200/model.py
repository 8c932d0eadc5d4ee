"""gpt-fast style façade over the decode / verify kernels: `Transformer`, `setup_caches`, `model(idx, input_pos)`.

Keeps the call surface of the reference engine (reference: engine/model.py:100-149) so `generate()`-style loops run
unchanged: one position -> one decode megakernel launch; several positions -> the M-token verify path with a causal
mask, in chunks of 64 (which also gives chunked prefill instead of the reference's token-by-token prompt loop,
reference: chat.py:85-86).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import packing
from .config import ModelArgs
from .engine import DecodeEngine


class Transformer:
    def __init__(self, config: ModelArgs) -> None:
        self.config = config
        self.packed: Optional[Dict[str, torch.Tensor]] = None
        self.engine: Optional[DecodeEngine] = None
        self.max_batch_size = -1
        self.max_seq_length = -1

    @classmethod
    def from_name(cls, name: str) -> "Transformer":
        return cls(ModelArgs.from_name(name))

    # ---- weights: a packed dict as the reference's load_packed returns (reference: chat.py:32-52) ----
    def load_packed(self, packed: Dict[str, torch.Tensor]) -> "Transformer":
        self.packed = packed
        self.engine = None
        return self

    def load_synthetic(self, seed: int = 0, device: str = "cuda", asym: bool = False) -> "Transformer":
        return self.load_packed(packing.synth_packed(self.config, seed, device=device, asym=asym))

    def setup_caches(self, max_batch_size: int, max_seq_length: int) -> None:
        if max_batch_size != 1:
            raise ValueError("this path is batch 1 (the reference megakernel is too)")
        if self.packed is None:
            raise RuntimeError("load weights first (load_packed / load_synthetic)")
        if self.engine is not None and self.max_seq_length >= max_seq_length:
            return
        max_seq_length = (max_seq_length + 7) // 8 * 8          # reference: engine/model.py:118
        self.engine = DecodeEngine(self.config, self.packed, max_seq=max_seq_length)
        self.max_batch_size, self.max_seq_length = 1, max_seq_length

    def forward(self, idx: torch.Tensor, input_pos: torch.Tensor, return_hidden: bool = False):
        """idx [1, S] token ids, input_pos [S] consecutive positions -> logits f32 [1, S, vocab] (and the post-norm
        hidden bf16 [1, S, dim] when return_hidden)."""
        if self.engine is None:
            raise RuntimeError("Caches must be initialized first")
        toks = idx.reshape(-1).to(torch.int32)
        S = toks.numel()
        pos0 = int(input_pos.reshape(-1)[0])
        if S == 1 and not return_hidden:
            lg = self.engine.decode(int(toks[0]), pos0).clone()
            return lg.view(1, 1, -1)
        outs, feats = [], []
        for s in range(0, S, 64):
            lg, ft = self.engine.verify(toks[s:s + 64], pos0 + s)
            outs.append(lg)
            feats.append(ft)
        logits = torch.cat(outs).unsqueeze(0)
        return (logits, torch.cat(feats).unsqueeze(0)) if return_hidden else logits

    __call__ = forward
