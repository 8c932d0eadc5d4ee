"""GPU: the reference's OWN megakernel (built from the reference checkout into oracle/_ref by oracle/build_ref.py)
as a second checker, at the only head shape it supports (40 query / 8 kv heads of 64, Granite multipliers).

Pins two things: the CPU oracle against the real reference kernel, and this library against it, with the reference's
own criterion (rel-L2 < 0.02 and equal argmax, reference: bench/verify_mega_test.py:54-56)."""
import os

import numpy as np
import pytest
import torch

from flint_b200 import packing
from flint_b200.config import ModelArgs
from flint_b200.engine import DecodeEngine
from oracle import build_ref
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _native_cfg(n_layer, vocab):
    return ModelArgs(block_size=64, vocab_size=vocab, n_layer=n_layer, n_head=40, n_local_heads=8, dim=2560,
                     intermediate_size=8192, rope_base=10000000, embedding_multiplier=12.0,
                     attention_multiplier=0.015625, residual_multiplier=0.22, logits_scaling=10.0)


def test_reference_megakernel_vs_oracle_vs_ours():
    ref = build_ref.load_module("flint_ref_decode")
    if ref is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    cfg = _native_cfg(2, 4096)
    W = packing.synth_packed(cfg, 0, device="cuda", norm_mode="ref")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 64)
    eng = DecodeEngine(cfg, W, max_seq=64)
    kc = torch.zeros(cfg.n_layer, 64, 8, 64, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    toks = [11, 4000, 77, 1234, 9, 2048]
    for pos, t in enumerate(toks):
        h = (W["embed"][t].float() * cfg.embedding_multiplier).to(torch.bfloat16)
        lr = ref.decode_mega_launch(W["qkv_q"], W["qkv_s"], W["o_q"], W["o_s"], W["n1"], W["gu_q"], W["gu_s"], W["d_q"],
                                    W["d_s"], W["n2"], W["nf"], W["lm_q"], W["lm_s"], h, kc, vc, pos, cfg.attn_scale,
                                    float(cfg.rope_base), cfg.residual_multiplier, cfg.logits_scaling)
        torch.cuda.synchronize()
        lr = lr.cpu().numpy()
        lo = orc.decode(t, pos)
        lu = eng.decode(t, pos).cpu().numpy()
        eng.check()
        rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
        assert rel(lo, lr) < 0.02, ("oracle vs reference kernel", pos, rel(lo, lr))
        assert rel(lu, lr) < 0.02, ("this library vs reference kernel", pos, rel(lu, lr))
        assert int(np.argmax(lo)) == int(np.argmax(lr)) == int(np.argmax(lu))
