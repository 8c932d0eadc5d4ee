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


@pytest.mark.parametrize("M", [8, 16])
def test_reference_verify_kernel_vs_oracle_vs_ours(M):
    """The reference's own `verify_mega_launch` (reference: kernels/verify_mega.cu:246-283) at its native head shape on a
    branching tree: the oracle and this library against it, per token row, with the reference's criterion
    (reference: bench/verify_mega_test.py:54-56)."""
    ref = build_ref.load_module("flint_ref_verify")
    if ref is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    from flint_b200.tree import static_tree
    cfg = _native_cfg(2, 4096)
    W = packing.synth_packed(cfg, 0, device="cuda", norm_mode="ref")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 128)
    eng = DecodeEngine(cfg, W, max_seq=128)
    kc = torch.zeros(cfg.n_layer, 128, 8, 64, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    T0 = 70                                            # a cached prefix: the same seeded rows in all three caches
    kv = (torch.randn(2, cfg.n_layer, T0, 8, 64, generator=torch.Generator().manual_seed(7)) * 0.5).bfloat16()
    for dst_k, dst_v in ((kc, vc), (eng.kc, eng.vc)):
        dst_k[:, :T0].copy_(kv[0])
        dst_v[:, :T0].copy_(kv[1])
    orc.kc[:, :T0] = kv[0].view(torch.int16).numpy().view(np.uint16)
    orc.vc[:, :T0] = kv[1].view(torch.int16).numpy().view(np.uint16)
    parent, depth = static_tree(M)
    amask = O.tree_mask(parent)
    toks = torch.randint(0, cfg.vocab_size, (M,), generator=torch.Generator().manual_seed(M)).tolist()
    h = (W["embed"][torch.tensor(toks, device="cuda")].float() * cfg.embedding_multiplier).to(torch.bfloat16)
    out = ref.verify_mega_launch(W["qkv_q"], W["qkv_s"], W["o_q"], W["o_s"], W["n1"], W["gu_q"], W["gu_s"], W["d_q"],
                                 W["d_s"], W["n2"], W["nf"], W["lm_q"], W["lm_s"], h, kc, vc,
                                 torch.tensor(depth, dtype=torch.int32, device="cuda"),
                                 torch.from_numpy(amask).cuda(), T0, M, cfg.attn_scale, float(cfg.rope_base),
                                 cfg.residual_multiplier, cfg.logits_scaling)
    torch.cuda.synchronize()
    lr = out[0].cpu().numpy()
    lo, _ = orc.verify(toks, T0, np.asarray(depth, np.int32), amask)
    lu, _ = eng.verify(toks, T0, depth, torch.from_numpy(amask))
    eng.check()
    lu = lu.cpu().numpy()
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    for m in range(M):
        assert rel(lo[m], lr[m]) < 0.02, ("oracle vs reference kernel", m, rel(lo[m], lr[m]))
        assert rel(lu[m], lr[m]) < 0.02, ("this library vs reference kernel", m, rel(lu[m], lr[m]))
        assert int(np.argmax(lr[m])) in (int(np.argmax(lo[m])), int(np.argmax(lu[m]))) or \
            lr[m].max() - lr[m][int(np.argmax(lu[m]))] < 2e-2 * max(1.0, float(np.abs(lr[m]).max()) / 2.56)
