"""CPU: packers and the oracle against the fixtures the reference itself produced (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from flint_b200 import packing
from flint_b200.config import ModelArgs
from oracle import oracle as O


def _bf(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_qpc_bit_exact_vs_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "packer_sym.npz"))
    W = _bf(g["W"])
    q, s = packing.qpc(W)
    assert np.array_equal(q.numpy(), g["q"])                      # every packed word identical
    assert np.array_equal(O._np(s), g["s"])                       # every bf16 scale identical
    nq, ns = O.np_qpc(g["W"])                                     # the oracle's numpy restatement too
    assert np.array_equal(nq, g["q"]) and np.array_equal(ns, g["s"])


def test_qpc_rejects_ragged_k():
    with pytest.raises(ValueError):
        packing.qpc(torch.zeros(4, 1376, dtype=torch.bfloat16))   # the reference fails on 1376 as well


def test_asym_bit_exact_vs_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "packer_asym.npz"))
    W = _bf(g["W"])
    q, s, z = packing.qpc_asym(W)
    sz = _bf(g["scales_and_zeros"])                               # [K/128, N, 2]
    rq, rs, rz = packing.from_gptfast(torch.from_numpy(g["w_int32"].astype(np.int32)), sz)
    assert torch.equal(q, rq) and torch.equal(s, rs) and torch.equal(z, rz)
    nq, ns, nz = O.np_qpc_asym(g["W"])
    assert np.array_equal(nq, q.numpy()) and np.array_equal(ns, O._np(s)) and np.array_equal(nz, O._np(z))
    # dequantised values: (q-8)*s+z in fp32, bit for bit against the reference's dequantiser
    dq = packing.dequant(q, s, z).numpy()
    assert np.array_equal(dq.view(np.uint32), g["dequant_f32"].view(np.uint32))
    assert np.array_equal(O.np_dequant(q.numpy(), O._np(s), O._np(z)).view(np.uint32), dq.view(np.uint32))
    assert np.array_equal(O.c_dequant(q, s, z).view(np.uint32), dq.view(np.uint32))


def test_dequant_sym_three_ways(golden_dir):
    g = np.load(os.path.join(golden_dir, "packer_sym.npz"))
    q, s = torch.from_numpy(g["q"]), _bf(g["s"])
    a = packing.dequant(q, s).numpy()
    assert np.array_equal(a.view(np.uint32), O.np_dequant(g["q"], g["s"]).view(np.uint32))
    assert np.array_equal(a.view(np.uint32), O.c_dequant(q, s).view(np.uint32))


def test_unpack_roundtrip():
    gen = torch.Generator().manual_seed(3)
    nib = torch.randint(0, 16, (5, 256), generator=gen, dtype=torch.int32)
    assert torch.equal(packing.unpack_nibbles(packing._pack_nibbles(nib)), nib)


def test_oracle_gemv_matches_dense():
    gen = torch.Generator().manual_seed(4)
    W = (torch.randn(40, 512, generator=gen) * 0.02).bfloat16()
    x = torch.randn(3, 512, generator=gen).bfloat16()
    for asym in (False, True):
        if asym:
            q, s, z = packing.qpc_asym(W)
        else:
            (q, s), z = packing.qpc(W), None
        ref = x.double() @ packing.dequant(q, s, z).double().T
        y = O.c_gemv(q, s, z, x)
        assert np.abs(y - ref.numpy()).max() < 2e-6 * max(1.0, float(ref.abs().max()))


def test_synth_packed_equals_pack_model():
    cfg = ModelArgs.from_name("tiny")
    a = packing.pack_model(packing.synth_weights(cfg, 0), cfg)
    b = packing.synth_packed(cfg, 0)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_oracle_vs_reference_engine_tiny(golden_dir):
    """The CPU oracle (megakernel rounding sites) against the reference's own PyTorch engine on the same
    fake-quantised weights. The two round at different places (the engine's RMSNorm rounds twice, its RoPE
    table is bf16), so logits agree to a few 1e-2, not bit for bit; the greedy tokens agree."""
    g = np.load(os.path.join(golden_dir, "engine_tiny.npz"))
    cfg = ModelArgs.from_name("tiny")
    m = O.OracleModel(cfg, packing.synth_packed(cfg, 0), max_seq=cfg.block_size)
    prompt, toks = g["prompt"].tolist(), g["tokens"].tolist()
    pos = 0
    for t in prompt[:-1]:
        m.decode(t, pos)
        pos += 1
    kept = {int(s): g["logits"][i] for i, s in enumerate(g["kept_steps"])}
    cur, agree, worst = prompt[-1], 0, 0.0
    for i in range(len(toks)):
        lg = m.decode(cur, pos)
        pos += 1
        agree += int(O.argmax_first(lg) == toks[i])
        if i in kept:
            worst = max(worst, float(np.abs(lg - kept[i]).max()))
        cur = toks[i]                                             # teacher-forced on the reference's tokens
    assert agree == len(toks), f"greedy agreement {agree}/{len(toks)}"
    assert worst < 3e-2, worst


def test_verify_chain_equals_sequential_decode():
    """verify(M tokens, chain mask) must reproduce M sequential decode steps (the reference's own check of
    its verify kernel, reference: bench/verify_mega_test.py:43-59)."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 0)
    a, b = O.OracleModel(cfg, P, 64), O.OracleModel(cfg, P, 64)
    toks = [5, 17, 99, 1024, 7, 4000]
    for p, t in enumerate(toks[:2]):
        a.decode(t, p)
        b.decode(t, p)
    seq = np.stack([a.decode(t, 2 + i) for i, t in enumerate(toks[2:])])
    lg, _ = b.verify(toks[2:], 2)
    assert np.array_equal(seq.argmax(-1), lg.argmax(-1))
    assert np.abs(seq - lg).max() < 1e-5
    assert np.array_equal(a.kc, b.kc) and np.array_equal(a.vc, b.vc)


def test_tree_verify_matches_per_path_decode():
    """A branching tree: every node's logits equal those of decoding its root-to-node path sequentially."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 0)
    parent = [-1, 0, 0, 1, 1, 2, 3]
    cand = [11, 22, 33, 44, 55, 66, 77]
    depth = [0, 1, 1, 2, 2, 2, 3]
    base = O.OracleModel(cfg, P, 64)
    prefix = [3, 1, 4, 1, 5]
    for p, t in enumerate(prefix):
        base.decode(t, p)
    lg, _ = base.verify(cand, len(prefix), depth, O.tree_mask(parent))
    for node in range(len(cand)):
        path = []
        j = node
        while j != -1:
            path.append(j)
            j = parent[j]
        path.reverse()
        m = O.OracleModel(cfg, P, 64)
        for p, t in enumerate(prefix):
            m.decode(t, p)
        for k, n in enumerate(path):
            out = m.decode(cand[n], len(prefix) + k)
        assert np.abs(out - lg[node]).max() < 1e-5, node
    assert O.tree_accept(cand, parent, [22, 44, 0, 77, 0, 0, 9]) == [0, 1, 3, 6]
    assert O.chain_accept([1, 2, 3], [1, 2, 4]) == 2


def test_oracle_one_ulp_sensitivity():
    """How far the ORACLE's own logits move when one bf16 ulp of one embedding element is flipped. Rounding to
    bf16 at every store site makes the step discontinuous: a flip either dies out (exactly 0) or cascades through
    the following layers. Any two correct implementations that sum in different orders differ by such flips, so this
    number, not fp32 epsilon, is the floor of implementation-to-implementation agreement."""
    cfg = ModelArgs.from_name("tiny")
    m = O.OracleModel(cfg, packing.synth_packed(cfg, 0), 8)
    h = m.embed_rows([17])
    base = m.step_h(h, 0)[0]
    moved = []
    for idx in range(0, cfg.dim, 37):
        h2 = h.copy()
        h2[0, idx] ^= 1
        moved.append(float(np.abs(m.step_h(h2, 0)[0] - base).max()))
    assert max(moved) > 1e-3          # cascades happen: agreement to fp32 epsilon is not attainable
    assert max(moved) < 2e-2          # and at 4 layers they stay inside the 2e-2 bar
