"""GPU: the speculative-decoding side kernels through the C ABI: sampling, acceptance, KV compaction, the draft head."""
import os

import numpy as np
import pytest
import torch

from flint_b200 import packing, tree
from flint_b200.config import ModelArgs
from flint_b200.draft import DraftHead, seeded_draft
from flint_b200.engine import DecodeEngine
from oracle import oracle as O
from oracle.draft_oracle import DraftOracle, sample_probs

pytestmark = pytest.mark.gpu


def _bf(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _f32(t):
    return O.bf16_to_f32(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))


@pytest.fixture(scope="module")
def eng():
    cfg = ModelArgs.from_name("tiny")
    e = DecodeEngine(cfg, {k: v.cuda() for k, v in packing.synth_packed(cfg, 0).items()}, max_seq=64)
    yield e
    e.close()


# ------------------------------------------------------------------------------------------------ sampling
def test_argmax_rows_first_index_on_ties(eng):
    lg = torch.randn(5, 4096, device="cuda")
    lg[2, 77] = lg[2, 900] = 50.0
    got = eng.sample(lg, 0.0).tolist()
    assert got == lg.argmax(-1).tolist() and got[2] == 77


@pytest.mark.parametrize("temperature,top_k", [(1.0, 0), (0.7, 5), (1.5, 40)])
def test_sampled_frequencies_follow_the_reference_distribution(eng, temperature, top_k):
    """20 000 draws from one logits vector (row stride 0, counters 0..n-1) against softmax(logits / T) over the top-k
    entries (reference: engine/generate.py:41-47): nothing outside the support, frequencies within 5 sigma."""
    g = torch.Generator().manual_seed(11)
    lg = (torch.randn(4096, generator=g) * 2.0).cuda()
    n = 20000
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    from flint_b200 import _lib
    import ctypes
    _lib.check(eng.lib.fb_sample(ctypes.c_void_p(lg.data_ptr()), 4096, n, 0, temperature, top_k, 123, 0,
                                 ctypes.c_void_p(out.data_ptr()), None), "fb_sample")
    counts = np.bincount(out.cpu().numpy(), minlength=4096).astype(np.float64)
    p = sample_probs(lg.cpu().numpy(), temperature, top_k)
    assert counts[p == 0].sum() == 0
    sigma = np.sqrt(n * p * (1 - p)) + 1.0
    assert np.all(np.abs(counts - n * p) < 5 * sigma), float(np.max(np.abs(counts - n * p) / sigma))
    # equal (seed, counter) -> equal tokens; another seed -> another sequence
    again = torch.empty(64, dtype=torch.int32, device="cuda")
    other = torch.empty(64, dtype=torch.int32, device="cuda")
    for buf, seed in ((again, 123), (other, 124)):
        _lib.check(eng.lib.fb_sample(ctypes.c_void_p(lg.data_ptr()), 4096, 64, 0, temperature, top_k, seed, 0,
                                     ctypes.c_void_p(buf.data_ptr()), None), "fb_sample")
    assert torch.equal(again, out[:64]) and not torch.equal(other, out[:64])


# ------------------------------------------------------------------------------------------------ acceptance, compaction
def test_accept_walks_match_the_host_functions(eng):
    t = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    for tgt, d in (([1, 2, 3, 9], [1, 2, 4]), ([5, 6], [7]), ([1, 2, 3, 4], [1, 2, 3])):
        res = eng.accept_chain(t(tgt), t(d)).tolist()
        acc = tree.chain_accept(tgt, d)
        assert res == [acc, tgt[acc]]
    parent = [-1, 0, 0, 1, 1, 2, 3]
    cand = [11, 22, 33, 44, 55, 66, 77]
    for tgt in ([22, 44, 0, 77, 0, 0, 9], [33, 0, 66, 0, 0, 5, 0], [0, 0, 0, 0, 0, 0, 0]):
        res = eng.accept_tree(t(cand), t(parent), t(tgt)).tolist()
        path = tree.tree_accept(cand, parent, tgt)
        assert res[0] == len(path) and res[2:2 + len(path)] == path and res[1] == tgt[path[-1]]


def test_kv_compact_equals_host_kv_move(eng):
    g = torch.Generator().manual_seed(3)
    eng.kc.copy_(torch.randn(eng.kc.shape, generator=g).bfloat16())
    eng.vc.copy_(torch.randn(eng.vc.shape, generator=g).bfloat16())
    k0, v0 = eng.kc.clone(), eng.vc.clone()
    path = [0, 2, 5, 6]
    acc = torch.tensor([len(path), 99] + path + [0] * 3, dtype=torch.int32, device="cuda")
    eng.kv_compact(acc, 10)
    torch.cuda.synchronize()
    k1, v1 = eng.kc.clone(), eng.vc.clone()
    eng.kc.copy_(k0)
    eng.vc.copy_(v0)
    eng.kv_move(*tree.kv_moves(path, 10))
    torch.cuda.synchronize()
    assert torch.equal(k1, eng.kc) and torch.equal(v1, eng.vc)
    assert torch.equal(k1[:, 11], k0[:, 12]) and torch.equal(k1[:, 12], k0[:, 15]) and torch.equal(k1[:, 13], k0[:, 16])


# ------------------------------------------------------------------------------------------------ draft head
def test_draft_forward_matches_the_reference_fixture(golden_dir):
    """The reference's own DraftHead output (tests/golden/draft_tiny.npz): plain causal mode, T = 6, positions 3..8."""
    g = np.load(os.path.join(golden_dir, "draft_tiny.npz"))
    dim, nh, inter = [int(x) for x in g["dims"]]
    m = DraftHead(dim, nh, inter, fuse=1, rope_base=10000.0)
    m.load_state_dict({k[3:]: _bf(g[k]) for k in g.files if k.startswith("sd_")})
    emb_t = torch.zeros(16, dim, dtype=torch.bfloat16, device="cuda")
    m.bind_target(emb_t, torch.ones(dim, dtype=torch.bfloat16, device="cuda"))
    m.setup_cache(8)
    out = m(_bf(g["feat"]).cuda(), _bf(g["emb"]).cuda(), torch.from_numpy(g["positions"]).cuda())
    ref = O.bf16_to_f32(g["out"])
    assert tuple(out.shape) == ref.shape
    assert np.abs(_f32(out) - ref).max() <= 2e-2 * np.abs(ref).max()
    assert np.abs(_f32(out) - ref).max() <= 2.0 ** -7 * np.abs(ref).max()        # in fact within two bf16 ulps


def test_draft_window_rollout_and_head_match_the_oracle():
    """Cache mode as the chain loop uses it (reference: spec_mega.py:59-87): a 12-row window primes slots 0..11, then
    three single-row steps at slots 12..14 whose token embeddings are looked up on the device; GQA heads (8 q / 2 kv),
    fused features (fuse = 2); the token head's top-3."""
    dim, nh, nkv, inter, fuse, vocab = 256, 8, 2, 512, 2, 1000
    m = seeded_draft(dim, nh, inter, seed=5, rope_base=10000.0, n_kv=nkv, fuse=fuse)
    g = torch.Generator().manual_seed(9)
    embed = (torch.randn(vocab, dim, generator=g) * 0.5).bfloat16().cuda()
    nf = (torch.rand(dim, generator=g) + 0.5).bfloat16().cuda()
    m.bind_target(embed, nf, logits_scaling=4.0)
    m.setup_cache(16)
    sd = {k: _f32(v) for k, v in m._w.items()}
    orc = DraftOracle(sd, nh, 10000.0, max_roll=16, n_kv=nkv)
    W = 12
    feat = (torch.randn(W, fuse * dim, generator=g)).bfloat16().cuda()
    toks = torch.full((W,), -1, dtype=torch.int32)
    toks[-1] = 17
    pos = torch.arange(W, dtype=torch.int32)
    out = m(feat, None, pos.cuda(), input_pos=pos.cuda(), tokens=toks.cuda())
    emb_np = np.zeros((W, dim), np.float32)
    emb_np[-1] = _f32(embed[17])
    ref = orc.forward(_f32(feat), emb_np, pos.numpy(), slots=np.arange(W))
    scale = np.abs(ref).max()
    assert np.abs(_f32(out) - ref).max() <= 2e-2 * scale
    f_dev, f_ref = out[W - 1:W], ref[W - 1:W]
    for i in range(3):
        t_dev, sc_dev = m.head(f_dev, top_b=3, want_scores=True)
        lg_ref = orc.head_logits(f_ref, _f32(nf), _f32(embed), 4.0)[0]
        top_ref = np.argsort(-lg_ref, kind="stable")[:3]
        # the device head must pick tokens whose oracle logits are the oracle's best ones (bf16 ties may swap)
        assert np.all(lg_ref[t_dev[0].cpu().numpy()] >= lg_ref[top_ref[2]] - 2.0 ** -6 * np.abs(lg_ref).max())
        assert abs(float(sc_dev[0, 0]) - float(lg_ref[top_ref[0]])) <= 2e-2 * np.abs(lg_ref).max()
        tok = int(t_dev[0, 0])
        sp = torch.tensor([W + i], dtype=torch.int32, device="cuda")
        f_dev = m(f_dev, None, sp, input_pos=sp, tokens=t_dev[0, 0:1])
        f_ref = orc.forward(f_ref, _f32(embed[tok])[None], np.array([W + i]), slots=np.array([W + i]))
        assert np.abs(_f32(f_dev) - f_ref).max() <= 3e-2 * np.abs(f_ref).max()
