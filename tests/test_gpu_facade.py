"""GPU: the gpt-fast style façade (`Transformer`, `generate`) and the speculative loops built on the kernels."""
import numpy as np
import pytest
import torch

from flint_b200 import packing
from flint_b200.config import ModelArgs
from flint_b200.draft import seeded_draft
from flint_b200.engine import DecodeEngine
from flint_b200.generate import generate, generate_tree
from flint_b200.model import Transformer
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _model():
    return Transformer.from_name("tiny").load_synthetic(seed=0)


def _prompt(n, seed=1234):
    return torch.randint(0, 4096, (n,), generator=torch.Generator().manual_seed(seed), dtype=torch.int32)


def _near_greedy(model, seq, T, tol=2e-2):
    """Every generated token of `seq` is the plain decode path's greedy choice given the tokens before it, or ties with
    it within the logit tolerance (a different kernel may resolve a near-tie the other way)."""
    eng = DecodeEngine(model.config, model.packed, max_seq=seq.numel() + 1)
    toks = seq.tolist()
    bad = 0
    for pos in range(len(toks) - 1):
        lg = eng.decode(toks[pos], pos).cpu().numpy()
        if pos >= T - 1:
            nxt = toks[pos + 1]
            if nxt != int(lg.argmax()) and lg.max() - lg[nxt] > tol:
                bad += 1
    eng.check()
    eng.close()
    return bad


def test_generate_greedy_equals_a_chained_decode_loop_after_the_same_prefill():
    """generate() is plumbing around the launches: the same prefill (causal chunks through the verify path) followed by a
    hand-written chained fb_decode loop gives the same tokens bit for bit."""
    model = _model()
    prompt, new = _prompt(70), 40                     # 70 > 64: two prefill chunks
    seq, stats = generate(model, prompt, new)
    assert seq.numel() == 70 + new and torch.equal(seq[:70].cpu(), prompt)
    eng = DecodeEngine(model.config, model.packed, max_seq=128)
    lg1, _ = eng.verify(prompt[:64].cuda(), 0)
    lg2, _ = eng.verify(prompt[64:].cuda(), 64)
    out = torch.zeros(new, dtype=torch.int32, device="cuda")
    out[0] = lg2[-1].argmax()
    for i in range(new - 1):
        eng.decode_chained(out[i:i + 1], 70 + i, out[i + 1:i + 2])
    eng.check()
    assert torch.equal(out, seq[70:])
    assert _near_greedy(model, seq, 70) == 0


def test_chunked_prefill_leaves_the_cache_a_token_by_token_prefill_leaves():
    model = _model()
    prompt = _prompt(150, 5)
    model.setup_caches(1, 256)
    lg, ft = model(prompt.view(1, -1), torch.arange(150), return_hidden=True)
    assert tuple(lg.shape) == (1, 150, 4096) and tuple(ft.shape) == (1, 150, 512)
    eng = DecodeEngine(model.config, model.packed, max_seq=256)
    last = None
    for p, t in enumerate(prompt.tolist()):
        last = eng.decode(t, p)
    eng.check()
    a = model.engine.kc[:, :150].float()
    assert (a - eng.kc[:, :150].float()).abs().max() < 0.05
    assert (model.engine.vc[:, :150].float() - eng.vc[:, :150].float()).abs().max() < 0.05
    assert (lg[0, -1] - last).abs().max() < 2e-2
    orc = O.OracleModel(model.config, {k: v.cpu() for k, v in model.packed.items()}, 256)
    for p, t in enumerate(prompt.tolist()):
        ref = orc.decode(t, p)
    assert np.abs(lg[0, -1].cpu().numpy() - ref).max() < 2e-2


def test_sampling_generate_is_on_device_and_reproducible():
    model = _model()
    prompt = _prompt(20, 7)
    a, _ = generate(model, prompt, 30, temperature=0.8, top_k=50, seed=3)
    b, _ = generate(model, prompt, 30, temperature=0.8, top_k=50, seed=3)
    c, _ = generate(model, prompt, 30, temperature=0.8, top_k=50, seed=4)
    g, _ = generate(model, prompt, 30)
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.equal(a, g)
    assert int(a.min()) >= 0 and int(a.max()) < 4096


def test_chain_speculation_output_is_greedy_decoding():
    """The reference's claim for its speculative loops: the output equals sequential greedy decoding whatever the draft
    proposes (reference: result.md:110-113). The draft head has seeded random weights, so most proposals are rejected;
    a second run with a draft that is forced to agree (its proposals replaced by the target's own tokens) is covered by
    the acceptance kernels' tests."""
    model = _model()
    cfg = model.config
    draft = seeded_draft(cfg.dim, cfg.n_head, cfg.intermediate_size, seed=1, rope_base=cfg.rope_base)
    prompt = _prompt(24, 9)
    seq, st = generate(model, prompt, 40, draft_model=draft, speculate_k=3)
    assert seq.numel() == 64 and sum(st["accept_counts"]) > 0
    assert _near_greedy(model, seq, 24) == 0


def test_tree_speculation_output_is_greedy_decoding():
    model = _model()
    cfg = model.config
    draft = seeded_draft(cfg.dim, cfg.n_head, cfg.intermediate_size, seed=2, rope_base=cfg.rope_base)
    prompt = _prompt(24, 10)
    seq, st = generate_tree(model, prompt, 24, draft, beam=2, depth=3, window=16)
    assert seq.numel() == 48 and st["passes"] > 0 and st["tree_nodes"] == 7
    assert _near_greedy(model, seq, 24) == 0


def test_tree_speculation_accepts_along_a_path_when_the_draft_is_right():
    """A draft whose proposals ARE the target's greedy continuation must be accepted to full depth: build the tree by
    hand from a greedy reference run, verify, accept and compact on the device, and continue decoding from the
    compacted cache: the continuation equals the greedy run."""
    from flint_b200.tree import tree_mask
    model = _model()
    prompt = _prompt(16, 11)
    ref, _ = generate(model, prompt, 12)
    ref = ref.tolist()
    eng = DecodeEngine(model.config, model.packed, max_seq=64)
    eng.verify(torch.tensor(ref[:15], dtype=torch.int32).cuda(), 0)               # prefill positions 0..14
    # root = token 15 (the last prompt token); right branch = greedy tokens 16, 17, 18; a wrong sibling at each depth
    cand = [ref[15], (ref[16] + 1) % 4096, ref[16], (ref[17] + 1) % 4096, ref[17], ref[18], (ref[18] + 1) % 4096]
    parent = [-1, 0, 0, 2, 2, 4, 4]
    depth = [0, 1, 1, 2, 2, 3, 3]
    c, p = torch.tensor(cand, dtype=torch.int32).cuda(), torch.tensor(parent, dtype=torch.int32).cuda()
    vlog, _ = eng.verify(c, 15, torch.tensor(depth, dtype=torch.int32).cuda(), torch.from_numpy(tree_mask(parent)).cuda())
    tgt = eng.sample(vlog, 0.0)
    acc = eng.accept_tree(c, p, tgt)
    eng.kv_compact(acc, 15)
    res = acc.tolist()
    assert res[0] == 4 and res[2:6] == [0, 2, 4, 5]
    nxt = torch.tensor([res[1]], dtype=torch.int32, device="cuda")
    out = [res[1]]
    for i in range(4):
        nn = torch.zeros(1, dtype=torch.int32, device="cuda")
        eng.decode_chained(nxt, 19 + i, nn)
        nxt = nn
        out.append(int(nn))
    eng.check()
    model2 = _model()
    full = ref[:19] + out
    assert _near_greedy(model2, torch.tensor(full, dtype=torch.int32), 16) == 0
