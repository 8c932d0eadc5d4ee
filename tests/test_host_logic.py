"""CPU: host-side logic that needs no GPU: the draft head against the reference's own output, trees, acceptance."""
import os

import numpy as np
import torch

from flint_b200 import tree
from flint_b200.draft import DraftHead
from oracle import oracle as O


def _bf(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_draft_head_matches_reference_forward(golden_dir):
    """The reference's DraftHead (reference: train/draft_model.py:24-64) evaluated on seeded inputs when the fixture was
    made; this re-implementation must load the same state dict and give the same bf16 output."""
    g = np.load(os.path.join(golden_dir, "draft_tiny.npz"))
    dim, nh, inter = [int(x) for x in g["dims"]]
    m = DraftHead(dim, nh, inter, fuse=1, rope_base=10000.0).to(torch.bfloat16).eval()
    sd = {k[3:]: _bf(g[k]) for k in g.files if k.startswith("sd_")}
    m.load_state_dict(sd, strict=True)
    with torch.no_grad():
        out = m(_bf(g["feat"]), _bf(g["emb"]), torch.from_numpy(g["positions"]))
    ref = _bf(g["out"]).float()
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


def test_static_trees_are_ancestor_closed_and_match_the_spec():
    p26, d26 = tree.static_tree(26)
    assert len(p26) == 26 and max(d26) == 5 and d26[0] == 0 and p26[0] == -1
    for n in (1, 16, 26, 40, 61, 64):
        p, d = tree.static_tree(n)
        assert len(p) == n
        for i in range(1, n):
            assert 0 <= p[i] < i and d[i] == d[p[i]] + 1
        kids = [sum(1 for q in p if q == i) for i in range(n)]
        for i in range(n):                       # per-depth branching limits (4, 2, 2, 1, 1); padding hangs off the root
            if i > 0:
                assert kids[i] <= tree.BRANCHING[d[i]] if d[i] < 5 else kids[i] == 0
    p16, d16 = tree.static_tree(16)
    assert p16 == p26[:16] and d16 == d26[:16]   # a BFS prefix of the 26-node tree
    m = tree.tree_mask(p26)
    assert np.array_equal(m, O.tree_mask(p26)) and m.trace() == 26 and (m[:, 0] == 1).all()


def test_accept_walks_and_kv_moves():
    parent = [-1, 0, 0, 1, 1, 2, 3]
    cand = [11, 22, 33, 44, 55, 66, 77]
    path = tree.tree_accept(cand, parent, [22, 44, 0, 77, 0, 0, 9])
    assert path == [0, 1, 3, 6] == O.tree_accept(cand, parent, [22, 44, 0, 77, 0, 0, 9])
    assert tree.kv_moves(path, 100) == ([103, 106], [102, 103])
    assert tree.chain_accept([1, 2, 3], [1, 2, 4]) == 2 == O.chain_accept([1, 2, 3], [1, 2, 4])
    assert tree.chain_accept([5], []) == 0
