"""CPU: host-side logic that needs no GPU: the draft-head oracle against the reference's own output, trees, acceptance."""
import os

import numpy as np
import torch

from flint_b200 import tree
from oracle import oracle as O


def test_draft_oracle_matches_reference_forward(golden_dir):
    """The reference's DraftHead (reference: train/draft_model.py:24-64) evaluated on seeded inputs when the fixture was
    made: the numpy restatement the CUDA draft kernels are checked against reproduces its bf16 output to one ulp."""
    from oracle.draft_oracle import DraftOracle
    g = np.load(os.path.join(golden_dir, "draft_tiny.npz"))
    dim, nh, inter = [int(x) for x in g["dims"]]
    sd = {k[3:]: O.bf16_to_f32(g[k]) for k in g.files if k.startswith("sd_")}
    m = DraftOracle(sd, nh, 10000.0)
    out = m.forward(O.bf16_to_f32(g["feat"])[0], O.bf16_to_f32(g["emb"])[0], g["positions"])
    ref = O.bf16_to_f32(g["out"])[0]
    assert np.abs(out - ref).max() <= 2.0 ** -8 * np.abs(ref).max()          # one bf16 ulp at the largest magnitude
    assert (out == ref).mean() > 0.5
    # cache mode with slots = 0..T-1 is the same computation
    m2 = DraftOracle(sd, nh, 10000.0, max_roll=8)
    out2 = m2.forward(O.bf16_to_f32(g["feat"])[0], O.bf16_to_f32(g["emb"])[0], g["positions"], slots=np.arange(6))
    assert np.array_equal(out, out2)


def test_sample_distribution_helper_masks_top_k():
    from oracle.draft_oracle import sample_probs
    lg = np.array([1.0, 3.0, 2.0, 3.0, -1.0], np.float32)
    p = sample_probs(lg, 1.0, 2)
    assert p[0] == 0 and p[4] == 0 and p[2] == 0 and abs(p[1] - 0.5) < 1e-12      # the two tied maxima survive
    p = sample_probs(lg, 0.5, 0)
    assert abs(p.sum() - 1) < 1e-12 and p.argmax() in (1, 3)


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


def test_build_time_extra_shapes_become_kernel_table_macros():
    """A model shape the built-in kernel table lacks is added by an environment variable at build time: the macros name
    one decode entry per shape and only the widths the re-layout kernels do not have yet."""
    from flint_b200.csrc.build import BUILT_IN_K, extra_shape_flags
    assert extra_shape_flags("") == []
    flags = extra_shape_flags("4096,4096,11008,128,1; 3072,3072,8192,128,3")
    assert flags[0] == "-DFB_EXTRA_DECODE_ENTRIES=FB_DECODE_ENTRY(4096,4096,11008,128,1),FB_DECODE_ENTRY(3072,3072,8192,128,3),"
    assert flags[1] == "-DFB_EXTRA_K(X)=X(3072) X(11008)"
    # the Python list mirrors the C++ one
    import os, re
    src = open(os.path.join(os.path.dirname(__file__), "..", "flint_b200", "csrc", "fb_api.cu")).read()
    line = [l for l in src.splitlines() if l.startswith("#define FB_FOR_EACH_K(X)")][0]
    assert tuple(int(v) for v in re.findall(r"X\((\d+)\)", line)) == BUILT_IN_K
    assert extra_shape_flags("2560,2560,8192,80,4") == ["-DFB_EXTRA_DECODE_ENTRIES=FB_DECODE_ENTRY(2560,2560,8192,80,4),"]
    import pytest
    with pytest.raises(ValueError):
        extra_shape_flags("4096,4096,11000,128,1")
    with pytest.raises(ValueError):
        extra_shape_flags("4096,4096,11008,128")
