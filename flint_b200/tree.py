"""Token trees for speculative decoding: the static EAGLE tree of the benchmark config, masks, acceptance walks.

The reference builds its trees dynamically from a beam (reference: spec_tree.py:53-104); the benchmark asks for a static
tree of 26 nodes, depth 5, per-depth branching (4, 2, 2, 1, 1). The rule used here is deterministic: enumerate the full
(4,2,2,1,1) tree (60 nodes below the root), score every node by the sum of child ranks along its path, keep the lowest
scores (ties in breadth-first order) — an ancestor-closed set, since a parent never scores higher than its child.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

BRANCHING = (4, 2, 2, 1, 1)


def _full_tree():
    nodes = [dict(parent=-1, depth=0, score=0)]            # breadth-first order
    frontier = [0]
    for d, br in enumerate(BRANCHING):
        nxt = []
        for p in frontier:
            for rank in range(br):
                nodes.append(dict(parent=p, depth=d + 1, score=nodes[p]["score"] + rank))
                nxt.append(len(nodes) - 1)
        frontier = nxt
    return nodes


def static_tree(n_nodes: int = 26) -> Tuple[List[int], List[int]]:
    """(parent[], depth[]) of the static tree with `n_nodes` nodes including the root, in breadth-first order.

    n <= 26: the first n nodes (BFS order) of the 26-node tree; 27..61: lowest-score nodes of the full tree;
    62..64: the full 61-node tree plus extra depth-1 children of the root as padding."""
    full = _full_tree()
    if n_nodes < 1 or n_nodes > 64:
        raise ValueError("1..64 nodes")
    def pick(k):
        order = sorted(range(1, len(full)), key=lambda i: (full[i]["score"], i))[:k - 1]
        return [0] + sorted(order)
    keep = pick(26)[:n_nodes] if n_nodes <= 26 else pick(min(n_nodes, len(full)))
    remap = {old: new for new, old in enumerate(keep)}
    parent = [-1 if full[i]["parent"] < 0 else remap[full[i]["parent"]] for i in keep]
    depth = [full[i]["depth"] for i in keep]
    while len(parent) < n_nodes:                           # padding nodes: extra children of the root
        parent.append(0)
        depth.append(1)
    return parent, depth


def tree_mask(parent: Sequence[int]) -> np.ndarray:
    """Ancestor-or-self mask uint8 [M, M] (reference: spec_tree.py:98-104)."""
    n = len(parent)
    m = np.zeros((n, n), dtype=np.uint8)
    for i in range(n):
        j = i
        while j != -1:
            m[i, j] = 1
            j = parent[j]
    return m


def chain_accept(target: Sequence[int], draft: Sequence[int]) -> int:
    """Longest prefix of the draft the target agrees with (reference: spec_mega.py:106-110)."""
    acc = 0
    for t, d in zip(target, draft):
        if int(t) != int(d):
            break
        acc += 1
    return acc


def tree_accept(cand: Sequence[int], parent: Sequence[int], target: Sequence[int]) -> List[int]:
    """Root-to-leaf walk along children whose token equals the target's choice (reference: spec_tree.py:108-118)."""
    children: Dict[int, List[int]] = {i: [] for i in range(len(cand))}
    for i, p in enumerate(parent):
        if p >= 0:
            children[p].append(i)
    path, cur = [0], 0
    while True:
        nxt = next((ch for ch in children[cur] if int(cand[ch]) == int(target[cur])), None)
        if nxt is None:
            return path
        path.append(nxt)
        cur = nxt


def kv_moves(path: Sequence[int], pos: int) -> Tuple[List[int], List[int]]:
    """Cache rows to copy so the accepted path becomes contiguous (reference: spec_tree.py:124-128)."""
    src, dst = [], []
    for step in range(1, len(path)):
        if pos + path[step] != pos + step:
            src.append(pos + path[step])
            dst.append(pos + step)
    return src, dst
