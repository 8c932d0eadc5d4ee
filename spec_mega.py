#!/usr/bin/env python3
"""spec_mega.py — speculative decoding on the int4 verify path (the reference's entry point, reference: spec_mega.py).

An EAGLE draft head proposes K tokens, the target scores K+1 in one weight pass (`fb_verify`), the longest agreeing
prefix is accepted. No trained draft checkpoint exists offline, so the draft head has seeded random weights (acceptance
is then ~0) and `--forced-accept a` reports the throughput the loop WOULD have at a fixed accepted length a, as the
benchmark config asks: tok/s = (a + 1) / (t_draft + t_verify(M) + t_kv_move) on the static 26-node tree.

    python spec_mega.py --selftest                 # chain spec-decode, real acceptance (random draft)
    python spec_mega.py --tree --forced-accept 3   # static 26-node tree, forced accepted length
"""
import argparse
import time

import torch

from flint_b200.config import ModelArgs
from flint_b200.draft import seeded_draft
from flint_b200.generate import generate
from flint_b200.model import Transformer
from flint_b200.tree import kv_moves, static_tree, tree_mask


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--K", type=int, default=3)
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--tree", action="store_true")
    ap.add_argument("--nodes", type=int, default=26)
    ap.add_argument("--forced-accept", type=int, default=0)
    ap.add_argument("--cache", type=int, default=1024)
    ap.add_argument("--selftest", action="store_true")
    a = ap.parse_args()
    torch.set_grad_enabled(False)
    model = Transformer.from_name(a.config).load_synthetic(seed=0)
    cfg: ModelArgs = model.config
    draft = seeded_draft(cfg.dim, cfg.n_head, cfg.intermediate_size, seed=1, rope_base=cfg.rope_base, device="cuda")
    draft.bind_target(model.packed["embed"], model.packed["nf"], cfg.logits_scaling)
    draft.setup_cache(32 + 8)
    if not a.tree:
        prompt = torch.randint(0, cfg.vocab_size, (32,), generator=torch.Generator().manual_seed(1234), dtype=torch.int32)
        t0 = time.perf_counter()
        seq, stats = generate(model, prompt, a.max_new, interactive=False, draft_model=draft, speculate_k=a.K)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        print(f"{a.max_new} tokens · {a.max_new / dt:.1f} tok/s · accept counts {stats['accept_counts']} (random draft head)")
        return
    # static tree: verify latency and the forced-accept throughput
    model.setup_caches(1, a.cache + 128)
    eng = model.engine
    eng.kc[:, :a.cache].normal_()
    eng.vc[:, :a.cache].normal_()
    parent, depth = static_tree(a.nodes)
    am = torch.from_numpy(tree_mask(parent)).cuda()
    dp = torch.tensor(depth, dtype=torch.int32, device="cuda")
    toks = torch.randint(0, cfg.vocab_size, (a.nodes,), device="cuda", dtype=torch.int32)
    feat = torch.randn(32, cfg.dim, device="cuda").bfloat16()
    wtok = torch.full((32,), -1, dtype=torch.int32, device="cuda")

    def timed(fn, n=5):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n

    t_ver = timed(lambda: eng.verify(toks, a.cache, dp, am))
    pos32 = torch.arange(32, dtype=torch.int32, device="cuda")
    steps = [torch.tensor([32 + i], dtype=torch.int32, device="cuda") for i in range(4)]

    def rollout():                                   # window prime + 4 single steps = a depth-5 chain, all on the device
        fp = draft(feat, None, pos32, input_pos=pos32, tokens=wtok)
        f = fp[31:32]
        t = draft.head(f).view(1)
        for i in range(4):
            f = draft(f, None, steps[i], input_pos=steps[i], tokens=t)[0:1]
            t = draft.head(f).view(1)
    t_draft_eager = timed(rollout)
    g = torch.cuda.CUDAGraph()                       # the reference replays its draft from a CUDA graph too
    with torch.cuda.graph(g):
        rollout()
    t_draft = timed(g.replay)
    path = [0] + list(range(1, a.forced_accept + 1))
    src, dst = kv_moves([0] + [p + 3 for p in path[1:]], a.cache)
    t_mv = timed(lambda: eng.kv_move(src, dst)) if src else 0.0
    print(f"verify M={a.nodes}: {t_ver * 1e3:.2f} ms   draft rollout: {t_draft * 1e3:.2f} ms graphed ({t_draft_eager * 1e3:.2f} ms eager)"
          f"   kv move: {t_mv * 1e3:.3f} ms")
    for acc in range(1, 6):
        print(f"forced accepted length {acc}: {(acc + 1) / (t_draft + t_ver + t_mv):.0f} tok/s")


if __name__ == "__main__":
    main()
