#!/usr/bin/env python3
"""spec_tree.py — TREE speculative decoding on the int4 verify path (the reference's entry point, reference: spec_tree.py).

The EAGLE draft head rolls a width-B beam to depth D; `fb_verify` scores the whole tree in one weight pass with a tree
attention mask; the longest root-to-leaf path the target's greedy choices agree with is accepted and its cache rows are
made contiguous, all on the device. No trained draft checkpoint exists offline: with `--draft FILE` a checkpoint in the
reference's format ({"dim", "nh", "inter", "fuse", "state"}) is loaded, otherwise the draft head has seeded random
weights and acceptance is near zero (the output still equals plain greedy decoding, which `--check` verifies).

    python spec_tree.py --selftest --B 2 --D 6 --config tiny --check
"""
import argparse
import time

import torch

from flint_b200.draft import DraftHead, seeded_draft
from flint_b200.generate import generate, generate_tree
from flint_b200.model import Transformer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--draft", default="")
    ap.add_argument("--B", type=int, default=2)
    ap.add_argument("--D", type=int, default=6)
    ap.add_argument("--W", type=int, default=32)
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--selftest", action="store_true")
    ap.add_argument("--check", action="store_true", help="compare with plain greedy decoding of the same prompt")
    a = ap.parse_args()
    torch.set_grad_enabled(False)
    model = Transformer.from_name(a.config).load_synthetic(seed=0)
    cfg = model.config
    if a.draft:
        ck = torch.load(a.draft, map_location="cpu")
        draft = DraftHead(ck["dim"], ck["nh"], ck["inter"], fuse=ck.get("fuse", 1), rope_base=cfg.rope_base)
        draft.load_state_dict(ck["state"])
    else:
        draft = seeded_draft(cfg.dim, cfg.n_head, cfg.intermediate_size, seed=1, rope_base=cfg.rope_base)
    prompt = torch.randint(0, cfg.vocab_size, (32,), generator=torch.Generator().manual_seed(1234), dtype=torch.int32)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    seq, st = generate_tree(model, prompt, a.max_new, draft, beam=a.B, depth=a.D, window=a.W)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print(f"{a.max_new} tokens · {a.max_new / dt:.1f} tok/s · {st['tokens_per_pass']:.2f} tokens/pass · tree {st['tree_nodes']} nodes "
          f"(TREE spec-decode on the verify path)")
    if a.check:
        ref, _ = generate(model, prompt, a.max_new)
        same = int((ref == seq).sum())
        print(f"equal to plain greedy decoding at {same}/{seq.numel()} positions")


if __name__ == "__main__":
    main()
