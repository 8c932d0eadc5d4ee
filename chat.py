#!/usr/bin/env python3
"""chat.py — token-level chat loop on the B200 decode megakernel (the reference's entry point, reference: chat.py).

The reference downloads Granite-4.1-3B and its tokenizer; neither is available offline, so this entry point runs on a
seeded synthetic model and speaks token ids: `--selftest` prefills a fixed random prompt, generates, prints tok/s.
With `--tokens "1 2 3"` the prompt is the given ids. Greedy by default (the megakernel path), `--temp/--topk` sample.

    python chat.py --selftest
    python chat.py --config granite-4.1-3b --max-new 256 --tokens "5 17 99"
"""
import argparse
import time

import torch

from flint_b200.config import ModelArgs
from flint_b200.generate import generate
from flint_b200.model import Transformer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--temp", type=float, default=0.0)
    ap.add_argument("--topk", type=int, default=0)
    ap.add_argument("--max-new", type=int, default=256)
    ap.add_argument("--maxseq", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tokens", default="")
    ap.add_argument("--selftest", action="store_true")
    a = ap.parse_args()
    torch.set_grad_enabled(False)
    print(f"building seeded synthetic {a.config} (int4 g128) ...", flush=True)
    model = Transformer.from_name(a.config).load_synthetic(seed=a.seed)
    model.config.block_size = a.maxseq
    cfg: ModelArgs = model.config
    if a.tokens:
        prompt = torch.tensor([int(t) for t in a.tokens.split()], dtype=torch.int32)
    else:
        prompt = torch.randint(0, cfg.vocab_size, (128 if a.selftest else 16,), generator=torch.Generator().manual_seed(1234),
                               dtype=torch.int32)
    kw = dict(temperature=a.temp, top_k=(a.topk or None))
    generate(model, prompt, 8, interactive=False, draft_model=None, **kw)          # warm-up: builds the context
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    seq, _ = generate(model, prompt, a.max_new, interactive=False, draft_model=None, **kw)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    new = seq[prompt.numel():].tolist()
    print(" ".join(str(t) for t in new[:64]) + (" ..." if len(new) > 64 else ""))
    print(f"\n{len(new)} tokens · {len(new) / dt:.1f} tok/s including the {prompt.numel()}-token prefill "
          f"(megakernel int4, {cfg.n_layer} layers, d {cfg.dim})")


if __name__ == "__main__":
    main()
