#!/usr/bin/env python3
"""chat.py — token-level chat loop on the B200 decode megakernel (the reference's entry point, reference: chat.py).

The reference downloads Granite-4.1-3B and its tokenizer; neither is available offline, so this entry point speaks token
ids. `--selftest` prefills a fixed random prompt, generates and prints tok/s (reference: chat.py:103-107). Without it
the turn loop of the reference runs (reference: chat.py:109-131): every line read from standard input is one user turn
given as token ids, the history of both sides is kept as the prompt of the next turn, the reply streams out token by
token through the callback, and a full context restarts the conversation from the latest turn. `--checkpoint DIR` loads a
Hugging Face checkpoint directory (safetensors + config.json) instead of the seeded synthetic model.

    python chat.py --selftest
    python chat.py --config granite-4.1-3b --max-new 256 --tokens "5 17 99"
    printf '5 17 99\n12 13\n' | python chat.py --config tiny --max-new 16
"""
import argparse
import sys
import time

import torch

from flint_b200.config import ModelArgs
from flint_b200.generate import generate
from flint_b200.model import Transformer


def respond(model, ids, max_new, kw, stream=True):
    """One assistant turn: prefill `ids`, generate, stream the ids as they are read back; returns (reply ids, seconds)."""
    prompt = torch.tensor(ids, dtype=torch.int32)
    shown = []

    def cb(t):
        shown.append(int(t))
        if stream:
            sys.stdout.write(f"{shown[-1]} ")
            sys.stdout.flush()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    generate(model, prompt, max_new, interactive=False, draft_model=None, callback=cb, **kw)
    torch.cuda.synchronize()
    return shown, time.perf_counter() - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--checkpoint", default="", help="Hugging Face checkpoint directory (safetensors + config.json)")
    ap.add_argument("--temp", type=float, default=0.0)
    ap.add_argument("--topk", type=int, default=0)
    ap.add_argument("--max-new", type=int, default=256)
    ap.add_argument("--maxseq", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tokens", default="")
    ap.add_argument("--selftest", action="store_true")
    a = ap.parse_args()
    torch.set_grad_enabled(False)
    if a.checkpoint:
        from flint_b200.checkpoint import load_hf_checkpoint
        print(f"loading + int4-packing {a.checkpoint} ...", flush=True)
        cfg, packed = load_hf_checkpoint(a.checkpoint, device="cuda")
        model = Transformer(cfg).load_packed(packed)
    else:
        print(f"building seeded synthetic {a.config} (int4 g128) ...", flush=True)
        model = Transformer.from_name(a.config).load_synthetic(seed=a.seed)
    model.config.block_size = a.maxseq
    cfg: ModelArgs = model.config
    kw = dict(temperature=a.temp, top_k=(a.topk or None), seed=a.seed)
    if a.selftest or a.tokens:
        if a.tokens:
            ids = [int(t) for t in a.tokens.split()]
        else:
            ids = torch.randint(0, cfg.vocab_size, (128,), generator=torch.Generator().manual_seed(1234)).tolist()
        respond(model, ids, 8, kw, stream=False)                                  # warm-up: builds the context
        new, dt = respond(model, ids, a.max_new, kw)
        print(f"\n{len(new)} tokens · {len(new) / dt:.1f} tok/s including the {len(ids)}-token prefill "
              f"(megakernel int4, {cfg.n_layer} layers, d {cfg.dim})")
        return
    print("flint_b200 chat on token ids: one line of ids per turn, empty line or EOF to quit.")
    history = []
    for line in sys.stdin:
        turn = [int(t) for t in line.split()]
        if not turn:
            break
        if any(t < 0 or t >= cfg.vocab_size for t in turn):
            print(f"(ids must be in [0, {cfg.vocab_size}))")
            continue
        ids = history + turn
        if len(ids) >= a.maxseq - a.max_new:                                      # reference: chat.py:117-120
            print("(context full — restarting conversation)")
            ids = turn[-(a.maxseq - a.max_new - 1):]
        sys.stdout.write("flint> ")
        reply, dt = respond(model, ids, a.max_new, kw)
        print(f"\n[{len(reply)} tokens · {len(reply) / max(dt, 1e-9):.1f} tok/s]")
        history = ids + reply


if __name__ == "__main__":
    main()
