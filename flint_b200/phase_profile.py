"""Per-phase timeline of one decode step (the run-time replacement of the reference's -DNOSYNC / -DNOATTN builds).

    python -m flint_b200.phase_profile --config granite-3b-class --cached 200

Every CTA stamps %globaltimer at the phase boundaries of every layer (fb_set_option(ctx, 2, buffer)); this prints,
per phase, the mean / min / max over CTAs of the time spent, averaged over the middle layers, and the layer period.
"""
import argparse

import numpy as np
import torch

from . import packing
from .config import ModelArgs
from .engine import DecodeEngine, query

NAMES = ["qkv wait+stage", "qkv gemv+epi", "attention", "o wait+stage", "o gemv+epi", "gu wait+stage", "gu gemv+epi",
         "down wait+stage", "down gemv+epi"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--cached", type=int, default=200, help="positions already in the KV cache")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--poll-words", type=int, default=-1, help="1: poll tagged words directly, 0: wait for arrival flags first")
    ap.add_argument("--chunks", type=int, default=0, help="attention chunks per kv head (0: the library's choice)")
    a = ap.parse_args()
    cfg = ModelArgs.from_name(a.config)
    W = packing.synth_packed(cfg, 0, device="cuda")
    eng = DecodeEngine(cfg, W, max_seq=max(cfg.block_size, a.cached + a.steps + 8))
    if a.chunks:
        eng.set_option(1, a.chunks)
    if a.poll_words >= 0:
        eng.set_option(5, a.poll_words)
    G = query(torch.cuda.current_device())["sm_count"]
    prof = torch.zeros(G * cfg.n_layer * 16, dtype=torch.int64, device="cuda")
    if a.cached > 2048:      # long contexts: seeded random keys and values instead of decoding every position
        eng.kc[:, :a.cached].normal_()
        eng.vc[:, :a.cached].normal_()
    else:
        for pos in range(a.cached):
            eng.decode(5 + pos, pos, want_logits=False)
    nxt = torch.zeros(a.steps + 1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        eng.decode_chained(nxt[i:i + 1], a.cached + i, nxt[i + 1:i + 2])
    e1.record()
    torch.cuda.synchronize()
    print(f"decode: {e0.elapsed_time(e1) / a.steps * 1e3:.1f} us/token over {a.steps} chained steps")
    eng.set_option(2, prof.data_ptr())
    eng.decode(77, a.cached + a.steps, want_logits=False)
    eng.check()
    p = prof.cpu().numpy().reshape(G, cfg.n_layer, 16).astype(np.float64)
    names = NAMES
    lo, hi = (1, cfg.n_layer - 1) if cfg.n_layer > 4 else (0, cfg.n_layer)
    d = np.diff(p[:, lo:hi, :len(names) + 1], axis=2) / 1e3
    print(f"{'phase':18s} {'mean':>7s} {'min':>7s} {'max':>7s}   (us per layer; mean/min/max over {G} CTAs)")
    for i, nm in enumerate(names):
        x = d[:, :, i].mean(1)
        print(f"{nm:18s} {x.mean():7.2f} {x.min():7.2f} {x.max():7.2f}")
    w = (p[:, lo:hi, 13] - p[:, lo:hi, 1]).mean() / 1e3
    t = (p[:, lo:hi, 14] - p[:, lo:hi, 13]).mean() / 1e3
    r = (p[:, lo:hi, 2] - p[:, lo:hi, 14]).mean() / 1e3
    print(f"qkv, warp 0: weights ready {w:.2f} us after staging, first tile product {t:.2f} us, rest of the phase {r:.2f} us")
    f = (p[:, lo:hi, 10] - p[:, lo:hi, 0]).mean() / 1e3
    g = (p[:, lo:hi, 11] - p[:, lo:hi, 10]).mean() / 1e3
    n = (p[:, lo:hi, 1] - p[:, lo:hi, 11]).mean() / 1e3
    print(f"qkv staging: flags seen after {f:.2f} us, gather {g:.2f} us, norm + convert {n:.2f} us")
    if hi - lo > 2:
        # the last CTA's down-phase flag post (stamp 12 of layer l) -> every CTA has seen all flags (stamp 10 of layer l+1)
        post = p[:, lo:hi - 1, 12].max(0)
        seen = p[:, lo + 1:hi, 10]
        print(f"flag hop: last post -> seen by a CTA: mean {(seen - post[None]).mean() / 1e3:.2f} us, "
              f"max {(seen - post[None]).max(0).mean() / 1e3:.2f} us")
    if hi - lo > 1:
        per = (p[:, lo + 1:hi, 0] - p[:, lo:hi - 1, 0]).mean() / 1e3
        print(f"layer period {per:.2f} us -> {per * cfg.n_layer / 1e3:.3f} ms for {cfg.n_layer} layers")


if __name__ == "__main__":
    main()
