"""Device time of one M-token tree verify on a synthetic int4 model (the speculative-decoding sibling of the decode path).

    python -m flint_b200.verify_bench --config granite-3b-class --m 16 --prompt-len 1024

Prints one line per tree size: CUDA-event time of a verify replayed from a CUDA graph (launch gaps removed), the same
launched eagerly, the weight bytes streamed per second and the multiply-add rate. `--no-graph --warmup 1 --iters 1` is
the short form that a launch-list capture wraps.
"""
import argparse

import torch

from . import packing
from .config import ModelArgs
from .engine import DecodeEngine
from .tree import static_tree, tree_mask


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--m", type=int, nargs="+", default=[1, 16, 26, 64])
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--path", type=int, default=0, help="GEMM implementation (fb_set_option 7): 0 by tree size, 1 warp-level bf16, 2 tcgen05, 3 tcgen05 chains, 4 warp-level fp16 subnormals")
    a = ap.parse_args()
    cfg = ModelArgs.from_name(a.config)
    W = packing.synth_packed(cfg, 0, device="cuda")
    eng = DecodeEngine(cfg, W, max_seq=a.prompt_len + 128)
    eng.set_option(7, a.path)
    eng.kc[:, :a.prompt_len].normal_()
    eng.vc[:, :a.prompt_len].normal_()
    bt = cfg.bytes_per_token(a.prompt_len)
    for M in a.m:
        parent, depth = static_tree(M)
        am = torch.from_numpy(tree_mask(parent)).cuda()
        dp = torch.tensor(depth, dtype=torch.int32, device="cuda")
        toks = torch.randint(0, cfg.vocab_size, (M,), device="cuda", dtype=torch.int32)
        for _ in range(a.warmup):
            eng.verify(toks, a.prompt_len, dp, am)
        torch.cuda.synchronize()

        def timed(fn):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)

        eager = min(timed(lambda: eng.verify(toks, a.prompt_len, dp, am)) for _ in range(a.iters))
        line = f"verify M={M}: eager {eager * 1e3:.0f} us"
        if not a.no_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                eng.verify(toks, a.prompt_len, dp, am)
            t = min(timed(g.replay) for _ in range(a.iters))
            line += (f"; graph {t * 1e3:.0f} us ({bt / t / 1e6:.0f} GB/s of weights+cache, "
                     f"{2 * M * cfg.int4_params() / t / 1e9:.1f} TFLOP/s)")
        eng.check()
        print(line)


if __name__ == "__main__":
    main()
