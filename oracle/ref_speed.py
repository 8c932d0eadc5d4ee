"""Times the reference's own decode megakernel (built from the reference checkout into oracle/_ref by build_ref.py) on this
GPU at its native Granite shape (40 q / 8 kv heads of 64, vocab 100352), with seeded synthetic weights, the way its
speed test does (reference: bench/megakernel_decode_test.py:80-88), and this library at the same shape beside it.

    python oracle/ref_speed.py

Test infrastructure: measures the comparison row "reference megakernel on the same B200"; nothing in the product uses it.
"""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flint_b200 import packing
from flint_b200.config import ModelArgs
from flint_b200.engine import DecodeEngine
from oracle import build_ref
ref = build_ref.load_module("flint_ref_decode")
cfg = ModelArgs.from_name("granite-4.1-3b")
W = packing.synth_packed(cfg, 0, device="cuda")
MAXSEQ = 512
kc = torch.zeros(cfg.n_layer, MAXSEQ, 8, 64, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros_like(kc)
h = torch.randn(cfg.dim, device="cuda").bfloat16()
def launch(pos):
    return ref.decode_mega_launch(W["qkv_q"], W["qkv_s"], W["o_q"], W["o_s"], W["n1"], W["gu_q"], W["gu_s"], W["d_q"], W["d_s"], W["n2"], W["nf"], W["lm_q"], W["lm_s"], h.clone(), kc, vc, pos, cfg.attn_scale, float(cfg.rope_base), cfg.residual_multiplier, cfg.logits_scaling)
for p in range(136): launch(p)
torch.cuda.synchronize(); t0 = time.perf_counter()
for p in range(136, 136 + 64): launch(p).argmax()
torch.cuda.synchronize(); dt = (time.perf_counter() - t0) / 64
bt = cfg.bytes_per_token(0)
print(f"REFERENCE megakernel on this B200, native Granite shape: {1/dt:.1f} tok/s, {dt*1e6:.0f} us/token, MBU(weights) vs 8TB/s {bt/dt/8e12:.3f}; occupancy {ref.decode_occupancy()}")
eng = DecodeEngine(cfg, W, max_seq=MAXSEQ)
nxt = torch.zeros(300, dtype=torch.int32, device="cuda")
for p in range(136): eng.decode(5 + p, p, want_logits=False)
torch.cuda.synchronize(); e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True); e0.record()
for i in range(64): eng.decode_chained(nxt[i:i+1], 136 + i, nxt[i+1:i+2])
e1.record(); torch.cuda.synchronize(); dt2 = e0.elapsed_time(e1) / 64 / 1e3
print(f"OURS same shape: {1/dt2:.1f} tok/s, {dt2*1e6:.0f} us/token, MBU {bt/dt2/8e12:.3f}", eng.status()["code"])
