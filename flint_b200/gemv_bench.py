"""Stand-alone int4 GEMV bandwidth probe on the streaming layout (the unit-test slice of the decode path).

    python -m flint_b200.gemv_bench --rows 400000 --k 2560 --iters 5

Prints one line per iteration: device time (CUDA events) and bytes of weight tiles streamed per second.
Also the small, self-contained launch that the ncu captures under profiles/ are taken from.
"""
import argparse
import ctypes

import torch

from . import _lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=400000)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--zeros", action="store_true")
    a = ap.parse_args()
    lib = _lib.load()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randint(-2 ** 31, 2 ** 31 - 1, (a.rows, a.k // 8), generator=g, device="cuda", dtype=torch.int64).to(torch.int32)
    s = (torch.rand(a.rows, a.k // 128, generator=g, device="cuda") * 0.01).bfloat16()
    z = (torch.rand(a.rows, a.k // 128, generator=g, device="cuda") * 0.01).bfloat16() if a.zeros else None
    x = torch.randn(a.k, generator=g, device="cuda").bfloat16()
    nb = lib.fb_stream_bytes(a.rows, a.k, int(a.zeros))
    st = torch.empty(nb + 16, dtype=torch.uint8, device="cuda")
    _lib.check(lib.fb_repack(P(q), P(s), P(z) if z is not None else None, a.rows, a.k, 0, 0, 0, P(st), None), "fb_repack")
    del q
    y = torch.zeros(a.rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    for it in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(lib.fb_gemv(P(st), a.rows, a.k, int(a.zeros), 0, 0, 0, P(x), P(y), P(status), None), "fb_gemv")
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        print(f"iter {it}: {ms * 1e3:.1f} us  {nb / ms / 1e6:.0f} GB/s  ({nb / 1e6:.0f} MB of tiles, status {int(status[0])})")


if __name__ == "__main__":
    main()
