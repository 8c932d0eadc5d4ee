"""What the tensor-parallel exchange of one decode step would cost as NCCL calls between kernels.

The decode megakernel exchanges the partial sums of the O and the down projection inside the kernel (peer stores over
NVLink, polled in local memory): 2 exchanges per layer, no launch. The conventional alternative is one NCCL all-reduce of
`dim` fp32 values after each of the two projections, i.e. 2 x n_layer collectives per token between 2 x n_layer + 1 kernel
launches. This script times exactly that sequence of collectives (nothing else: no GEMV, no attention), eagerly and
replayed from a CUDA graph, so the number is a LOWER bound of what a launch-per-phase design pays per token on top of
its compute. Run under torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 -m flint_b200.tp_exchange_bench

Prints one JSON line on rank 0: ms per token of the collectives alone, max over ranks, CUDA-event timed.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .config import ModelArgs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--graph", action="store_true", help="also time the sequence replayed from a CUDA graph")
    a = ap.parse_args()
    cfg = ModelArgs.from_name(a.config)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))

    def say(msg):
        if rank == 0:
            print(f"# {msg}", flush=True)
    x = torch.zeros(cfg.dim, dtype=torch.float32, device=dev)
    n = 2 * cfg.n_layer

    def token():
        for _ in range(n):
            dist.all_reduce(x)

    say("process group up")
    for _ in range(5):
        token()
    torch.cuda.synchronize()
    say("warm-up done")

    def timed(fn) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    eager_ms = timed(token)
    say(f"eager {eager_ms:.3f} ms per token")
    graph_ms = None
    if a.graph:
      try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            token()
        torch.cuda.synchronize()
        graph_ms = timed(g.replay)
      except Exception as e:  # the eager figure stands alone where NCCL cannot be captured
        graph_ms = None
        say(f"graph capture unavailable: {type(e).__name__}")
    if rank == 0:
        print(json.dumps({"what": "NCCL all-reduce x (2 x n_layer) per token, collectives only", "config": a.config, "world": world,
                          "collectives_per_token": n, "floats_per_collective": cfg.dim, "eager_ms_per_token": eager_ms,
                          "graph_ms_per_token": graph_ms}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
