"""CPU, world_size 2 over gloo: the host side of the tensor-parallel path (slicing + what the exchange must add up to)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flint_b200 import packing
from flint_b200.config import ModelArgs
from flint_b200.tp import shard_packed
from oracle import oracle as O


def _cfg():
    # small shape whose slices keep whole int4 groups: 8 q / 2 kv heads of 64, FFN 1536, vocab 1024
    return ModelArgs(block_size=32, vocab_size=1024, n_layer=2, n_head=8, n_local_heads=2, dim=512, intermediate_size=1536)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    P = packing.synth_packed(cfg, 0)
    S = shard_packed(P, cfg, rank, world)
    g = torch.Generator().manual_seed(1)
    ao = torch.randn(cfg.dim, generator=g).bfloat16()
    act = torch.randn(cfg.ffn_padded, generator=g).bfloat16()
    xn = torch.randn(cfg.dim, generator=g).bfloat16()
    ko, fl = cfg.dim // world, cfg.ffn_padded // world
    # K-sharded projections: the partial sums of the ranks add up to the full product (what the in-kernel exchange sums)
    for name, x, k in (("o", ao, ko), ("d", act, fl)):
        part = torch.from_numpy(O.c_gemv(S[f"{name}_q"][0], S[f"{name}_s"][0], None, x[rank * k:(rank + 1) * k])[0])
        dist.all_reduce(part)
        full = O.c_gemv(P[f"{name}_q"][0], P[f"{name}_s"][0], None, x)[0]
        assert np.abs(part.numpy() - full).max() < 1e-4 * (np.abs(full).max() + 1)
    # row-sharded projections: the ranks' outputs concatenate to the full product, in head / FFN / vocabulary order
    y = torch.from_numpy(O.c_gemv(S["lm_q"], S["lm_s"], None, xn)[0])
    got = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(got, y)
    assert np.array_equal(torch.cat(got).numpy(), O.c_gemv(P["lm_q"], P["lm_s"], None, xn)[0])
    hd, nhl, nkvl = cfg.head_dim, cfg.n_head // world, cfg.n_local_heads // world
    yq = O.c_gemv(S["qkv_q"][1], S["qkv_s"][1], None, xn)[0]
    fullq = O.c_gemv(P["qkv_q"][1], P["qkv_s"][1], None, xn)[0]
    qd, kvd = cfg.n_head * hd, cfg.n_local_heads * hd
    assert np.array_equal(yq[:nhl * hd], fullq[rank * nhl * hd:(rank + 1) * nhl * hd])
    assert np.array_equal(yq[nhl * hd:(nhl + nkvl) * hd], fullq[qd + rank * nkvl * hd:qd + (rank + 1) * nkvl * hd])
    assert np.array_equal(yq[(nhl + nkvl) * hd:], fullq[qd + kvd + rank * nkvl * hd:qd + kvd + (rank + 1) * nkvl * hd])
    yg = O.c_gemv(S["gu_q"][0], S["gu_s"][0], None, xn)[0]
    fullg = O.c_gemv(P["gu_q"][0], P["gu_s"][0], None, xn)[0]
    f = cfg.ffn_padded
    assert np.array_equal(yg[:fl], fullg[rank * fl:(rank + 1) * fl]) and np.array_equal(yg[fl:], fullg[f + rank * fl:f + (rank + 1) * fl])
    ret[rank] = 1
    dist.destroy_process_group()


def test_shards_reassemble_over_gloo_world2():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: 1, 1: 1}


def test_shard_rejects_split_groups():
    import pytest
    cfg = ModelArgs.from_name("tiny")                 # FFN 1408 = 11 groups: no even split
    with pytest.raises(ValueError):
        shard_packed(packing.synth_packed(cfg, 0), cfg, 0, 2)


def test_o_window_widens_to_whole_groups_and_partials_add_up():
    """A rank whose attention width is not a multiple of the int4 group (320 columns: the 3B-class model over 8 ranks, or
    the small `tiny-window` model over 2) reads its columns widened to the enclosing groups and feeds zeros for the
    neighbour's: the ranks' partial sums still add up to the full product, with the original weights."""
    from flint_b200.tp import can_shard, max_tp, o_window
    big = ModelArgs.from_name("granite-3b-class")
    assert max_tp(big, 8) == 8 and [o_window(big, r, 8) for r in (0, 1, 7)] == [(0, 384, 0), (256, 640, 64), (2176, 2560, 64)]
    assert all(o_window(big, r, 4) == (640 * r, 640 * r + 640, 0) for r in range(4))
    cfg = ModelArgs.from_name("tiny-window")
    assert can_shard(cfg, 2) and [o_window(cfg, r, 2) for r in (0, 1)] == [(0, 384, 0), (256, 640, 64)]
    P = packing.synth_packed(cfg, 0)
    ao = torch.randn(cfg.dim, generator=torch.Generator().manual_seed(3)).bfloat16()
    full = O.c_gemv(P["o_q"][0], P["o_s"][0], None, ao)[0]
    tot = np.zeros_like(full)
    for r in range(2):
        S = shard_packed(P, cfg, r, 2)
        lo, hi, off = o_window(cfg, r, 2)
        assert S["o_q"].shape[-1] * 8 == hi - lo == 384
        x = torch.zeros(hi - lo, dtype=torch.bfloat16)
        x[off:off + 320] = ao[320 * r:320 * r + 320]          # the rank's own attention output; zeros elsewhere
        tot += O.c_gemv(S["o_q"][0], S["o_s"][0], None, x)[0]
    assert np.abs(tot - full).max() < 1e-4 * (np.abs(full).max() + 1)
