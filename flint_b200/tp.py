"""Tensor parallelism of the decode path over 2/4/8 GPUs of one box: host side.

Megatron-style sharding of every int4 matrix: QKV by heads (rows), O by this rank's heads (columns = K), gate/up by
FFN rows, down by FFN columns (K), LM head by vocabulary rows; norms and the embedding table are replicated. Where a
rank's attention width is not a multiple of the int4 group (the 3B-class model over 8 ranks: 320 columns), its O slice
is widened to the enclosing group boundaries and the kernel feeds zeros for the neighbour's columns (`o_window`). The two
K-sharded projections leave partial sums that the kernel exchanges itself (peer stores into every rank's inbox,
tagged words, summed in rank order so every rank holds bit-identical residuals); this module only slices the packed
tensors, creates one engine per process and passes the IPC handles of the inboxes around once, through
torch.distributed. The reference has no counterpart (it imports a `tp` module that its repository does not contain,
reference: engine/generate.py:238-241); the check is TP-N == TP-1.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .config import GROUP, ModelArgs


def _rows(t: torch.Tensor, a: int, b: int) -> torch.Tensor:
    return t[..., a:b, :]


def o_window(cfg: ModelArgs, rank: int, size: int):
    """Columns of the O projection rank `rank` reads: its heads' columns widened to whole int4 groups.

    Returns (lo, hi, off): the rank holds columns [lo, hi) of every O row and its own attention output starts `off`
    columns into that window; the kernel feeds zeros for the columns of the window that belong to a neighbour, so no
    weight is re-quantised and every rank's dequantised values stay bit-exact. For shapes whose per-rank width is a
    multiple of 128 the window is exactly the rank's columns (off = 0)."""
    w = (cfg.n_head // size) * cfg.head_dim
    start = rank * w
    lo = start // GROUP * GROUP
    hi = (start + w + GROUP - 1) // GROUP * GROUP
    return lo, hi, start - lo


def can_shard(cfg: ModelArgs, size: int) -> bool:
    nh, nkv, f, v = cfg.n_head, cfg.n_local_heads, cfg.ffn_padded, cfg.vocab_size
    if size == 1:
        return True
    if nh % size or nkv % size or (f // GROUP) % size or v % size:
        return False
    widths = {o_window(cfg, r, size)[1] - o_window(cfg, r, size)[0] for r in range(size)}
    return len(widths) == 1                                    # one kernel shape for every rank


def max_tp(cfg: ModelArgs, world: int) -> int:
    """Largest tensor-parallel degree <= world (a power-of-two divisor of it) this model splits into."""
    tp = world
    while tp > 1 and (world % tp or not can_shard(cfg, tp)):
        tp //= 2
    return max(tp, 1)


def shard_packed(P: Dict[str, torch.Tensor], cfg: ModelArgs, rank: int, size: int) -> Dict[str, torch.Tensor]:
    """This rank's slice of a packed model (the dict `pack_model` / `synth_packed` return)."""
    hd, nh, nkv, f, v = cfg.head_dim, cfg.n_head, cfg.n_local_heads, cfg.ffn_padded, cfg.vocab_size
    if not can_shard(cfg, size):
        raise ValueError(f"model does not shard over {size} ranks with whole int4 groups")
    nhl, nkvl, fl, vl = nh // size, nkv // size, f // size, v // size
    qd, kvd = nh * hd, nkv * hd
    lo, hi, _ = o_window(cfg, rank, size)
    out: Dict[str, torch.Tensor] = {}
    for suf in ("q", "s", "z"):
        if f"qkv_{suf}" not in P:
            continue
        per = 8 if suf == "q" else GROUP                       # columns per stored element along K
        t = P[f"qkv_{suf}"]
        out[f"qkv_{suf}"] = torch.cat([_rows(t, rank * nhl * hd, (rank + 1) * nhl * hd),
                                       _rows(t, qd + rank * nkvl * hd, qd + (rank + 1) * nkvl * hd),
                                       _rows(t, qd + kvd + rank * nkvl * hd, qd + kvd + (rank + 1) * nkvl * hd)], -2).contiguous()
        out[f"o_{suf}"] = P[f"o_{suf}"][..., lo // per:hi // per].contiguous()
        t = P[f"gu_{suf}"]
        out[f"gu_{suf}"] = torch.cat([_rows(t, rank * fl, (rank + 1) * fl), _rows(t, f + rank * fl, f + (rank + 1) * fl)],
                                     -2).contiguous()
        out[f"d_{suf}"] = P[f"d_{suf}"][..., rank * fl // per:(rank + 1) * fl // per].contiguous()
        out[f"lm_{suf}"] = P[f"lm_{suf}"][rank * vl:(rank + 1) * vl].contiguous()
    for k in ("n1", "n2", "nf", "embed"):
        out[k] = P[k]
    return out


def make_tp_engine(cfg: ModelArgs, packed_full: Dict[str, torch.Tensor], max_seq: int, group=None,
                   device: Optional[torch.device] = None):
    """One engine per process (rank = torch.distributed rank of `group`); exchanges the inbox handles once."""
    import torch.distributed as dist
    from .engine import DecodeEngine
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    local = shard_packed(packed_full, cfg, rank, size)
    eng = DecodeEngine(cfg, local, max_seq=max_seq, device=device, tp_rank=rank, tp_size=size)
    handles = [None] * size
    dist.all_gather_object(handles, eng.tp_export(), group=group)
    eng.tp_connect(handles)
    dist.barrier(group)
    return eng
