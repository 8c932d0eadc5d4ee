"""Tensor parallelism of the decode path over 2/4/8 GPUs of one box: host side.

Megatron-style sharding of every int4 matrix: QKV by heads (rows), O by this rank's heads (columns = K), gate/up by
FFN rows, down by FFN columns (K), LM head by vocabulary rows; norms and the embedding table are replicated. The two
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


def shard_packed(P: Dict[str, torch.Tensor], cfg: ModelArgs, rank: int, size: int) -> Dict[str, torch.Tensor]:
    """This rank's slice of a packed model (the dict `pack_model` / `synth_packed` return)."""
    hd, nh, nkv, f, v = cfg.head_dim, cfg.n_head, cfg.n_local_heads, cfg.ffn_padded, cfg.vocab_size
    if nh % size or nkv % size or (f // GROUP) % size or v % size or ((nh // size) * hd) % GROUP:
        raise ValueError(f"model does not shard over {size} ranks with whole int4 groups")
    nhl, nkvl, fl, vl = nh // size, nkv // size, f // size, v // size
    qd, kvd = nh * hd, nkv * hd
    out: Dict[str, torch.Tensor] = {}
    for suf in ("q", "s", "z"):
        if f"qkv_{suf}" not in P:
            continue
        per = 8 if suf == "q" else GROUP                       # columns per stored element along K
        t = P[f"qkv_{suf}"]
        out[f"qkv_{suf}"] = torch.cat([_rows(t, rank * nhl * hd, (rank + 1) * nhl * hd),
                                       _rows(t, qd + rank * nkvl * hd, qd + (rank + 1) * nkvl * hd),
                                       _rows(t, qd + kvd + rank * nkvl * hd, qd + kvd + (rank + 1) * nkvl * hd)], -2).contiguous()
        ko = nhl * hd
        out[f"o_{suf}"] = P[f"o_{suf}"][..., rank * ko // per:(rank + 1) * ko // per].contiguous()
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
