"""`generate()` with the reference engine's signature (reference: engine/generate.py:137-206), plus the tree loop.

Everything per token stays on the device:
  * greedy: step t+1 reads step t's arg-max from device memory (reference loop: chat.py:76-81,97-101);
  * temperature / top-k: the decode launch is followed by `fb_sample` on its logits, whose token the next launch reads —
    no host sync and no PyTorch kernels in the loop (the reference syncs per token, reference: engine/generate.py:52-66);
  * chain speculation (reference loop: spec_mega.py:89-117): the EAGLE draft head rolls out K tokens with the
    extension's draft kernels, the target scores K+1 candidates in one `fb_verify` pass, arg-max and the acceptance walk
    run on the device; the host reads 8 bytes per pass (accepted count, next token) to advance its position;
  * tree speculation (reference loop: spec_tree.py:53-130): a width-B beam to depth D, one tree-masked `fb_verify`,
    `fb_accept_tree` + `fb_kv_compact` on the device.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .model import Transformer


def _prefill(model: Transformer, prompt: torch.Tensor, temperature: float, top_k, seed: int):
    """Causal chunks of 64 through the verify path; returns (first new token on the device [1], features [T, dim])."""
    eng = model.engine
    T = prompt.numel()
    logits, feats = model(prompt.view(1, -1), torch.arange(T), return_hidden=True)
    first = eng.sample(logits[0, -1].contiguous(), temperature, top_k, seed, 0)
    return first, feats[0]


@torch.no_grad()
def generate(model: Transformer, prompt: torch.Tensor, max_new_tokens: int, *, interactive: bool = False,
             draft_model=None, speculate_k: Optional[int] = 8, callback=lambda x: x, temperature: float = 0.0,
             top_k: Optional[int] = None, seed: int = 0, window: int = 32):
    """Returns (sequence [T + max_new_tokens] int, {"accept_counts": [...]})."""
    T = prompt.numel()
    T_new = T + max_new_tokens
    is_spec = draft_model is not None
    K = int(speculate_k or 0) if is_spec else 0
    max_seq = min(T_new, model.config.block_size) + (K + 1 if is_spec else 0)
    model.setup_caches(max_batch_size=1, max_seq_length=max_seq)
    eng = model.engine
    dev = eng.device
    seq = torch.empty(T_new + K + 1, dtype=torch.int32, device=dev)
    seq[:T] = prompt.to(dev)
    accept_counts = [0] * (K + 1)
    first, feats = _prefill(model, prompt, temperature, top_k, seed)
    seq[T:T + 1] = first
    if not is_spec:
        greedy = temperature <= 0
        lg = None if greedy else torch.empty(model.config.vocab_size, dtype=torch.float32, device=dev)
        for i in range(T, T_new - 1):                      # chained on the device: no host sync in the loop
            if greedy:
                eng.decode_chained(seq[i:i + 1], i, seq[i + 1:i + 2])
            else:
                eng.decode_chained(seq[i:i + 1], i, eng.next_token, lg)
                eng.sample(lg, temperature, top_k, seed, i - T + 1, out=seq[i + 1:i + 2])
        eng.check()
        for i in range(T, T_new):
            callback(seq[i])
        return seq[:T_new], {"accept_counts": accept_counts}

    # ---- chain speculative decoding with an EAGLE draft head (greedy acceptance) ----
    if temperature > 0:
        raise ValueError("speculative decoding accepts greedily: temperature must be 0")
    P = model.packed
    draft_model.bind_target(P["embed"], P["nf"], model.config.logits_scaling)
    W = int(window)
    draft_model.setup_cache(W + K + 2)
    fdim = draft_model.fdim
    gfeat = torch.zeros(W, fdim, dtype=torch.bfloat16, device=dev)
    gtok = torch.full((W,), -1, dtype=torch.int32, device=dev)       # context embeddings are zero rows, the last one the
    gpos = torch.arange(W, dtype=torch.int32, device=dev)            # newest token's (reference: spec_mega.py:98-99)
    step_pos = [torch.tensor([W + i], dtype=torch.int32, device=dev) for i in range(K)]
    cand = torch.zeros(K + 1, dtype=torch.int32, device=dev)
    tgt = torch.zeros(K + 1, dtype=torch.int32, device=dev)
    acc_dev = torch.zeros(2, dtype=torch.int32, device=dev)
    acc_host = torch.zeros(2, dtype=torch.int32).pin_memory()
    n, pos = T + 1, T
    nxt = seq[T:T + 1]
    while n < T_new:
        # window of the last W features, front-padded with the oldest one (reference: spec_mega.py:93-97)
        N = feats.shape[0]
        if N >= W:
            gfeat.copy_(feats[N - W:])
        else:
            gfeat[W - N:].copy_(feats)
            gfeat[:W - N].copy_(feats[0:1].expand(W - N, -1))
        gtok[W - 1:W].copy_(nxt)
        cand[0:1].copy_(nxt)
        fp = draft_model(gfeat, None, gpos, input_pos=gpos, tokens=gtok)
        f_new = fp[W - 1:W]
        t_new = draft_model.head(f_new).view(1)
        cand[1:2].copy_(t_new)
        for i in range(K - 1):
            fp = draft_model(f_new, None, step_pos[i], input_pos=step_pos[i], tokens=t_new)
            f_new = fp[0:1]
            t_new = draft_model.head(f_new).view(1)
            cand[2 + i:3 + i].copy_(t_new)
        vlog, vfeat = eng.verify(cand, pos)                 # chain mask, depth = index
        eng.sample(vlog, 0.0, out=tgt)                      # the target's greedy token at every candidate position
        eng.accept_chain(tgt, cand[1:], out=acc_dev)
        acc_host.copy_(acc_dev, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()        # the one host read of the pass: 8 bytes
        acc, nx = int(acc_host[0]), int(acc_host[1])
        accept_counts[acc] += 1
        take = min(acc + 1, T_new - n)
        seq[n:n + acc].copy_(cand[1:1 + acc])
        seq[n + acc] = nx
        for j in range(take):
            callback(seq[n + j])
        feats = torch.cat([feats, vfeat[:acc + 1]])
        n += acc + 1
        pos += 1 + acc
        nxt = seq[n - 1:n]
    eng.check()
    return seq[:T_new], {"accept_counts": accept_counts}


@torch.no_grad()
def generate_tree(model: Transformer, prompt: torch.Tensor, max_new_tokens: int, draft_model, *, beam: int = 2, depth: int = 6,
                  window: int = 32, callback=lambda x: x):
    """Tree speculative decoding (reference: spec_tree.py:53-130): the draft rolls a width-`beam` beam to `depth`; the
    target scores the whole tree in one tree-masked verify pass; the longest path the target's greedy choices agree with
    is accepted and its cache rows are compacted. Returns (sequence, {"passes", "tokens_per_pass", "tree_nodes"})."""
    cfg = model.config
    T = prompt.numel()
    T_new = T + max_new_tokens
    M = 1 + beam * depth
    model.setup_caches(max_batch_size=1, max_seq_length=min(T_new, cfg.block_size) + M + depth + 2)
    eng = model.engine
    dev = eng.device
    P = model.packed
    draft_model.bind_target(P["embed"], P["nf"], cfg.logits_scaling)
    draft_model.setup_cache(window + depth + 2)
    first, feats = _prefill(model, prompt, 0.0, None, 0)
    out: List[int] = prompt.tolist()
    nxt, pos, passes = int(first.item()), T, 0
    tgt = torch.zeros(M, dtype=torch.int32, device=dev)
    acc_dev = torch.zeros(2 + M, dtype=torch.int32, device=dev)
    while len(out) < T_new:
        out.append(nxt)
        callback(nxt)
        if len(out) >= T_new:
            break
        # ---- beam draft: every node is one full-window forward over context + its own history (reference: spec_tree.py:56-83)
        fctx = feats[-window:]
        Wc = fctx.shape[0]

        def fwd(hist_f, hist_t):
            rows = torch.cat([fctx] + ([torch.stack(hist_f)] if hist_f else []))
            toks = torch.zeros(rows.shape[0], dtype=torch.int32, device=dev)     # context rows carry token 0's embedding
            toks[Wc - 1] = nxt
            for i, t in enumerate(hist_t):
                toks[Wc + i] = t
            posn = torch.arange(pos - Wc, pos - Wc + rows.shape[0], dtype=torch.int32, device=dev)
            return draft_model(rows, None, posn, tokens=toks)[-1]

        tok_a, dep_a, par_a = [], [], []
        f0 = fwd([], [])
        ti, tv = draft_model.head(f0.view(1, -1), top_b=beam, want_scores=True)
        ti, tv = ti[0].tolist(), tv[0].tolist()
        beams = []
        for b in range(beam):
            tok_a.append(ti[b]); dep_a.append(1); par_a.append(-1)
            beams.append(dict(lp=tv[b], node=len(tok_a) - 1, hist_f=[f0], hist_t=[ti[b]]))
        for d in range(2, depth + 1):
            fns = [fwd(bm["hist_f"], bm["hist_t"]) for bm in beams]
            ti, tv = draft_model.head(torch.stack(fns), top_b=beam, want_scores=True)
            ti, tv = ti.tolist(), tv.tolist()                                    # one host read per depth
            cands = [(bm["lp"] + tv[k][b], k, ti[k][b]) for k, bm in enumerate(beams) for b in range(beam)]
            cands.sort(key=lambda x: -x[0])
            nb = []
            for lp, k, t in cands[:beam]:
                bm = beams[k]
                tok_a.append(t); dep_a.append(d); par_a.append(bm["node"])
                nb.append(dict(lp=lp, node=len(tok_a) - 1, hist_f=bm["hist_f"] + [fns[k]], hist_t=bm["hist_t"] + [t]))
            beams = nb
        cand = [nxt] + tok_a
        dpt = [0] + dep_a
        cpar = [-1] + [0 if p == -1 else 1 + p for p in par_a]
        from .tree import tree_mask
        amask = torch.from_numpy(tree_mask(cpar)).to(dev)
        cand_d = torch.tensor(cand, dtype=torch.int32, device=dev)
        par_d = torch.tensor(cpar, dtype=torch.int32, device=dev)
        vlog, vfeat = eng.verify(cand_d, pos, torch.tensor(dpt, dtype=torch.int32, device=dev), amask)
        eng.sample(vlog, 0.0, out=tgt[:len(cand)])
        eng.accept_tree(cand_d, par_d, tgt[:len(cand)], out=acc_dev)
        eng.kv_compact(acc_dev, pos)                          # accepted rows become contiguous, on the device
        res = acc_dev.tolist()                                # the one host read of the verify side
        L, nx, path = res[0], res[1], res[2:2 + res[0]]
        for step in range(1, L):
            if len(out) < T_new:
                out.append(cand[path[step]])
                callback(cand[path[step]])
        feats = torch.cat([feats, vfeat[torch.tensor(path, device=dev)]])
        pos += L
        nxt = nx
        passes += 1
    eng.check()
    seq = torch.tensor(out[:T_new], dtype=torch.int32, device=dev)
    return seq, {"passes": passes, "tokens_per_pass": (len(out) - T) / max(passes, 1), "tree_nodes": M}
