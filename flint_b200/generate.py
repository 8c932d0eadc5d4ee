"""`generate()` with the reference engine's signature (reference: engine/generate.py:137-206).

Greedy decoding (temperature 0, the megakernel path's mode, reference: chat.py:76-77) keeps the token chain on the
device: step t+1 reads step t's arg-max from device memory, the host never synchronises inside the loop. Sampling
(temperature > 0, top-k) follows the reference's `sample()` (reference: engine/generate.py:38-55) on the logits the
kernel returns. Speculative decoding takes an EAGLE draft head (flint_b200.draft.DraftHead) and verifies K+1 tokens
per pass on the verify path (reference loop: spec_mega.py:89-117).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .draft import rmsnorm
from .model import Transformer
from .tree import chain_accept


def multinomial_sample_one_no_sync(probs_sort):
    q = torch.empty_like(probs_sort).exponential_(1)
    return torch.argmax(probs_sort / q, dim=-1, keepdim=True).to(dtype=torch.int)


def logits_to_probs(logits, temperature: float = 1.0, top_k: Optional[int] = None):
    logits = logits / max(temperature, 1e-5)
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = torch.where(logits < v.select(-1, -1).unsqueeze(-1), -float("Inf"), logits)
    return torch.nn.functional.softmax(logits, dim=-1)


def sample(logits, temperature: float = 1.0, top_k: Optional[int] = None):
    probs = logits_to_probs(logits[0, -1], temperature, top_k)
    return multinomial_sample_one_no_sync(probs), probs


@torch.no_grad()
def generate(model: Transformer, prompt: torch.Tensor, max_new_tokens: int, *, interactive: bool = False,
             draft_model=None, speculate_k: Optional[int] = 8, callback=lambda x: x, temperature: float = 0.0,
             top_k: Optional[int] = None):
    """Returns (sequence [T + max_new_tokens] int, {"accept_counts": [...]})."""
    T = prompt.numel()
    T_new = T + max_new_tokens
    is_spec = draft_model is not None
    max_seq = min(T_new, model.config.block_size) + (speculate_k + 1 if is_spec else 0)
    model.setup_caches(max_batch_size=1, max_seq_length=max_seq)
    eng = model.engine
    dev = eng.device
    seq = torch.empty(T_new, dtype=torch.int32, device=dev)
    seq[:T] = prompt.to(dev)
    accept_counts = [0] * ((speculate_k or 0) + 1)
    greedy = temperature <= 0
    # ---- prefill: causal chunks of 64 through the verify path; the last chunk's last row gives the first new token
    logits, feats = model(prompt.view(1, -1), torch.arange(T), return_hidden=True)
    first = logits[0, -1].argmax().to(torch.int32) if greedy else sample(logits, temperature, top_k)[0].view(())
    seq[T] = first
    callback(first)
    if not is_spec:
        pos = T
        if greedy:
            for i in range(T, T_new - 1):                       # chained on the device: no host sync in the loop
                eng.decode_chained(seq[i:i + 1], pos, seq[i + 1:i + 2])
                pos += 1
            eng.check()
            for i in range(T + 1, T_new):
                callback(seq[i])
        else:
            for i in range(T, T_new - 1):
                lg = model(seq[i].view(1, 1), torch.tensor([pos]))
                seq[i + 1] = sample(lg, temperature, top_k)[0].view(())
                callback(seq[i + 1])
                pos += 1
        return seq, {"accept_counts": accept_counts}
    # ---- chain speculative decoding with an EAGLE draft head (greedy acceptance) ----
    P = model.packed
    embed, nf = P["embed"], P["nf"]
    cfg = model.config
    K = speculate_k

    def head_tok(f):                                            # feature -> token (reference: spec_mega.py:43-44)
        return (F.linear(rmsnorm(f.float(), nf.float()), embed.float()) / cfg.logits_scaling).argmax(-1)

    ctx_f = feats[0]                                            # [T, dim] features of the prompt positions
    n, pos, nxt = T + 1, T, first.view(1)
    while n < T_new:
        # draft K tokens from the feature window (full-window forward per step, as the reference's eager path does)
        hist_f, hist_t, d = ctx_f[-32:], [], []
        emb_ctx = torch.zeros(hist_f.shape[0], cfg.dim, dtype=torch.bfloat16, device=dev)
        emb_ctx[-1] = (embed[int(nxt)].float() * cfg.embedding_multiplier).to(torch.bfloat16)
        cur_f, cur_e = hist_f, emb_ctx
        for _ in range(K):
            base = pos - cur_f.shape[0] + 1
            fp = draft_model(cur_f.unsqueeze(0), cur_e.unsqueeze(0), torch.arange(base, base + cur_f.shape[0], device=dev))
            f_new = fp[0, -1, -cfg.dim:]
            t_new = int(head_tok(f_new))
            d.append(t_new)
            cur_f = torch.cat([cur_f, f_new.unsqueeze(0)])
            cur_e = torch.cat([cur_e, (embed[t_new].float() * cfg.embedding_multiplier).to(torch.bfloat16).unsqueeze(0)])
            pos += 0
        cand = torch.tensor([int(nxt)] + d, dtype=torch.int32, device=dev)
        vlog, vfeat = eng.verify(cand, pos)                     # chain mask, depth = index
        tgt = vlog.argmax(-1).tolist()
        acc = chain_accept(tgt, d)
        accept_counts[acc] += 1
        new = d[:acc] + [tgt[acc]]
        take = min(len(new), T_new - n)
        seq[n:n + take] = torch.tensor(new[:take], dtype=torch.int32, device=dev)
        for t in new[:take]:
            callback(torch.tensor(t))
        ctx_f = torch.cat([ctx_f, vfeat[:acc + 1]])
        n += take
        pos += 1 + acc
        nxt = torch.tensor([tgt[acc]], device=dev)
    return seq, {"accept_counts": accept_counts}
