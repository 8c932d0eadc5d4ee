#!/usr/bin/env python3
"""Generate the committed golden fixtures by IMPORTING the reference's own Python code.

Run where the reference checkout is readable (its path is the first argument, or $FLINT_REFERENCE):

    python tests/golden/make_golden.py /path/to/flint

It writes, next to this script:
  packer_sym.npz   chat.qpc on a seeded bf16 matrix (incl. an all-zero group and saturating values)
  packer_asym.npz  engine/quantize.py group_quantize_tensor + group_dequantize_tensor on the same matrix
  engine_tiny.npz  engine/model.py Transformer (bf16, CPU) on the tiny config with the fake-quantised
                   seeded weights: 16-token prompt, 64 greedy steps, logits of selected steps
  draft_tiny.npz   train/draft_model.py DraftHead forward on seeded inputs (shape/semantics anchor)

The fixtures are the outputs of the reference; the tests compare this repository's packers and the CPU
oracle with them. Nothing at test time reads the reference checkout.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flint_b200.config import ModelArgs  # noqa: E402
from flint_b200 import packing  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLINT_REFERENCE")
    if not ref or not os.path.isdir(ref):
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference   (or set FLINT_REFERENCE)")
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ref, "engine"))
    sys.path.insert(0, os.path.join(ref, "train"))
    torch.set_grad_enabled(False)
    argv, sys.argv = sys.argv, ["x"]
    import chat as ref_chat                      # reference: chat.py
    import quantize as ref_quant                 # reference: engine/quantize.py
    import model as ref_model                    # reference: engine/model.py
    import draft_model as ref_draft              # reference: train/draft_model.py
    sys.argv = argv

    # ---------------------------------------------------------------- packers
    g = torch.Generator().manual_seed(11)
    W = (torch.randn(24, 384, generator=g) * 0.02).to(torch.bfloat16)
    W[3, 128:256] = 0                            # all-zero group
    W[5, :128] = 0
    W[5, 7] = 0.5                                # one dominant value: everything else rounds to 0
    W[7, 256:] = W[7, 256:].abs()                # one-signed group (matters for the asymmetric packer)
    W[9, 0:128] = 1e-30                          # denormal-scale group
    q, s = ref_chat.qpc(W)
    np.savez_compressed(os.path.join(HERE, "packer_sym.npz"), W=bits(W), q=q.numpy(), s=bits(s))

    w_int32, sz = ref_quant.group_quantize_tensor(W, n_bit=4, groupsize=128)
    scales = sz.transpose(0, 1)[..., 0].contiguous()
    zeros = sz.transpose(0, 1)[..., 1].contiguous()
    dq = ref_quant.group_dequantize_tensor_from_qparams(w_int32, scales.float(), zeros.float(), 4, 128)
    np.savez_compressed(os.path.join(HERE, "packer_asym.npz"), W=bits(W), w_int32=w_int32.numpy().astype(np.uint8),
                        scales_and_zeros=bits(sz), dequant_f32=dq.float().numpy())

    # ---------------------------------------------------------------- engine on the tiny config
    cfg = ModelArgs.from_name("tiny")
    w = packing.synth_weights(cfg, seed=0, device="cpu")
    P = packing.pack_model(w, cfg)
    margs = ref_model.ModelArgs(block_size=cfg.block_size, vocab_size=cfg.vocab_size, n_layer=cfg.n_layer,
                                n_head=cfg.n_head, dim=cfg.dim, intermediate_size=cfg.intermediate_size,
                                n_local_heads=cfg.n_local_heads, rope_base=cfg.rope_base, norm_eps=cfg.norm_eps)
    m = ref_model.Transformer(margs).to(torch.bfloat16)
    hd, d, f = cfg.head_dim, cfg.dim, cfg.intermediate_size

    def permute(wm, n_head):                     # reference: engine/scripts/convert_hf_checkpoint.py:75-81
        return wm.view(n_head, 2, hd // 2, d).transpose(1, 2).reshape(hd * n_head, d)

    def fq(q_, s_):                              # fake-quantised bf16 weight = bf16(dequant)
        return packing.dequant(q_, s_).to(torch.bfloat16)

    sd = {"tok_embeddings.weight": w["embed"], "norm.weight": w["nf"], "output.weight": fq(P["lm_q"], P["lm_s"])}
    nq, nkv = cfg.n_head * hd, cfg.n_local_heads * hd
    for l in range(cfg.n_layer):
        qkv = fq(P["qkv_q"][l], P["qkv_s"][l])
        wq, wk, wv = qkv[:nq], qkv[nq:nq + nkv], qkv[nq + nkv:]
        sd[f"layers.{l}.attention.wqkv.weight"] = torch.cat([permute(wq, cfg.n_head), permute(wk, cfg.n_local_heads), wv])
        sd[f"layers.{l}.attention.wo.weight"] = fq(P["o_q"][l], P["o_s"][l])
        gu = fq(P["gu_q"][l], P["gu_s"][l])
        sd[f"layers.{l}.feed_forward.w1.weight"] = gu[:f]
        sd[f"layers.{l}.feed_forward.w3.weight"] = gu[cfg.ffn_padded:cfg.ffn_padded + f]
        sd[f"layers.{l}.feed_forward.w2.weight"] = fq(P["d_q"][l], P["d_s"][l])[:, :f]
        sd[f"layers.{l}.attention_norm.weight"] = w["layers"][l]["n1"]
        sd[f"layers.{l}.ffn_norm.weight"] = w["layers"][l]["n2"]
    m.load_state_dict(sd, strict=True)
    m.eval()
    m.setup_caches(max_batch_size=1, max_seq_length=cfg.block_size)
    pg = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=pg)
    steps = 64
    logits = m(prompt.view(1, -1), torch.arange(16))          # prefill in one pass (reference: engine/generate.py:57-60)
    keep = {0, 1, 2, 31, 63}
    kept, toks = [], []
    cur = int(logits[0, -1].float().argmax())
    kept.append(logits[0, -1].float().numpy())                 # logits that produced generated token 0
    toks.append(cur)
    for i in range(1, steps):
        lg = m(torch.tensor([[cur]]), torch.tensor([16 + i - 1]))
        cur = int(lg[0, -1].float().argmax())
        toks.append(cur)
        if i in keep:
            kept.append(lg[0, -1].float().numpy())
    np.savez_compressed(os.path.join(HERE, "engine_tiny.npz"), prompt=prompt.numpy().astype(np.int32),
                        tokens=np.asarray(toks, np.int32), kept_steps=np.asarray(sorted(keep), np.int32),
                        logits=np.stack(kept).astype(np.float32))

    # ---------------------------------------------------------------- draft head
    torch.manual_seed(5)
    ddim, dnh, dinter = 64, 2, 128             # small on purpose: the fixture stays ~100 KB
    dh = ref_draft.DraftHead(ddim, dnh, dinter, fuse=1, rope_base=cfg.rope_base)
    for p in dh.parameters():
        if p.dim() == 2:
            p.data.normal_(0, 0.02)
    dh = dh.to(torch.bfloat16).eval()
    feat = torch.randn(1, 6, ddim).to(torch.bfloat16)
    emb = (torch.randn(1, 6, ddim) * 0.02).to(torch.bfloat16)
    out = dh(feat, emb, torch.arange(3, 9))
    np.savez_compressed(os.path.join(HERE, "draft_tiny.npz"),
                        **{"sd_" + k: bits(v) for k, v in dh.state_dict().items()},
                        dims=np.asarray([ddim, dnh, dinter], np.int32), feat=bits(feat), emb=bits(emb), positions=np.arange(3, 9, dtype=np.int32), out=bits(out))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
