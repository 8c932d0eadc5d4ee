"""Real-checkpoint ingestion: a Hugging Face checkpoint directory (config.json + *.safetensors) -> the packed dict the
megakernel boundary takes.

Follows the reference's loader (reference: chat.py:32-52): q/k/v rows are concatenated RAW (HF Llama / Granite
checkpoints already use the half-split RoPE convention the kernels implement; no gpt-fast permutation, reference:
engine/scripts/convert_hf_checkpoint.py:75-81 is NOT applied), gate is stacked on up, the LM head is `lm_head.weight` or,
for tied checkpoints, the embedding itself, every matrix packed with the symmetric (or asymmetric) int4 group-128 packer.
The model's scalar multipliers come from config.json (Granite: embedding_multiplier, attention_multiplier,
residual_multiplier, logits_scaling; reference: chat.py:19-21, engine/model.py:77-79). Layers are packed one at a time, so
peak memory stays near the packed size. FFN widths that are not a multiple of 128 are padded with zero rows / columns.
"""
from __future__ import annotations

import json
import os
from glob import glob
from typing import Dict, Tuple

import torch

from .config import ModelArgs
from .packing import _pad_cols, _pad_rows, qpc, qpc_asym


def config_from_hf(cfg_json: dict, block_size: int = 0) -> ModelArgs:
    """ModelArgs from the fields of a Hugging Face Llama- or Granite-style config.json."""
    d, nh = int(cfg_json["hidden_size"]), int(cfg_json["num_attention_heads"])
    if "head_dim" in cfg_json and cfg_json["head_dim"] and int(cfg_json["head_dim"]) != d // nh:
        raise ValueError("head_dim must equal hidden_size / num_attention_heads on this path")
    return ModelArgs(
        block_size=int(block_size or cfg_json.get("max_position_embeddings", 4096)),
        vocab_size=int(cfg_json["vocab_size"]), n_layer=int(cfg_json["num_hidden_layers"]), n_head=nh, dim=d,
        intermediate_size=int(cfg_json["intermediate_size"]),
        n_local_heads=int(cfg_json.get("num_key_value_heads") or nh), rope_base=float(cfg_json.get("rope_theta", 10000.0)),
        norm_eps=float(cfg_json.get("rms_norm_eps", 1e-5)),
        embedding_multiplier=float(cfg_json.get("embedding_multiplier", 1.0)),
        attention_multiplier=(float(cfg_json["attention_multiplier"]) if cfg_json.get("attention_multiplier") is not None else None),
        residual_multiplier=float(cfg_json.get("residual_multiplier", 1.0)),
        logits_scaling=float(cfg_json.get("logits_scaling", 1.0)),
        tie_embeddings=bool(cfg_json.get("tie_word_embeddings", False)))


class _Shards:
    """Lazy access to the tensors of every *.safetensors file in a directory."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self.files = sorted(glob(os.path.join(path, "*.safetensors")))
        if not self.files:
            raise FileNotFoundError(f"no *.safetensors in {path}")
        self.handles = [safe_open(f, framework="pt", device="cpu") for f in self.files]
        self.where = {k: h for h in self.handles for k in h.keys()}

    def __contains__(self, k):
        return k in self.where

    def get(self, k: str) -> torch.Tensor:
        if k not in self.where:
            raise KeyError(f"checkpoint lacks {k}")
        return self.where[k].get_tensor(k)


def load_hf_checkpoint(path: str, device: str = "cuda", asym: bool = False, block_size: int = 0) -> Tuple[ModelArgs, Dict[str, torch.Tensor]]:
    """(ModelArgs, packed dict on `device`) from a Hugging Face checkpoint directory."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = config_from_hf(json.load(f), block_size)
    sd = _Shards(path)
    pk = qpc_asym if asym else qpc
    f_pad = cfg.ffn_padded
    dev = torch.device(device)

    def W(name):
        return sd.get(name).to(device=dev, dtype=torch.bfloat16)

    names = ("qkv", "o", "gu", "d")
    acc = {n: [] for n in names}
    n1, n2 = [], []
    for l in range(cfg.n_layer):
        p = f"model.layers.{l}."
        acc["qkv"].append(pk(torch.cat([W(p + "self_attn.q_proj.weight"), W(p + "self_attn.k_proj.weight"),
                                        W(p + "self_attn.v_proj.weight")], 0)))
        acc["o"].append(pk(W(p + "self_attn.o_proj.weight")))
        acc["gu"].append(pk(torch.cat([_pad_rows(W(p + "mlp.gate_proj.weight"), f_pad),
                                       _pad_rows(W(p + "mlp.up_proj.weight"), f_pad)], 0)))
        acc["d"].append(pk(_pad_cols(W(p + "mlp.down_proj.weight"), f_pad)))
        n1.append(W(p + "input_layernorm.weight"))
        n2.append(W(p + "post_attention_layernorm.weight"))
    P: Dict[str, torch.Tensor] = {}
    for n in names:
        P[n + "_q"] = torch.stack([a[0] for a in acc[n]]).contiguous()
        P[n + "_s"] = torch.stack([a[1] for a in acc[n]]).contiguous()
        if asym:
            P[n + "_z"] = torch.stack([a[2] for a in acc[n]]).contiguous()
    P["n1"], P["n2"] = torch.stack(n1).contiguous(), torch.stack(n2).contiguous()
    P["nf"] = W("model.norm.weight").contiguous()
    P["embed"] = W("model.embed_tokens.weight").contiguous()
    tied = cfg.tie_embeddings or "lm_head.weight" not in sd
    cfg.tie_embeddings = tied
    lm = pk(P["embed"] if tied else W("lm_head.weight"))
    P["lm_q"], P["lm_s"] = lm[0], lm[1]
    if asym:
        P["lm_z"] = lm[2]
    return cfg, P
