"""CPU: real-checkpoint ingestion on a synthetic Hugging Face checkpoint the test writes itself (config.json +
two safetensors shards with HF key names): the packed tensors equal the packer's output on the same matrices bit for bit
and the Granite scalar multipliers arrive in the model configuration."""
import json
import os

import torch
from safetensors.torch import save_file

from flint_b200 import packing
from flint_b200.checkpoint import config_from_hf, load_hf_checkpoint
from flint_b200.config import ModelArgs


def _write_hf(tmp, cfg, w, tied, extra):
    sd = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["nf"]}
    for l, lw in enumerate(w["layers"]):
        p = f"model.layers.{l}."
        sd.update({p + "self_attn.q_proj.weight": lw["wq"], p + "self_attn.k_proj.weight": lw["wk"],
                   p + "self_attn.v_proj.weight": lw["wv"], p + "self_attn.o_proj.weight": lw["wo"],
                   p + "mlp.gate_proj.weight": lw["w_gate"], p + "mlp.up_proj.weight": lw["w_up"],
                   p + "mlp.down_proj.weight": lw["w_down"], p + "input_layernorm.weight": lw["n1"],
                   p + "post_attention_layernorm.weight": lw["n2"]})
    if not tied:
        sd["lm_head.weight"] = w["lm_head"]
    keys = sorted(sd)
    half = len(keys) // 2
    save_file({k: sd[k].contiguous() for k in keys[:half]}, os.path.join(tmp, "model-00001-of-00002.safetensors"))
    save_file({k: sd[k].contiguous() for k in keys[half:]}, os.path.join(tmp, "model-00002-of-00002.safetensors"))
    hf = dict(hidden_size=cfg.dim, num_attention_heads=cfg.n_head, num_key_value_heads=cfg.n_local_heads,
              num_hidden_layers=cfg.n_layer, intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size,
              rope_theta=cfg.rope_base, rms_norm_eps=cfg.norm_eps, tie_word_embeddings=tied, max_position_embeddings=512)
    hf.update(extra)
    json.dump(hf, open(os.path.join(tmp, "config.json"), "w"))


def test_tied_granite_style_checkpoint_round_trip(tmp_path):
    cfg = ModelArgs.from_name("tiny")                       # FFN 1376: exercises the zero padding to 1408
    w = packing.synth_weights(cfg, seed=3, device="cpu", norm_mode="ref")
    gran = dict(embedding_multiplier=12.0, attention_multiplier=0.015625, residual_multiplier=0.22, logits_scaling=10.0)
    _write_hf(str(tmp_path), cfg, w, True, gran)
    got_cfg, P = load_hf_checkpoint(str(tmp_path), device="cpu")
    want = packing.pack_model(w, cfg)
    assert set(P) == set(want)
    for k in want:
        assert torch.equal(P[k], want[k]), k
    assert (got_cfg.embedding_multiplier, got_cfg.attention_multiplier, got_cfg.residual_multiplier, got_cfg.logits_scaling) == \
        (12.0, 0.015625, 0.22, 10.0)
    assert got_cfg.attn_scale == 0.015625 and got_cfg.tie_embeddings and got_cfg.block_size == 512
    assert (got_cfg.n_layer, got_cfg.dim, got_cfg.n_head, got_cfg.n_local_heads, got_cfg.ffn_padded) == (4, 512, 8, 2, 1408)


def test_untied_asymmetric_checkpoint(tmp_path):
    cfg = ModelArgs(block_size=64, vocab_size=512, n_layer=2, n_head=4, n_local_heads=2, dim=256, intermediate_size=512,
                    tie_embeddings=False)
    w = packing.synth_weights(cfg, seed=4, device="cpu")
    _write_hf(str(tmp_path), cfg, w, False, {})
    got_cfg, P = load_hf_checkpoint(str(tmp_path), device="cpu", asym=True)
    want = packing.pack_model(w, cfg, asym=True)
    for k in want:
        assert torch.equal(P[k], want[k]), k
    assert not got_cfg.tie_embeddings and got_cfg.attn_scale == 64 ** -0.5 and got_cfg.logits_scaling == 1.0


def test_config_rejects_a_detached_head_dim():
    import pytest
    with pytest.raises(ValueError):
        config_from_hf(dict(hidden_size=512, num_attention_heads=8, head_dim=128, vocab_size=10, num_hidden_layers=1,
                            intermediate_size=1024))
