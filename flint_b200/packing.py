"""int4 group-128 weight packing and seeded synthetic models (host side, torch; CPU or CUDA tensors).

Two packers, both producing the same container: `q int32[OUT, IN/8]` (nibble m of word c holds column
8c+m at bits [4m, 4m+4)), `s bf16[OUT, IN/128]` and, for the asymmetric packer, `z bf16[OUT, IN/128]`.
The kernels dequantise every weight as `(nibble - 8) * float(s) + float(z)` in fp32 (z = 0 when absent),
which is the arithmetic of the reference megakernel (reference: kernels/megakernel_decode.cu:30,34)
and, with z, of gpt-fast's group dequantiser (reference: engine/quantize.py:138-155).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .config import GROUP, ModelArgs

_SHIFTS = tuple(4 * m for m in range(8))


def _pack_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """uint nibbles [OUT, IN] (values 0..15, any integer dtype) -> int32 words [OUT, IN/8]."""
    out_rows, k = nib.shape
    n = nib.to(torch.int64).view(out_rows, k // 8, 8)
    word = torch.zeros(out_rows, k // 8, dtype=torch.int64, device=nib.device)
    for m, sh in enumerate(_SHIFTS):
        word |= n[..., m] << sh
    # two's-complement bit-cast of the low 32 bits
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32).contiguous()


def qpc(W: torch.Tensor, G: int = GROUP) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int4 pack, bit-identical to the reference packer (reference: chat.py:23-30).

    scale = absmax(group)/7 in fp32, q = clamp(round_half_even(W/scale), -8, 7), nibble = q+8, scale -> bf16.
    A group of all zeros has scale 0 and W/scale = NaN; the reference's NaN -> integer cast lands on
    nibble 0 for every element of that group, which this packer reproduces explicitly.
    """
    out_rows, k = W.shape
    if k % G != 0:
        raise ValueError(f"IN={k} is not a multiple of the group size {G} (pad the matrix with zero columns)")
    Wg = W.float().view(out_rows, k // G, G)
    s = Wg.abs().amax(-1, keepdim=True) / 7.0
    q = torch.clamp(torch.round(Wg / s), -8, 7)
    nib = torch.where(torch.isnan(q), torch.zeros_like(q), q + 8.0)
    return _pack_nibbles(nib.view(out_rows, k)), s.squeeze(-1).to(torch.bfloat16).contiguous()


def qpc_asym(W: torch.Tensor, G: int = GROUP) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Asymmetric int4 pack with bf16 scales and zeros (gpt-fast math, reference: engine/quantize.py:58-76,102-128).

    scale = (max-min).clamp(1e-6)/15, zero = min + 8*scale (both rounded to bf16),
    q = clamp(round((w - (zero - 8*scale)) / scale), 0, 15), computed in the dtype of W exactly as the
    reference does when it is handed bf16 weights (reference: engine/quantize.py:359-364).
    Returns (q words, s, z) in the container described in the module docstring.
    """
    out_rows, k = W.shape
    if k % G != 0:
        raise ValueError(f"IN={k} is not a multiple of the group size {G}")
    g = W.reshape(-1, G)
    max_val = g.amax(dim=1, keepdim=True)
    min_val = g.amin(dim=1, keepdim=True)
    scales = ((max_val - min_val).clamp(min=1e-6) / 15).to(torch.bfloat16)
    zeros = (min_val + ((max_val - min_val).clamp(min=1e-6) / 15) * 8).to(torch.bfloat16)
    lo = zeros - scales * 8
    q = g.sub(lo).div(scales).round().clamp_(0, 15).to(torch.int32)
    return (_pack_nibbles(q.view(out_rows, k)),
            scales.view(out_rows, k // G).contiguous(), zeros.view(out_rows, k // G).contiguous())


def from_gptfast(w_int32: torch.Tensor, scales_and_zeros: torch.Tensor):
    """Convert gpt-fast's `group_quantize_tensor` outputs (reference: engine/quantize.py:131-135) into the
    container used here: `w_int32[N, K]` (values 0..15) and `scales_and_zeros bf16[K/128, N, 2]`."""
    q = _pack_nibbles(w_int32)
    sz = scales_and_zeros.transpose(0, 1).contiguous()
    return q, sz[..., 0].contiguous(), sz[..., 1].contiguous()


def unpack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """int32 words [OUT, IN/8] -> int32 nibbles [OUT, IN] (0..15)."""
    w = q.to(torch.int64) & 0xFFFFFFFF
    parts = [((w >> sh) & 0xF) for sh in _SHIFTS]
    return torch.stack(parts, dim=-1).view(q.shape[0], q.shape[1] * 8).to(torch.int32)


def dequant(q: torch.Tensor, s: torch.Tensor, z: Optional[torch.Tensor] = None, G: int = GROUP) -> torch.Tensor:
    """fp32 [OUT, IN] = (nibble - 8) * float(s) + float(z): the dequantisation contract of the kernels."""
    nib = unpack_nibbles(q).float() - 8.0
    out_rows, k = nib.shape
    w = nib.view(out_rows, k // G, G) * s.float().unsqueeze(-1)
    if z is not None:
        w = w + z.float().unsqueeze(-1)
    return w.view(out_rows, k)


# --------------------------------------------------------------------------------------------------
# Seeded synthetic models (stand-ins for the Granite / Llama checkpoints the reference downloads,
# reference: chat.py:32-52). Weight order and distribution are fixed so every test sees the same model.
# --------------------------------------------------------------------------------------------------

def synth_weights(cfg: ModelArgs, seed: int = 0, device: str = "cpu", norm_mode: str = "ones") -> Dict[str, object]:
    """bf16 N(0, 0.02) matrices in the order [embed, per layer: wq wk wv wo w_gate w_up w_down, lm_head].

    norm_mode "ones" gives RMSNorm weights of 1; "ref" gives |N(0,1)|+0.5 as the reference's kernel tests
    use (reference: bench/megakernel_decode_test.py:37-38). The CPU and CUDA generators give different
    streams, so fixtures are always generated on CPU.
    """
    gen = torch.Generator(device=device).manual_seed(seed)
    d, hd = cfg.dim, cfg.head_dim

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def norm():
        if norm_mode == "ones":
            return torch.ones(d, dtype=torch.bfloat16, device=device)
        return (torch.randn(d, generator=gen, device=device, dtype=torch.float32).abs() + 0.5).to(torch.bfloat16)

    w: Dict[str, object] = {"embed": mat(cfg.vocab_size, d), "layers": []}
    for _ in range(cfg.n_layer):
        w["layers"].append(dict(
            wq=mat(cfg.n_head * hd, d), wk=mat(cfg.n_local_heads * hd, d), wv=mat(cfg.n_local_heads * hd, d),
            wo=mat(d, cfg.n_head * hd), w_gate=mat(cfg.intermediate_size, d), w_up=mat(cfg.intermediate_size, d),
            w_down=mat(d, cfg.intermediate_size), n1=norm(), n2=norm()))
    w["nf"] = norm()
    if not cfg.tie_embeddings:
        w["lm_head"] = mat(cfg.vocab_size, d)
    return w


def _pad_rows(m: torch.Tensor, rows: int) -> torch.Tensor:
    if m.shape[0] == rows:
        return m
    return torch.cat([m, torch.zeros(rows - m.shape[0], m.shape[1], dtype=m.dtype, device=m.device)], 0)


def _pad_cols(m: torch.Tensor, cols: int) -> torch.Tensor:
    if m.shape[1] == cols:
        return m
    return torch.cat([m, torch.zeros(m.shape[0], cols - m.shape[1], dtype=m.dtype, device=m.device)], 1)


def pack_model(w: Dict[str, object], cfg: ModelArgs, asym: bool = False) -> Dict[str, torch.Tensor]:
    """Pack a model into the stacked tensors the megakernel boundary takes (reference: chat.py:32-52).

    q/k/v rows are concatenated RAW (half-split RoPE needs no permutation), gate is stacked on up, the
    tied LM head is the int4 pack of the embedding. FFN widths that are not a multiple of 128 are padded
    with zero rows (gate/up) and zero columns (down). With asym=True every matrix also gets `*_z` zeros.
    """
    f = cfg.ffn_padded
    pk = qpc_asym if asym else qpc
    names = ("qkv", "o", "gu", "d")
    acc = {n: [] for n in names}
    for lw in w["layers"]:
        acc["qkv"].append(pk(torch.cat([lw["wq"], lw["wk"], lw["wv"]], 0)))
        acc["o"].append(pk(lw["wo"]))
        acc["gu"].append(pk(torch.cat([_pad_rows(lw["w_gate"], f), _pad_rows(lw["w_up"], f)], 0)))
        acc["d"].append(pk(_pad_cols(lw["w_down"], f)))
    P: Dict[str, torch.Tensor] = {}
    for n in names:
        P[n + "_q"] = torch.stack([a[0] for a in acc[n]]).contiguous()
        P[n + "_s"] = torch.stack([a[1] for a in acc[n]]).contiguous()
        if asym:
            P[n + "_z"] = torch.stack([a[2] for a in acc[n]]).contiguous()
    P["n1"] = torch.stack([lw["n1"] for lw in w["layers"]]).contiguous()
    P["n2"] = torch.stack([lw["n2"] for lw in w["layers"]]).contiguous()
    P["nf"] = w["nf"].contiguous()
    P["embed"] = w["embed"].contiguous()
    lm = pk(w["embed"] if cfg.tie_embeddings else w["lm_head"])
    P["lm_q"], P["lm_s"] = lm[0], lm[1]
    if asym:
        P["lm_z"] = lm[2]
    return P


def synth_packed(cfg: ModelArgs, seed: int = 0, device: str = "cpu", asym: bool = False,
                 norm_mode: str = "ones") -> Dict[str, torch.Tensor]:
    """Seeded synthetic model, generated and packed layer by layer so that peak memory stays near the
    packed size (a 3B-class model is 6.6 GB as bf16 matrices but 1.7 GB packed)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    d, hd, f = cfg.dim, cfg.head_dim, cfg.ffn_padded
    pk = qpc_asym if asym else qpc

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def norm():
        if norm_mode == "ones":
            return torch.ones(d, dtype=torch.bfloat16, device=device)
        return (torch.randn(d, generator=gen, device=device, dtype=torch.float32).abs() + 0.5).to(torch.bfloat16)

    names = ("qkv", "o", "gu", "d")
    acc = {n: [] for n in names}
    n1, n2 = [], []
    embed = mat(cfg.vocab_size, d)
    for _ in range(cfg.n_layer):
        wq, wk, wv = mat(cfg.n_head * hd, d), mat(cfg.n_local_heads * hd, d), mat(cfg.n_local_heads * hd, d)
        wo = mat(d, cfg.n_head * hd)
        wg, wu = mat(cfg.intermediate_size, d), mat(cfg.intermediate_size, d)
        wd = mat(d, cfg.intermediate_size)
        a, b = norm(), norm()
        acc["qkv"].append(pk(torch.cat([wq, wk, wv], 0)))
        acc["o"].append(pk(wo))
        acc["gu"].append(pk(torch.cat([_pad_rows(wg, f), _pad_rows(wu, f)], 0)))
        acc["d"].append(pk(_pad_cols(wd, f)))
        n1.append(a)
        n2.append(b)
    P: Dict[str, torch.Tensor] = {}
    for n in names:
        P[n + "_q"] = torch.stack([a[0] for a in acc[n]]).contiguous()
        P[n + "_s"] = torch.stack([a[1] for a in acc[n]]).contiguous()
        if asym:
            P[n + "_z"] = torch.stack([a[2] for a in acc[n]]).contiguous()
    P["n1"], P["n2"] = torch.stack(n1).contiguous(), torch.stack(n2).contiguous()
    P["nf"] = norm()
    P["embed"] = embed
    lm = pk(embed if cfg.tie_embeddings else mat(cfg.vocab_size, d))
    P["lm_q"], P["lm_s"] = lm[0], lm[1]
    if asym:
        P["lm_z"] = lm[2]
    return P
