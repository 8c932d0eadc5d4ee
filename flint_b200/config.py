"""Model configuration for the batch-1 int4 decode path.

`ModelArgs` keeps the field names of the reference's gpt-fast dataclass
(reference: engine/model.py:20-45) so that code written against
`Transformer.from_name(...)`/`ModelArgs.from_name(...)` keeps working, and adds
the few facts the megakernel needs that the reference keeps as module globals
(reference: chat.py:19-21): tied embeddings and the padded FFN width.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

GROUP = 128  # int4 quantisation group size along K (reference: chat.py:23, engine/quantize.py:58)


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of k that is >= n (reference: engine/model.py:15-18)."""
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class ModelArgs:
    block_size: int = 2048
    vocab_size: int = 32000
    n_layer: int = 32
    n_head: int = 32
    dim: int = 4096
    intermediate_size: Optional[int] = None
    n_local_heads: int = -1
    head_dim: int = 64
    rope_base: float = 10000
    norm_eps: float = 1e-5
    # Granite-style scalar multipliers (reference: engine/model.py:31-35); 1.0 / None = plain Llama.
    embedding_multiplier: float = 1.0
    attention_multiplier: Optional[float] = None
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0
    # Not in the reference dataclass: the megakernel path ties the LM head to int4(embedding)
    # (reference: chat.py:51); the 8B-class config has its own head.
    tie_embeddings: bool = True

    def __post_init__(self):
        if self.n_local_heads == -1:
            self.n_local_heads = self.n_head
        if self.intermediate_size is None:
            hidden_dim = 4 * self.dim
            self.intermediate_size = find_multiple(int(2 * hidden_dim / 3), 256)
        self.head_dim = self.dim // self.n_head

    # ---- derived quantities used by the packer, the oracle and the kernels ----
    @property
    def ffn_padded(self) -> int:
        """FFN width rounded up to the int4 group (1376 -> 1408); padding rows/columns are zero weights."""
        return find_multiple(self.intermediate_size, GROUP)

    @property
    def qkv_rows(self) -> int:
        return (self.n_head + 2 * self.n_local_heads) * self.head_dim

    @property
    def attn_scale(self) -> float:
        return self.attention_multiplier if self.attention_multiplier is not None else self.head_dim ** -0.5

    def int4_params(self) -> int:
        """Number of int4 weights one decode step streams (all GEMV matrices incl. LM head)."""
        d, f = self.dim, self.ffn_padded
        per_layer = self.qkv_rows * d + d * (self.n_head * self.head_dim) + 2 * f * d + d * f
        return self.n_layer * per_layer + self.vocab_size * d

    def bytes_per_token(self, mean_cached_len: float = 0.0, has_zeros: bool = False) -> float:
        """Algorithmic HBM bytes per decode step: nibbles + bf16 group scales (+ zeros) + bf16 K/V rows attended.

        Same definition as the reference's MBU figure (reference: bench/megakernel_decode_test.py:77-78,88)
        extended by the KV term.
        """
        p = self.int4_params()
        kv_pos = 2 * self.n_layer * self.n_local_heads * self.head_dim * 2
        return p * 0.5 + (p // GROUP) * 2 * (2 if has_zeros else 1) + kv_pos * mean_cached_len

    @classmethod
    def from_name(cls, name: str) -> "ModelArgs":
        if name in transformer_configs:
            return cls(**transformer_configs[name])
        hits = [k for k in transformer_configs if k.lower() in str(name).lower()]
        if not hits:
            raise KeyError(f"unknown model config {name!r}; known: {sorted(transformer_configs)}")
        hits.sort(key=len, reverse=True)
        return cls(**transformer_configs[hits[0]])

    def to_dict(self):
        return asdict(self)


transformer_configs = {
    # Tiny CPU-runnable decoder: 4 layers, d 512, 8 q / 2 kv heads, hd 64, SwiGLU 1376, vocab 4096, tied.
    "tiny": dict(block_size=256, vocab_size=4096, n_layer=4, n_head=8, n_local_heads=2, dim=512,
                 intermediate_size=1376, rope_base=10000),
    # Small decoder with heads of 80 whose 2-rank split owns 320 attention columns = 2.5 int4 groups: the same O-window
    # situation as the 3B-class model over 8 ranks, testable on 2 GPUs.
    "tiny-window": dict(block_size=256, vocab_size=512, n_layer=2, n_head=8, n_local_heads=2, dim=640,
                        intermediate_size=1024, rope_base=10000),
    # 3B-class Granite-shaped dense decoder (the headline single-GPU config).
    "granite-3b-class": dict(block_size=4096, vocab_size=49160, n_layer=40, n_head=32, n_local_heads=8, dim=2560,
                             intermediate_size=8192, rope_base=10000),
    # Same model with a 32768-position KV cache (long-context decode).
    "granite-3b-class-32k": dict(block_size=32768 + 256, vocab_size=49160, n_layer=40, n_head=32, n_local_heads=8,
                                 dim=2560, intermediate_size=8192, rope_base=10000),
    # 1B-class Llama-shaped decoder (32 query / 8 kv heads of 64, tied head): a fourth width for the kernel table.
    "llama-1b-class": dict(block_size=8192, vocab_size=128256, n_layer=16, n_head=32, n_local_heads=8, dim=2048,
                           intermediate_size=8192, rope_base=500000),
    # 8B-class Llama-shaped decoder, untied head (the tensor-parallel config); same shape as the
    # reference's "llama-3-8b" entry (reference: engine/model.py:74).
    "llama-8b-class": dict(block_size=8192, vocab_size=128256, n_layer=32, n_head=32, n_local_heads=8, dim=4096,
                           intermediate_size=14336, rope_base=500000, tie_embeddings=False),
    "llama-3-8b": dict(block_size=8192, vocab_size=128256, n_layer=32, n_head=32, n_local_heads=8, dim=4096,
                       intermediate_size=14336, rope_base=500000, tie_embeddings=False),
    # The only shape the reference kernels can run (reference: chat.py:19-21, engine/model.py:77-79).
    "granite-4.1-3b": dict(block_size=8192, n_layer=40, n_head=40, n_local_heads=8, dim=2560,
                           intermediate_size=8192, vocab_size=100352, rope_base=10000000,
                           embedding_multiplier=12.0, attention_multiplier=0.015625, residual_multiplier=0.22,
                           logits_scaling=10.0),
}
