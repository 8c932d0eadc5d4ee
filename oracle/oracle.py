"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle.

`flint_oracle.c` (same folder) restates the reference's decode / tree-verify step; this module compiles it
with gcc, loads it with ctypes and adds numpy restatements of the two reference packers. Nothing in the
product package may import this module: it is the checker, used by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.

Reference lines restated here (paths inside the reference project):
  np_qpc            chat.py:23-30                      symmetric int4 g128 pack
  np_qpc_asym       engine/quantize.py:58-76,102-128   asymmetric int4 g128 pack (bf16 scales and zeros)
  np_dequant        kernels/megakernel_decode.cu:30,34 ; engine/quantize.py:150-153
  static_tree       spec_tree.py:98-104                ancestor-or-self mask of a token tree
  chain_accept      spec_mega.py:106-110               longest agreeing prefix
  tree_accept       spec_tree.py:108-118               longest agreeing root-to-leaf walk
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(HERE, "flint_oracle.c")
_SO = os.path.join(HERE, "libflint_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """gcc -O3 -fopenmp the C restatement into oracle/libflint_oracle.so (rebuilt when the source is newer)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        tmp = _SO + f".tmp{os.getpid()}"
        subprocess.check_call(["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11",
                               "-o", tmp, _SRC, "-lm"])
        os.replace(tmp, _SO)
    return _SO


class _Desc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("n_layer", "dim", "n_head", "n_kv", "head_dim", "ffn", "vocab", "max_seq", "has_zeros")] + \
               [(n, ctypes.c_float) for n in ("eps", "rope_base", "attn_scale", "resid", "logits_scaling")]


_WNAMES = ("qkv_q", "o_q", "gu_q", "d_q", "lm_q", "qkv_s", "o_s", "gu_s", "d_s", "lm_s",
           "qkv_z", "o_z", "gu_z", "d_z", "lm_z", "n1", "n2", "nf")


class _Weights(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in _WNAMES]


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.fo_step.restype = ctypes.c_int
        _lib.fo_argmax.restype = ctypes.c_int
    return _lib


def set_threads(n: int = 0) -> int:
    """OpenMP threads of the oracle (0 = leave as is); returns the count in force. Process launchers often export
    OMP_NUM_THREADS=1, which would turn the timed CPU baseline into a one-core run."""
    lib().fo_set_threads.restype = ctypes.c_int
    return int(lib().fo_set_threads(ctypes.c_int(int(n))))


def _np(t) -> np.ndarray:
    """torch tensor (bf16 viewed as int16) or ndarray -> C-contiguous ndarray sharing or copying the bits."""
    if isinstance(t, np.ndarray):
        return np.ascontiguousarray(t)
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------------------------------------------ bf16 helpers
def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits (uint16), round-to-nearest-even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + (0x7FFF + ((u >> 16) & 1))
    out = (r >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    out[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return out


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------------------------------ packers
def _np_pack(nib: np.ndarray) -> np.ndarray:
    rows, k = nib.shape
    n = nib.astype(np.uint32).reshape(rows, k // 8, 8)
    word = np.zeros((rows, k // 8), dtype=np.uint32)
    for m in range(8):
        word |= n[..., m] << np.uint32(4 * m)
    return word.view(np.int32)


def np_qpc(W_bf16_bits: np.ndarray, G: int = 128) -> Tuple[np.ndarray, np.ndarray]:
    """Symmetric pack of a bf16 matrix given as uint16 bits -> (int32 words, bf16-bit scales)."""
    W = bf16_to_f32(W_bf16_bits)
    rows, k = W.shape
    Wg = W.reshape(rows, k // G, G)
    s = (np.abs(Wg).max(-1, keepdims=True) / np.float32(7.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.clip(np.rint(Wg / s), -8, 7)
    nib = np.where(np.isnan(q), 0.0, q + 8.0)
    return _np_pack(nib.reshape(rows, k)), bf16_round(s[..., 0])


def np_qpc_asym(W_bf16_bits: np.ndarray, G: int = 128):
    """Asymmetric pack; every intermediate is rounded to bf16 as torch does for bf16 operands."""
    rb = lambda a: bf16_to_f32(bf16_round(a))
    W = bf16_to_f32(W_bf16_bits)
    rows, k = W.shape
    g = W.reshape(-1, G)
    mx, mn = g.max(1, keepdims=True), g.min(1, keepdims=True)
    rng = np.maximum(rb(mx - mn), np.float32(1e-6))
    rng = rb(rng)
    scales = rb(rng / np.float32(15))
    zeros = rb(mn + rb(scales * np.float32(8)))
    lo = rb(zeros - rb(scales * np.float32(8)))
    q = np.clip(np.rint(rb(rb(g - lo) / scales)), 0, 15)
    return (_np_pack(q.reshape(rows, k)), bf16_round(scales).reshape(rows, k // G),
            bf16_round(zeros).reshape(rows, k // G))


def np_dequant(q: np.ndarray, s_bits: np.ndarray, z_bits: Optional[np.ndarray] = None, G: int = 128) -> np.ndarray:
    w = q.view(np.uint32)
    rows, words = w.shape
    nib = np.stack([(w >> np.uint32(4 * m)) & np.uint32(0xF) for m in range(8)], -1).reshape(rows, words * 8)
    v = (nib.astype(np.float32) - np.float32(8.0)).reshape(rows, -1, G) * bf16_to_f32(s_bits)[..., None]
    if z_bits is not None:
        v = v + bf16_to_f32(z_bits)[..., None]
    return v.reshape(rows, words * 8).astype(np.float32)


def c_dequant(q, s, z=None) -> np.ndarray:
    qa, sa = _np(q), _np(s)
    za = _np(z) if z is not None else None
    rows, words = qa.shape
    out = np.empty((rows, words * 8), dtype=np.float32)
    lib().fo_dequant(_ptr(qa), _ptr(sa), _ptr(za), ctypes.c_int(rows), ctypes.c_int(words * 8), _ptr(out))
    return out


def c_gemv(q, s, z, x_bf16) -> np.ndarray:
    """y[M, rows] fp32 for x bf16 [M, K] (or [K])."""
    qa, sa = _np(q), _np(s)
    za = _np(z) if z is not None else None
    xa = _np(x_bf16)
    if xa.ndim == 1:
        xa = xa[None]
    xf = np.ascontiguousarray(bf16_to_f32(xa))
    rows, words = qa.shape
    M = xf.shape[0]
    y = np.empty((M, rows), dtype=np.float32)
    lib().fo_gemv(_ptr(qa), _ptr(sa), _ptr(za), ctypes.c_int(rows), ctypes.c_int(words * 8), _ptr(xf),
                  ctypes.c_int(M), _ptr(y), ctypes.c_int(rows))
    return y


# ------------------------------------------------------------------------------------------------ the model
class OracleModel:
    """Holds a packed model (the dict made by the packer: qkv_q, qkv_s, ..., n1, n2, nf, embed, lm_q, lm_s and
    optional *_z) plus its own KV cache, and steps it on the CPU."""

    def __init__(self, cfg, packed: Dict[str, object], max_seq: Optional[int] = None):
        self.cfg = cfg
        self.max_seq = int(max_seq or cfg.block_size)
        self.has_zeros = "qkv_z" in packed
        self._keep = {k: _np(v) for k, v in packed.items()}
        self.desc = _Desc(cfg.n_layer, cfg.dim, cfg.n_head, cfg.n_local_heads, cfg.head_dim, cfg.ffn_padded,
                          cfg.vocab_size, self.max_seq, int(self.has_zeros), cfg.norm_eps, float(cfg.rope_base),
                          float(cfg.attn_scale), float(cfg.residual_multiplier), float(cfg.logits_scaling))
        w = _Weights()
        for n in _WNAMES:
            a = self._keep.get(n)
            setattr(w, n, None if a is None else a.ctypes.data)
        self.w = w
        kvshape = (cfg.n_layer, self.max_seq, cfg.n_local_heads, cfg.head_dim)
        self.kc = np.zeros(kvshape, dtype=np.uint16)
        self.vc = np.zeros(kvshape, dtype=np.uint16)
        self.embed = self._keep["embed"]

    def embed_rows(self, tokens: Sequence[int]) -> np.ndarray:
        """h = bf16(float(embed[token]) * embedding_multiplier)   (reference: chat.py:72)."""
        rows = bf16_to_f32(self.embed[np.asarray(tokens, dtype=np.int64)])
        return bf16_round(rows * np.float32(self.cfg.embedding_multiplier))

    def step_h(self, h_bits: np.ndarray, pos: int, depth=None, amask=None, want_logits=True):
        h = np.ascontiguousarray(h_bits, dtype=np.uint16).reshape(-1, self.cfg.dim).copy()
        M = h.shape[0]
        depth = np.zeros(M, np.int32) if depth is None else np.ascontiguousarray(depth, dtype=np.int32)
        amask = np.tril(np.ones((M, M), np.uint8)) if amask is None else np.ascontiguousarray(amask, dtype=np.uint8)
        logits = np.empty((M, self.cfg.vocab_size), dtype=np.float32) if want_logits else None
        feat = np.empty((M, self.cfg.dim), dtype=np.uint16)
        rc = lib().fo_step(ctypes.byref(self.desc), ctypes.byref(self.w), _ptr(h), _ptr(self.kc), _ptr(self.vc),
                           _ptr(depth), _ptr(amask), ctypes.c_int(pos), ctypes.c_int(M), _ptr(logits), _ptr(feat))
        if rc != 0:
            raise ValueError(f"oracle step rejected its arguments (code {rc})")
        return logits, feat, h

    def decode(self, token: int, pos: int) -> np.ndarray:
        """One greedy-decode step: logits f32 [vocab]."""
        return self.step_h(self.embed_rows([token]), pos)[0][0]

    def verify(self, tokens: Sequence[int], pos: int, depth=None, amask=None):
        """M-token tree verify: (logits [M, vocab], feature bf16 bits [M, dim]). Chain by default."""
        M = len(tokens)
        if depth is None:
            depth = np.arange(M, dtype=np.int32)
        lg, ft, _ = self.step_h(self.embed_rows(tokens), pos, depth, amask)
        return lg, ft

    def kv_move(self, src: Sequence[int], dst: Sequence[int]):
        """Tree KV surgery, sequential like the reference loop (reference: spec_tree.py:126-128)."""
        for a, b in zip(src, dst):
            if a != b:
                self.kc[:, b] = self.kc[:, a]
                self.vc[:, b] = self.vc[:, a]


def argmax_first(v: np.ndarray) -> int:
    return int(np.argmax(v))


# ------------------------------------------------------------------------------------------------ trees
def tree_mask(parent: Sequence[int]) -> np.ndarray:
    """Ancestor-or-self mask; parent[i] is the index of node i's parent, -1 for the root."""
    n = len(parent)
    m = np.zeros((n, n), dtype=np.uint8)
    for i in range(n):
        j = i
        while j != -1:
            m[i, j] = 1
            j = parent[j]
    return m


def chain_accept(target: Sequence[int], draft: Sequence[int]) -> int:
    acc = 0
    for j in range(len(draft)):
        if int(target[j]) == int(draft[j]):
            acc += 1
        else:
            break
    return acc


def tree_accept(cand: Sequence[int], parent: Sequence[int], target: Sequence[int]) -> List[int]:
    children: Dict[int, List[int]] = {i: [] for i in range(len(cand))}
    for i, p in enumerate(parent):
        if p >= 0:
            children[p].append(i)
    path, cur = [0], 0
    while True:
        nxt = None
        for ch in children[cur]:
            if cand[ch] == target[cur]:
                nxt = ch
                break
        if nxt is None:
            return path
        path.append(nxt)
        cur = nxt
