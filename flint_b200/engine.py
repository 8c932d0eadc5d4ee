"""Host side of the decode path: the context object and the reference-shaped launch functions.

`decode_mega_launch(...)` takes the same positional arguments and returns the same tensor as the reference's
pybind11 function (reference: kernels/megakernel_decode.cu:204-237), so the loops in chat.py / spec_mega.py
(reference: chat.py:71-74, spec_mega.py:46-49) run unchanged; `DecodeEngine` is the explicit form that also
does the embedding lookup and the argmax on the device. PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import _lib
from .config import ModelArgs


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def query(device: int = 0) -> Dict[str, int]:
    caps = _lib.Caps()
    _lib.check(_lib.load().fb_query(device, ctypes.byref(caps)), "fb_query")
    return {n: getattr(caps, n) for n, _ in caps._fields_}


class DecodeEngine:
    """One model bound to one GPU: streaming-layout weights, scratch, a KV cache and the megakernel launches."""

    def __init__(self, cfg: ModelArgs, packed: Dict[str, torch.Tensor], max_seq: Optional[int] = None,
                 device: Optional[torch.device] = None, kc: Optional[torch.Tensor] = None,
                 vc: Optional[torch.Tensor] = None, tp_rank: int = 0, tp_size: int = 1):
        """`packed` holds this rank's slice when tp_size > 1 (flint_b200.tp.shard_packed); cfg is the full model."""
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("flint_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.cfg = cfg
        self.device = torch.device(device if device is not None else packed["qkv_q"].device)
        if self.device.type != "cuda":
            raise ValueError("packed weights must live on the GPU that runs the kernels")
        self.dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.has_zeros = "qkv_z" in packed
        self.max_seq = int(max_seq or cfg.block_size)
        self.tp_rank, self.tp_size = int(tp_rank), int(tp_size)
        for what, n in (("query heads", cfg.n_head), ("kv heads", cfg.n_local_heads), ("FFN width / 128", cfg.ffn_padded // 128),
                        ("vocabulary", cfg.vocab_size)):
            if n % self.tp_size:
                raise ValueError(f"{what} ({n}) does not divide over {self.tp_size} ranks")
        self.n_kv_local = cfg.n_local_heads // self.tp_size
        self.vocab_local = cfg.vocab_size // self.tp_size
        d = _lib.ModelDesc(cfg.n_layer, cfg.dim, cfg.n_head // self.tp_size, self.n_kv_local, cfg.head_dim,
                           cfg.ffn_padded // self.tp_size, self.vocab_local, int(self.has_zeros), cfg.norm_eps,
                           float(cfg.rope_base), float(cfg.attn_scale), float(cfg.residual_multiplier),
                           float(cfg.embedding_multiplier), float(cfg.logits_scaling))
        self._ctx = ctypes.c_void_p()
        _lib.check(self.lib.fb_ctx_create_tp(ctypes.byref(d), self.dev_index, self.tp_rank, self.tp_size,
                                             self.tp_rank * self.vocab_local, ctypes.byref(self._ctx)), "fb_ctx_create")
        # keep-alive: the norms and the embedding table stay caller-side tensors
        self._keep = {k: packed[k].contiguous() for k in ("n1", "n2", "nf") if k in packed}
        if "embed" in packed and packed["embed"] is not None:
            self._keep["embed"] = packed["embed"].contiguous()
        w = _lib.WeightPtrs()
        for name in _lib.WEIGHT_FIELDS:
            t = self._keep.get(name, packed.get(name))
            if t is not None:
                if t.device != self.device or not t.is_contiguous():
                    raise ValueError(f"{name}: must be a contiguous tensor on {self.device}")
                setattr(w, name, t.data_ptr())
        _lib.check(self.lib.fb_bind_weights(self._ctx, ctypes.byref(w), _stream_ptr(self.device)), "fb_bind_weights")
        torch.cuda.synchronize(self.device)
        shape = (cfg.n_layer, self.max_seq, self.n_kv_local, cfg.head_dim)
        self.kc = kc if kc is not None else torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.vc = vc if vc is not None else torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.bind_kv(self.kc, self.vc)
        self._logits = torch.empty(cfg.vocab_size, dtype=torch.float32, device=self.device)
        self._next = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ plumbing
    def bind_kv(self, kc: torch.Tensor, vc: torch.Tensor):
        want = (self.cfg.n_layer, kc.shape[1], self.n_kv_local, self.cfg.head_dim)
        for t in (kc, vc):
            if tuple(t.shape) != want or t.dtype != torch.bfloat16 or not t.is_contiguous() or t.device != self.device:
                raise ValueError(f"KV cache must be contiguous bf16 {want} on {self.device}")
        self.kc, self.vc, self.max_seq = kc, vc, kc.shape[1]
        _lib.check(self.lib.fb_bind_kv(self._ctx, _ptr(kc), _ptr(vc), self.max_seq), "fb_bind_kv")

    # ------------------------------------------------------------------ tensor parallel wiring
    def tp_export(self) -> bytes:
        """64-byte IPC handle of this rank's inbox; exchange it with every other rank (any transport)."""
        buf = ctypes.create_string_buffer(64)
        _lib.check(self.lib.fb_tp_export(self._ctx, buf), "fb_tp_export")
        return buf.raw

    def tp_connect(self, handles):
        """handles[p] = rank p's exported handle."""
        blob = b"".join(handles)
        _lib.check(self.lib.fb_tp_connect(self._ctx, ctypes.c_char_p(blob), len(handles)), "fb_tp_connect")

    def set_option(self, what: int, value: int):
        _lib.check(self.lib.fb_set_option(self._ctx, what, value), "fb_set_option")

    def status(self) -> Dict[str, int]:
        """Synchronises, then returns the device status of the launches so far (code 0 = clean)."""
        torch.cuda.synchronize(self.device)
        st = _lib.Status()
        _lib.check(self.lib.fb_last_status(self._ctx, ctypes.byref(st)), "fb_last_status")
        return {n: getattr(st, n) for n, _ in st._fields_}

    def check(self):
        st = self.status()
        if st["code"] != 0:
            raise _lib.FlintError(st["code"], f"device status {st}")

    def close(self):
        if getattr(self, "_ctx", None) is not None and self._ctx.value:
            self.lib.fb_ctx_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ launches (asynchronous on the current stream)
    def decode(self, token: int, pos: int, logits: Optional[torch.Tensor] = None,
               next_token: Optional[torch.Tensor] = None, want_logits: bool = True) -> torch.Tensor:
        """One step from a host token id. Returns the f32 [vocab] logits tensor (a reused buffer unless given)."""
        lg = logits if logits is not None else (self._logits if want_logits else None)
        nx = next_token if next_token is not None else self._next
        _lib.check(self.lib.fb_decode(self._ctx, int(token), None, None, int(pos), _ptr(lg), _ptr(nx),
                                      _stream_ptr(self.device)), "fb_decode")
        return lg

    def decode_chained(self, token_dev: torch.Tensor, pos: int, next_token: torch.Tensor,
                       logits: Optional[torch.Tensor] = None):
        """One step whose input token is read from device memory (the previous step's argmax): no host sync."""
        _lib.check(self.lib.fb_decode(self._ctx, 0, _ptr(token_dev), None, int(pos), _ptr(logits), _ptr(next_token),
                                      _stream_ptr(self.device)), "fb_decode")

    def decode_h(self, h: torch.Tensor, pos: int, logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One step from an already multiplied embedding h bf16 [dim] (clobbered, as the reference does)."""
        lg = logits if logits is not None else torch.empty(self.cfg.vocab_size, dtype=torch.float32, device=self.device)
        _lib.check(self.lib.fb_decode(self._ctx, 0, None, _ptr(h), int(pos), _ptr(lg), _ptr(self._next),
                                      _stream_ptr(self.device)), "fb_decode")
        return lg

    @property
    def next_token(self) -> torch.Tensor:
        return self._next

    # ------------------------------------------------------------------ M-token tree verification
    def _tree_args(self, M: int, depth, amask):
        if depth is None:
            depth = torch.arange(M, dtype=torch.int32, device=self.device)            # chain: depth = index
        if amask is None:
            amask = torch.tril(torch.ones(M, M, dtype=torch.uint8, device=self.device))  # chain: causal
        depth = torch.as_tensor(depth, device=self.device).to(torch.int32).contiguous()
        amask = torch.as_tensor(amask, device=self.device).to(torch.uint8).contiguous()
        if depth.numel() != M or tuple(amask.shape) != (M, M):
            raise ValueError("depth must have M entries and amask must be [M, M]")
        return depth, amask

    def verify(self, tokens, pos: int, depth=None, amask=None, want_logits: bool = True):
        """Score M candidate tokens in one weight pass: returns (logits f32 [M, vocab] or None, feature bf16 [M, dim]).
        Node m lands in cache slot pos+m (reference: kernels/verify_mega.cu:153-158)."""
        tok = torch.as_tensor(tokens, device=self.device).to(torch.int32).contiguous()
        M = tok.numel()
        depth, amask = self._tree_args(M, depth, amask)
        logits = torch.empty(M, self.cfg.vocab_size, dtype=torch.float32, device=self.device) if want_logits else None
        feat = torch.empty(M, self.cfg.dim, dtype=torch.bfloat16, device=self.device)
        _lib.check(self.lib.fb_verify(self._ctx, _ptr(tok), None, _ptr(depth), _ptr(amask), M, int(pos), _ptr(logits),
                                      _ptr(feat), _stream_ptr(self.device)), "fb_verify")
        self._keepalive = (tok, depth, amask)
        return logits, feat

    def verify_h(self, h: torch.Tensor, pos: int, depth, amask):
        """Same, from already multiplied embeddings h bf16 [M, dim] (the reference's calling convention)."""
        M = h.shape[0]
        depth, amask = self._tree_args(M, depth, amask)
        logits = torch.empty(M, self.cfg.vocab_size, dtype=torch.float32, device=self.device)
        feat = torch.empty(M, self.cfg.dim, dtype=torch.bfloat16, device=self.device)
        hc = h.contiguous()
        _lib.check(self.lib.fb_verify(self._ctx, None, _ptr(hc), _ptr(depth), _ptr(amask), M, int(pos), _ptr(logits),
                                      _ptr(feat), _stream_ptr(self.device)), "fb_verify")
        self._keepalive = (hc, depth, amask)
        return logits, feat

    # ------------------------------------------------------------------ token choice and acceptance on the device
    def sample(self, logits: torch.Tensor, temperature: float = 0.0, top_k: Optional[int] = None, seed: int = 0,
               counter: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row of `logits` (f32 [vocab] or [rows, vocab]) without a host sync: arg-max when temperature <= 0,
        else a draw from softmax(logits / temperature) over the top_k entries (reference: engine/generate.py:37-55)."""
        lg = logits if logits.dim() == 2 else logits.view(1, -1)
        if lg.dtype != torch.float32 or lg.stride(-1) != 1:
            raise ValueError("logits must be f32 with contiguous rows")
        rows, vocab = lg.shape
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=lg.device)
        _lib.check(self.lib.fb_sample(_ptr(lg), vocab, rows, lg.stride(0) if rows > 1 else 0, float(temperature),
                                      int(top_k or 0), int(seed), int(counter), _ptr(out), _stream_ptr(self.device)), "fb_sample")
        return out

    def accept_chain(self, target: torch.Tensor, draft: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Device int32 [2]: accepted count and the target's next token (reference: spec_mega.py:106-113)."""
        out = out if out is not None else torch.empty(2, dtype=torch.int32, device=self.device)
        _lib.check(self.lib.fb_accept_chain(_ptr(target), _ptr(draft), int(draft.numel()), _ptr(out),
                                            _stream_ptr(self.device)), "fb_accept_chain")
        return out

    def accept_tree(self, cand: torch.Tensor, parent: torch.Tensor, target: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Device int32 [2 + M]: path length (root included), the target's token at its end, the path's node indices
        (reference: spec_tree.py:108-118)."""
        M = int(cand.numel())
        out = out if out is not None else torch.zeros(2 + M, dtype=torch.int32, device=self.device)
        _lib.check(self.lib.fb_accept_tree(_ptr(cand), _ptr(parent), _ptr(target), M, _ptr(out), _stream_ptr(self.device)),
                   "fb_accept_tree")
        return out

    def kv_compact(self, accept: torch.Tensor, pos: int):
        """Moves the accepted path's cache rows to slots pos+1.. on the device, from accept_tree's output."""
        _lib.check(self.lib.fb_kv_compact(self._ctx, _ptr(accept), int(pos), _stream_ptr(self.device)), "fb_kv_compact")

    def kv_move(self, src, dst):
        """cache[:, dst[i]] = cache[:, src[i]] in order, K and V, every layer (reference: spec_tree.py:126-128)."""
        n = len(src)
        a = (ctypes.c_int32 * n)(*[int(x) for x in src])
        b = (ctypes.c_int32 * n)(*[int(x) for x in dst])
        _lib.check(self.lib.fb_kv_move(self._ctx, a, b, n, _stream_ptr(self.device)), "fb_kv_move")


# --------------------------------------------------------------------------------------------------
# Reference-shaped launch function. The reference infers every dimension from tensor sizes
# (reference: kernels/megakernel_decode.cu:210-211) and so does this wrapper; the context is cached on the
# identity of the weight and cache tensors, so weights are re-laid out once, not per call.
# --------------------------------------------------------------------------------------------------
_engines: Dict[tuple, DecodeEngine] = {}


def _engine_for(Wqkv, s_qkv, Wo, s_o, n1, Wgu, s_gu, Wd, s_d, n2, nf, Wlm, s_lm, h_dim, kc, vc,
                scale, rope_base, resid, logits_scaling) -> DecodeEngine:
    key = (Wqkv.data_ptr(), Wo.data_ptr(), Wgu.data_ptr(), Wd.data_ptr(), Wlm.data_ptr(), kc.data_ptr(), vc.data_ptr(),
           float(scale), float(rope_base), float(resid), float(logits_scaling))
    eng = _engines.get(key)
    if eng is not None:
        return eng
    n_layer, max_seq, n_kv, hd = kc.shape
    dim = int(h_dim)
    cfg = ModelArgs(block_size=max_seq, vocab_size=Wlm.shape[0], n_layer=n_layer, n_head=dim // hd, dim=dim,
                    intermediate_size=Wd.shape[2] * 8, n_local_heads=n_kv, rope_base=rope_base,
                    attention_multiplier=float(scale), residual_multiplier=float(resid),
                    logits_scaling=float(logits_scaling))
    packed = dict(qkv_q=Wqkv, qkv_s=s_qkv, o_q=Wo, o_s=s_o, n1=n1, gu_q=Wgu, gu_s=s_gu, d_q=Wd, d_s=s_d, n2=n2, nf=nf,
                  lm_q=Wlm, lm_s=s_lm)
    eng = DecodeEngine(cfg, packed, max_seq=max_seq, kc=kc, vc=vc)
    _engines[key] = eng
    return eng


def decode_mega_launch(Wqkv, s_qkv, Wo, s_o, n1, Wgu, s_gu, Wd, s_d, n2, nf, Wlm, s_lm, h, kc, vc, pos,
                       scale, rope_base, resid, logits_scaling) -> torch.Tensor:
    """Drop-in for the reference's `decode_mega_launch`: same arguments, returns a new f32 [vocab] logits tensor;
    `h` is clobbered and rows `pos` of kc/vc are written, as in the reference."""
    eng = _engine_for(Wqkv, s_qkv, Wo, s_o, n1, Wgu, s_gu, Wd, s_d, n2, nf, Wlm, s_lm, h.shape[0], kc, vc,
                      scale, rope_base, resid, logits_scaling)
    return eng.decode_h(h, int(pos))


def verify_mega_launch(Wqkv, s_qkv, Wo, s_o, n1, Wgu, s_gu, Wd, s_d, n2, nf, Wlm, s_lm, h, kc, vc, depth, amask, pos, M,
                       scale, rope_base, resid, logits_scaling):
    """Drop-in for the reference's `verify_mega_launch` (reference: kernels/verify_mega.cu:246-283): same arguments,
    returns [logits f32 [M, vocab], feature bf16 [M, dim]]. Any M in 1..64 is accepted."""
    eng = _engine_for(Wqkv, s_qkv, Wo, s_o, n1, Wgu, s_gu, Wd, s_d, n2, nf, Wlm, s_lm, h.shape[1], kc, vc,
                      scale, rope_base, resid, logits_scaling)
    if int(M) != h.shape[0]:
        raise ValueError("M must equal h.shape[0]")
    logits, feat = eng.verify_h(h, int(pos), depth, amask)
    return [logits, feat]


def decode_occupancy():
    """[registers/thread, blocks/SM, #SMs, warps/SM, total warps] (reference: kernels/megakernel_decode.cu:239-245)."""
    c = query(torch.cuda.current_device())
    return [c["regs_decode_kernel"], 1, c["sm_count"], 15, 15 * c["sm_count"]]
