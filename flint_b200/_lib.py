"""ctypes binding of libflintb200.so (the C ABI declared in include/flint_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be resolved, import of the
product path fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLINT_B200_LIB", os.path.join(HERE, "libflintb200.so"))

FB_OK, FB_ERR_ARG, FB_ERR_SHAPE, FB_ERR_CUDA, FB_ERR_STATE, FB_ERR_TIMEOUT, FB_ERR_RANGE = range(7)
ERR_NAMES = {0: "FB_OK", 1: "FB_ERR_ARG", 2: "FB_ERR_SHAPE", 3: "FB_ERR_CUDA", 4: "FB_ERR_STATE",
             5: "FB_ERR_TIMEOUT", 6: "FB_ERR_RANGE"}


class FlintError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {ERR_NAMES.get(code, code)}")
        self.code = code


class Caps(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("device", "sm_count", "cc_major", "cc_minor", "smem_per_block_optin",
                                              "l2_bytes", "cooperative_launch", "regs_decode_kernel")] + \
               [("total_mem_bytes", ctypes.c_int64)]


class ModelDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("n_layer", "dim", "n_head", "n_kv_head", "head_dim", "ffn", "vocab",
                                              "has_zeros")] + \
               [(n, ctypes.c_float) for n in ("rms_eps", "rope_base", "attn_scale", "resid_mult", "emb_mult",
                                              "logits_scaling")]


WEIGHT_FIELDS = ("qkv_q", "qkv_s", "qkv_z", "o_q", "o_s", "o_z", "gu_q", "gu_s", "gu_z", "d_q", "d_s", "d_z",
                 "lm_q", "lm_s", "lm_z", "n1", "n2", "nf", "embed")


class WeightPtrs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in WEIGHT_FIELDS]


class DraftDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("dim", "n_head", "n_kv_head", "inter", "fuse", "vocab", "max_roll",
                                              "max_tokens")] + \
               [(n, ctypes.c_float) for n in ("rope_base", "rms_eps", "logits_scaling")]


DRAFT_WEIGHT_FIELDS = ("merge", "n1", "n2", "q", "k", "v", "o", "gate", "up", "down", "fout", "nf", "embed")


class DraftWeights(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in DRAFT_WEIGHT_FIELDS]


class Status(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("code", "cuda_error", "where", "layer", "block", "expected", "seen")]


# every symbol include/flint_b200.h declares, with its prototype
_PROTOS = {
    "fb_query": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(Caps)]),
    "fb_ctx_create": (ctypes.c_int, [ctypes.POINTER(ModelDesc), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]),
    "fb_ctx_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "fb_ctx_create_tp": (ctypes.c_int, [ctypes.POINTER(ModelDesc), ctypes.c_int, ctypes.c_int32, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]),
    "fb_tp_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "fb_tp_connect": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32]),
    "fb_tp_connect_local": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32]),
    "fb_last_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Status)]),
    "fb_bind_weights": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(WeightPtrs), ctypes.c_void_p]),
    "fb_bind_kv": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32]),
    "fb_decode": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_stream_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
    "fb_repack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                 ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_dequant": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                  ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_gemv": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                               ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                               ctypes.c_void_p]),
    "fb_gemv_static": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_set_option": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64]),
    "fb_verify": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                 ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_kv_compact": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]),
    "fb_sample": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_float,
                                 ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_accept_chain": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_accept_tree": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p,
                                      ctypes.c_void_p]),
    "fb_draft_create": (ctypes.c_int, [ctypes.POINTER(DraftDesc), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]),
    "fb_draft_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "fb_draft_bind": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(DraftWeights)]),
    "fb_draft_forward": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "fb_draft_head": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p]),
    "fb_kv_move": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32),
                                  ctypes.c_int32, ctypes.c_void_p]),
}
EXPORTED_SYMBOLS = tuple(_PROTOS)

_lib = None


def load() -> ctypes.CDLL:
    """Load the library and bind every prototype; raises if the CUDA extension has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m flint_b200.csrc.build` "
                          "(nvcc, sm_100a); there is no CPU fallback")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _PROTOS.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str):
    if code != FB_OK:
        raise FlintError(code, what)
