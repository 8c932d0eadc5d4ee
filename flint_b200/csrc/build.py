"""Build libflintb200.so (sm_100a) in-tree with nvcc. Usage: python -m flint_b200.csrc.build [--force]"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.environ.get("FLINT_B200_BUILD_OUT") or os.path.join(os.path.dirname(HERE), "libflintb200.so")
SOURCES = ["fb_api.cu", "fb_spec.cu"]
HEADERS = sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))) + [os.path.join(ROOT, "include", "flint_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


BUILT_IN_K = (256, 384, 512, 640, 768, 1024, 1280, 1408, 1536, 1792, 2048, 2560, 3584, 4096, 7168, 8192, 14336)


def extra_shape_flags(spec: str):
    """FLINT_B200_EXTRA_SHAPES="dim,ko,ffn,head_dim,gqa[;...]" -> the macros that add decode kernels (and the re-layout
    kernels of their widths) for model shapes the built-in table lacks: a new model is a rebuild, not a source edit.
    ko = attention output width of one rank (= n_head * head_dim on one GPU), gqa = n_head / n_kv_head. Shapes the tile
    schedule cannot serve fail at compile time (static_assert)."""
    shapes = [tuple(int(x) for x in part.split(",")) for part in spec.replace(" ", "").split(";") if part]
    if not shapes:
        return []
    for sh in shapes:
        if len(sh) != 5 or any(v <= 0 for v in sh) or any(v % 128 for v in sh[:3]):
            raise ValueError(f"FLINT_B200_EXTRA_SHAPES: bad shape {sh} (dim,ko,ffn,head_dim,gqa; widths multiples of 128)")
    entries = ",".join("FB_DECODE_ENTRY(%d,%d,%d,%d,%d)" % sh for sh in shapes) + ","
    ks = sorted({k for sh in shapes for k in sh[:3]} - set(BUILT_IN_K))
    flags = ["-DFB_EXTRA_DECODE_ENTRIES=" + entries]
    if ks:
        flags.append("-DFB_EXTRA_K(X)=" + " ".join(f"X({k})" for k in ks))
    return flags


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = os.environ.get("FLINT_B200_NVCC_FLAGS", "").split() + extra_shape_flags(os.environ.get("FLINT_B200_EXTRA_SHAPES", ""))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    # one object per translation unit, compiled side by side, then one link
    procs, objs = [], []
    for src in SOURCES:
        obj = os.path.join(objdir, os.path.splitext(src)[0] + f".{os.getpid()}.o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, os.path.join(HERE, src)]
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, p in procs:
        if p.wait() != 0:
            raise subprocess.CalledProcessError(p.returncode, cmd)
    tmp = LIB + f".tmp{os.getpid()}"
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", tmp] + objs + ["-lcudart"])
    os.replace(tmp, LIB)
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
