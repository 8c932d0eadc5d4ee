"""TEST INFRASTRUCTURE ONLY: build the reference's own CUDA kernels, from the sources where they lie in the reference
checkout, into oracle/_ref/ (git-ignored). Nothing is copied into this repository.

    python -m oracle.build_ref [/path/to/reference]

Without an argument the checkout is taken from $FLINT_REFERENCE, else from a folder named `reference` beside this
repository.

The two files need nothing but nvcc and the PyTorch extension headers (reference: chat.py:62-63, spec_mega.py:29-31
build them the same way, with -O3 --use_fast_math). The resulting pybind11 modules are used by the GPU tests as a
second checker at the reference's native head shape (40 query / 8 kv heads of 64) and by nothing else.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
TARGETS = {"flint_ref_decode": "kernels/megakernel_decode.cu", "flint_ref_verify": "kernels/verify_mega.cu"}


def build(ref: str = None, verbose: bool = False):
    ref = ref or os.environ.get("FLINT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    if not os.path.isdir(ref):
        raise FileNotFoundError(f"reference checkout not found at {ref}")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    built = []
    for name, rel in TARGETS.items():
        so = os.path.join(OUT, name + ".so")
        src = os.path.join(ref, rel)
        if os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(src):
            built.append(so)
            continue
        load(name=name, sources=[src], extra_cuda_cflags=["-O3", "--use_fast_math", "-gencode",
                                                           "arch=compute_100a,code=sm_100a"],
             build_directory=OUT, verbose=verbose, is_python_module=False)
        built.append(so)
    return built


def load_module(name: str):
    """Import a built module from oracle/_ref (None if it was not built)."""
    so = os.path.join(OUT, name + ".so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
