"""Build the reference's own CUDA extensions for sm_100a, in place, as a GPU-side cross-check.

TEST INFRASTRUCTURE ONLY.  Nothing here is copied: the sources are compiled where they lie in a
checkout of lkorinek/convlogic (src/convlogic/cuda, src/difflogic/cuda, src/common) and only the
built modules land in ``oracle/_ref/`` (git-ignored).  The tests and the benchmark use them, when
present, to compare against / time the reference's kernels on the same GPU; they are never on the
product path.

    python oracle/build_ref.py --reference /path/to/convlogic
"""

import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(reference, verbose=False):
    from torch.utils.cpp_extension import load

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    src = os.path.join(reference, "src")
    flags = ["-O3", "-Wno-deprecated-declarations", "-gencode", "arch=compute_100a,code=sm_100a"]
    mods = {
        "convlogic_cuda": [os.path.join(src, "convlogic", "cuda", f) for f in
                           ("convlogic.cpp", "convlogic_kernel.cu", "treelogic_kernel.cu", "full_convlogic_kernel.cu")],
        "difflogic_cuda": [os.path.join(src, "difflogic", "cuda", f) for f in ("difflogic.cpp", "difflogic_kernel.cu")],
    }
    for name, sources in mods.items():
        bdir = os.path.join(OUT, name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=sources, extra_include_paths=[os.path.join(src, "common")], extra_cuda_cflags=flags,
             extra_cflags=["-O3"], build_directory=bdir, verbose=verbose, is_python_module=False)
        print("built", os.path.join(bdir, name + ".so"))


def load_ref(name):
    """Import a built reference module (``convlogic_cuda`` / ``difflogic_cuda``) or return None."""
    import importlib.util

    path = os.path.join(OUT, name, name + ".so")
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    build(a.reference, verbose=True)
