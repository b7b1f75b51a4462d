"""Build the sm_100a extension in-tree: ``python -m odysseus_transformer_b200.build_ext``.

The kernels are compiled only for Blackwell (``-gencode arch=compute_100a,code=sm_100a``); nvcc
cross-compiles without a GPU.  The result is ``odysseus_transformer_b200/_C.so`` next to this file,
so it travels with the source tree and is the library Python imports.
"""
from __future__ import annotations

import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")

# ODY_EXTRA_NVCC_FLAGS: extra flags for development builds, e.g. -DODY_ATTN_TRACE (clock-stamp timelines of the attention kernels)
NVCC_FLAGS = os.environ.get("ODY_EXTRA_NVCC_FLAGS", "").split() + ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cpp")) + glob.glob(os.path.join(CSRC, "*.cu")))


def _stamp() -> str:
    import hashlib
    h = hashlib.sha256()
    for f in sorted(glob.glob(os.path.join(CSRC, "*"))):
        if os.path.isfile(f):
            h.update(f.encode())
            h.update(open(f, "rb").read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile (if sources changed) and return the path of the built ``_C.so``."""
    target = os.path.join(HERE, "_C.so")
    stamp_file = os.path.join(BUILD, "stamp")
    stamp = _stamp()
    if not force and os.path.exists(target) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return target
    from torch.utils import cpp_extension
    os.makedirs(BUILD, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name="_C", sources=sources(), extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=["-lcuda"] if False else [], build_directory=BUILD, verbose=verbose, is_python_module=False)
    built = os.path.join(BUILD, "_C.so")
    shutil.copyfile(built, target + ".tmp")
    os.replace(target + ".tmp", target)      # readers of the tree never see a half-written library
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return target


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
