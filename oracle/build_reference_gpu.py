"""Build the reference project's own CUDA kernels for sm_100a, from its sources where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE, not product: the built modules are only loaded by fa_bench/reference_gpu.py (a same-GPU
comparison row) and never by the library.  The reference compiles each kernel version as a torch C++ extension
(its bindings/load.py:107-131: `torch.utils.cpp_extension.load` on `<version>/<name>.cu` + `binding.cpp`); this
recipe does the same with an explicit sm_100a target and a build directory under oracle/_ref/, so that the
shared objects travel to a GPU machine that has no copy of the reference.

    python oracle/build_reference_gpu.py /path/to/reference [version ...]      # or FA_B200_REFERENCE_ROOT
"""

from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# kernel versions of the hot path and their source files (reference bindings/load.py:21-38)
SOURCES = {
    "v5_wmma": ["wmma_attention.cu", "binding.cpp"],
    "v8_gqa_ss": ["gqa_ss_attention.cu", "binding.cpp"],
    "v9_fp8": ["fp8_attention.cu", "binding.cpp"],
    "v10_nvfp4": ["nvfp4_attention.cu", "binding.cpp"],
    "v11_mla": ["mla_attention.cu", "binding.cpp"],
}


def build(reference_root: str, versions=None) -> list:
    from torch.utils.cpp_extension import load
    built = []
    for name in versions or SOURCES:
        src_dir = os.path.join(reference_root, "kernels", name)
        sources = [os.path.join(src_dir, f) for f in SOURCES[name]]
        if not all(os.path.exists(s) for s in sources):
            print(f"{name}: sources not found under {src_dir}, skipped")
            continue
        build_dir = os.path.join(OUT, name)
        os.makedirs(build_dir, exist_ok=True)
        load(name=f"fa_{name}", sources=sources, build_directory=build_dir, verbose=False,
             extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a"])
        built.append(os.path.join(build_dir, f"fa_{name}.so"))
        print(f"{name}: {built[-1]}")
    return built


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 and os.path.isdir(sys.argv[1]) else os.environ.get("FA_B200_REFERENCE_ROOT", "")
    names = [a for a in sys.argv[1:] if a in SOURCES]
    if not root:
        raise SystemExit("usage: build_reference_gpu.py /path/to/reference [version ...]")
    build(root, names or None)
