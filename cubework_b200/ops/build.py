"""Builds the CUDA extension in-tree for sm_100a (``cubework_b200/ops/_C*.so``).

``python -m cubework_b200.ops.build`` or ``build()``; compiles only what changed (ninja).  nvcc
cross-compiles, so this runs on a machine without a GPU.
"""
import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")
NAME = "cubework_b200_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xptxas", "-v", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def so_path():
    return os.path.join(HERE, NAME + ".so")


NOALLOC_SRC = os.path.join(CSRC, "noalloc", "noalloc_layer_norm_bwd.cu")


def noalloc_so_path():
    return os.path.join(HERE, "libcubework_noalloc.so")


def build_noalloc(verbose=False):
    """The allocation-free entry point is a plain CUDA library (no torch, no Python): one nvcc call."""
    import subprocess
    out = noalloc_so_path()
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(NOALLOC_SRC),
                                                            os.path.getmtime(NOALLOC_SRC[:-3] + ".h")):
        return out
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-o", out, NOALLOC_SRC]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    subprocess.run(cmd, check=True)
    return out


def build(verbose=False):
    build_noalloc(verbose)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    from torch.utils import cpp_extension
    os.makedirs(BUILD_DIR, exist_ok=True)
    cpp_extension.load(name=NAME, sources=sources(), extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=NVCC_FLAGS, extra_ldflags=["-lcuda"], build_directory=BUILD_DIR,
                       verbose=verbose, is_python_module=False)
    built = os.path.join(BUILD_DIR, NAME + ".so")
    if not os.path.exists(built):
        raise RuntimeError(f"build produced no {built}")
    shutil.copy2(built, so_path())
    return so_path()


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
