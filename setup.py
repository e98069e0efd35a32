"""Builds and installs ``cubework_b200`` together with its CUDA extension.

``pip install .`` (or ``python setup.py build_ext --inplace`` in a checkout) compiles every source under
``cubework_b200/ops/csrc`` for sm_100a (``-gencode arch=compute_100a,code=sm_100a``; nvcc cross-compiles, no GPU is
needed at build time) into ``cubework_b200/ops/cubework_b200_C.so`` and the allocation-free plain-C library
``libcubework_noalloc.so`` next to it.  The flags are the ones of :mod:`cubework_b200.ops.build`, which remains the
way to rebuild in place during development (``python -m cubework_b200.ops.build``).

The reference package is pure Python (setup.py:23-37 declares no extension); everything built here is new.
"""
import glob
import os
import subprocess

from setuptools import setup

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("cubework_b200", "ops", "csrc")


def _nvcc_flags():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_cw_build", os.path.join(HERE, "cubework_b200", "ops", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _extensions():
    from torch.utils.cpp_extension import CUDAExtension
    b = _nvcc_flags()
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))
    return [CUDAExtension(name="cubework_b200.ops.cubework_b200_C", sources=sources,
                          extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": list(b.NVCC_FLAGS)},
                          libraries=["cuda"])]


def _build_ext_class():
    from torch.utils.cpp_extension import BuildExtension

    class BuildWithNoAlloc(BuildExtension):
        """Also builds the stand-alone allocation-free library (plain nvcc, no torch)."""

        def run(self):
            super().run()
            b = _nvcc_flags()
            out_dir = os.path.join(self.build_lib, "cubework_b200", "ops") if not self.inplace else \
                os.path.join(HERE, "cubework_b200", "ops")
            os.makedirs(out_dir, exist_ok=True)
            subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
                            "-Xcompiler", "-fPIC", "-o", os.path.join(out_dir, "libcubework_noalloc.so"), b.NOALLOC_SRC],
                           check=True)

        def get_ext_filename(self, ext_name):
            # the loader (cubework_b200/ops/ext.py) opens the library under a fixed name, without the ABI tag
            return os.path.join(*ext_name.split(".")) + ".so"

    return BuildWithNoAlloc.with_options(no_python_abi_suffix=True)


os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
setup(ext_modules=_extensions(), cmdclass={"build_ext": _build_ext_class()},
      package_data={"cubework_b200.ops": ["csrc/*", "csrc/noalloc/*", "*.so"]})
