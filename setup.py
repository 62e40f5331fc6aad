"""`pip install -e .` / `python setup.py build_ext --inplace`: the package plus its sm_100a extension.

The reference builds one `CUDAExtension("nanotitan_cuda")` with no architecture flags (its setup.py:8-36).
Here the same module name is built for sm_100a only, from every source under `nanotitan_b200/csrc`, with the
flags `nanotitan_b200.ops.ext` uses for its in-place ninja build, and lands in `nanotitan_b200/csrc/_build/`,
where `nanotitan_b200.ops.ext.get_ext()` looks for it.  Either route gives the same shared object; the
in-place build (`python -c 'import __graft_entry__ as g; g.build()'`) is incremental and needs no install.
"""
import os
import sys
from pathlib import Path

from setuptools import find_packages, setup

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))  # build front ends run this file from elsewhere; the source list lives in the package


def extension():
    from torch.utils.cpp_extension import CUDAExtension

    from nanotitan_b200.ops import ext

    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"  # the -gencode flag below is the one that counts
    ext.BUILD_DIR.mkdir(parents=True, exist_ok=True)  # where `build_ext --inplace` puts the module
    sources = [os.path.relpath(s, ROOT) for s in ext.sources()]
    flags = [f for f in ext.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
    return CUDAExtension(
        name="nanotitan_b200.csrc._build." + ext.EXT_NAME,
        sources=sources,
        include_dirs=[str(ext.CSRC), str(ext.CSRC / "runtime")],
        extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": flags},
    )


def build_ext_command():
    from torch.utils.cpp_extension import BuildExtension

    return BuildExtension.with_options(use_ninja=True)


if __name__ == "__main__":
    setup(
        packages=find_packages(include=["nanotitan_b200*", "src*", "scripts*"]),
        ext_modules=[extension()],
        cmdclass={"build_ext": build_ext_command()},
    )
