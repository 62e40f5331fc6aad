"""Build and load the `nanotitan_cuda` extension (sm_100a only, in-tree).

`build_extension()` compiles every source under `nanotitan_b200/csrc` with
``-gencode arch=compute_100a,code=sm_100a`` into `nanotitan_b200/csrc/_build/`
(nvcc cross-compiles, no GPU needed).  `get_ext()` imports the built shared object
from that folder; it never falls back to another implementation: on a machine with
a GPU a missing extension is an error, not a silent slow path.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from functools import lru_cache
from pathlib import Path
from types import ModuleType

CSRC = Path(__file__).resolve().parent.parent / "csrc"
BUILD_DIR = CSRC / "_build"
EXT_NAME = "nanotitan_cuda"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xptxas", "-v",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]


def sources() -> list[str]:
    found = sorted(str(p) for p in CSRC.rglob("*.cu") if "_build" not in p.parts)
    found += sorted(str(p) for p in CSRC.rglob("*.cpp") if "_build" not in p.parts and "standalone" not in p.parts)
    return found


def so_path() -> Path | None:
    hits = sorted(BUILD_DIR.glob(f"{EXT_NAME}*.so"), key=lambda p: p.stat().st_mtime)
    return hits[-1] if hits else None  # the newest, when both build routes have left one


def build_extension(verbose: bool = False) -> Path:
    """Compile (incrementally, with ninja) and return the path of the shared object."""
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    # The arch comes from NVCC_FLAGS; keep torch from appending its own list for the visible GPU.
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    cpp_extension.load(
        name=EXT_NAME,
        sources=sources(),
        extra_include_paths=[str(CSRC), str(CSRC / "runtime")],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        build_directory=str(BUILD_DIR),
        verbose=verbose,
        is_python_module=True,
    )
    path = so_path()
    if path is None:
        raise RuntimeError(f"build finished but no {EXT_NAME}*.so in {BUILD_DIR}")
    get_ext.cache_clear()
    return path


def have_ext() -> bool:
    return so_path() is not None


@lru_cache
def get_ext() -> ModuleType:
    path = so_path()
    if path is None:
        raise RuntimeError(
            f"The {EXT_NAME} extension is not built. Run `python -c 'import __graft_entry__ as g; "
            "g.build()'` (or nanotitan_b200.ops.ext.build_extension()) first."
        )
    import torch  # noqa: F401  (libtorch symbols must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[EXT_NAME] = module
    return module


def native(t) -> bool:
    """True when `t` lives on a GPU, where the CUDA kernels are the code path."""
    return t.is_cuda


# ------------------------------------------------------------------ type stub
STUB_PATH = Path(__file__).resolve().parent / f"{EXT_NAME}.pyi"


def stub_text() -> str:
    """A .pyi for the built extension, from the signatures pybind11 puts in the first docstring line."""
    import re

    ext = get_ext()

    def clean(sig: str) -> str:
        sig = sig.replace("torch.Tensor", "Tensor")
        sig = re.sub(r"collections\.abc\.Sequence\[([^\]]+)\]", r"list[\1]", sig)
        sig = sig.replace("typing.SupportsInt", "int").replace("typing.SupportsFloat", "float")
        return re.sub(rf"self: {EXT_NAME}\.\w+", "self", sig)

    out = [f'"""Type stub of the `{EXT_NAME}` extension, generated from the signatures pybind11 records',
           "(`python -m nanotitan_b200.ops.ext --stub` rewrites it).  The module itself is built from nanotitan_b200/csrc",
           'and loaded by `nanotitan_b200.ops.ext.get_ext()`."""',
           "from __future__ import annotations", "", "import torch", "", "Tensor = torch.Tensor", ""]
    for name in sorted(n for n in dir(ext) if not n.startswith("_")):
        obj = getattr(ext, name)
        doc = (obj.__doc__ or "").strip().splitlines()
        if isinstance(obj, type):
            out.append(f"class {name}:")
            for member in sorted(m for m in dir(obj) if not m.startswith("_") or m == "__init__"):
                first = (getattr(obj, member).__doc__ or "").strip().splitlines()[:1]
                if first and first[0].startswith(member + "("):
                    out.append(f"    def {clean(first[0])}: ...")
                else:
                    out.append(f"    {member}: int")
            out.append("")
        elif doc and doc[0].startswith(name + "("):
            out.append(f"def {clean(doc[0])}:")
            rest = " ".join(x.strip() for x in doc[1:] if x.strip())
            out.append(f'    """{rest}"""' if rest else "    ...")
            out.append("")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    if "--stub" in sys.argv:
        STUB_PATH.write_text(stub_text())
        print(f"wrote {STUB_PATH}")
    else:
        print(build_extension(verbose="--verbose" in sys.argv))
