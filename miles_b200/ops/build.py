"""Build the in-tree CUDA extension for sm_100a.

`python -m miles_b200.ops.build` compiles every `.cu` / `.cpp` under `csrc/` with
`-gencode arch=compute_100a,code=sm_100a -lineinfo` into `miles_b200/ops/_build/miles_b200_C.so`.
nvcc cross-compiles without a GPU, so the build also runs on CPU-only machines; the resulting `.so`
stays in the tree (git-ignored) and is what `miles_b200.ops.cuda` loads at run time.
"""
from __future__ import annotations

import glob
import os

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")
EXT_NAME = "miles_b200_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT162_OPERATORS__",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def so_path() -> str:
    return os.path.join(BUILD_DIR, EXT_NAME + ".so")


def build(verbose: bool = False):
    """Compile (incrementally, via ninja) and import the extension module."""
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    # link against the system libstdc++.so (the same one libtorch uses); a toolchain that links it statically
    # gives the extension a second, uninitialised copy of the iostream state
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    # torch adds its own -gencode list unless it finds one in the flags; ours targets sm_100a only
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return cpp_extension.load(
        name=EXT_NAME, sources=sources(), extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[CSRC], build_directory=BUILD_DIR, verbose=verbose, with_cuda=True)


def load():
    """Import the already-built extension from the tree (no compilation)."""
    import importlib.util

    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    path = so_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build the CUDA extension with `python -m miles_b200.ops.build` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`)")
    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    import sys

    m = build(verbose="-v" in sys.argv)
    print("built", so_path(), "with", len([n for n in dir(m) if not n.startswith("_")]), "entry points")
