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


DEBUG_SUFFIX = "_debug"                       # the build with device-side index checks (csrc/debug.cuh)


def debug_requested() -> bool:
    return os.environ.get("MILES_DEBUG_KERNELS", "0") == "1"


def so_path(debug: bool | None = None) -> str:
    debug = debug_requested() if debug is None else debug
    return os.path.join(BUILD_DIR + (DEBUG_SUFFIX if debug else ""), EXT_NAME + (DEBUG_SUFFIX if debug else "") + ".so")


def build(verbose: bool = False, debug: bool = False):
    """Compile (incrementally, via ninja) and import the extension module.  `debug`: the variant whose kernels check the
    indices they take from tensors (`-DMILES_DEBUG_BOUNDS`; loaded instead of the normal one with MILES_DEBUG_KERNELS=1)."""
    from torch.utils import cpp_extension

    if debug:
        d = BUILD_DIR + DEBUG_SUFFIX
        os.makedirs(d, exist_ok=True)
        os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
        if os.path.exists("/usr/bin/g++"):
            os.environ["CXX"] = "/usr/bin/g++"
            os.environ["CC"] = "/usr/bin/gcc"
        return cpp_extension.load(
            name=EXT_NAME + DEBUG_SUFFIX, sources=sources(), extra_cflags=["-O3", "-std=c++17"],
            extra_cuda_cflags=NVCC_FLAGS + ["-DMILES_DEBUG_BOUNDS"], extra_include_paths=[CSRC], build_directory=d, verbose=verbose,
            with_cuda=True, is_python_module=True)
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

    debug = debug_requested()
    path = so_path(debug)
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build the CUDA extension with `python -m miles_b200.ops.build` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`)")
    spec = importlib.util.spec_from_file_location(EXT_NAME + (DEBUG_SUFFIX if debug else ""), path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    import sys

    m = build(verbose="-v" in sys.argv, debug="--debug" in sys.argv)
    print("built", so_path("--debug" in sys.argv), "with", len([n for n in dir(m) if not n.startswith("_")]), "entry points")
