"""In-tree build of the two native pieces of the package, for sm_100a only.

  1. gemm_kernels/libgemm_sm100.so  - CUDA kernels + C ABI (include/gemm_sm100.h), nvcc, no torch.
  2. gemm_kernels/_C.*.so           - the PyTorch binding (gemm_kernels/__init__.cpp), g++, links 1.

The reference builds one CUDAExtension from __init__.cpp + sm90a/gemm_test.cu with
-arch=sm_90a (kernels/setup.py:10-24, build.sh:6-7).  Here the kernel library is kept free
of torch headers, so it compiles in seconds and can be loaded by non-Python hosts.

Usage:  python build_native.py [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
PKG = HERE / "gemm_kernels"
CSRC = HERE / "csrc"
LIB = PKG / "libgemm_sm100.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--restrict",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; this package builds for sm_100a only and needs CUDA >= 12.8")
    return cand


def _cxx() -> str:
    """Host compiler of the torch binding.  GEMM_KERNELS_CXX overrides; otherwise the system g++ is
    preferred over $CXX: a $CXX compiler wrapper that re-orders the C++ standard include
    directories produced a binding whose error messages with integer arguments crashed inside
    iostream formatting."""
    override = os.environ.get("GEMM_KERNELS_CXX")
    if override:
        return override
    if Path("/usr/bin/g++").exists():
        return "/usr/bin/g++"
    return os.environ.get("CXX", "g++")


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"command failed ({res.returncode}): {' '.join(cmd)}")
    if verbose:
        sys.stdout.write(res.stdout + res.stderr)


def ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_C{suffix}"


def build_kernel_library(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [REPO / "include" / "gemm_sm100.h"]
    if not force and _newer(LIB, sources):
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB)] + [str(s) for s in sorted(CSRC.glob("*.cu"))]
    _run(cmd, verbose)
    return LIB


def build_torch_binding(force: bool = False, verbose: bool = False) -> Path:
    out = ext_path()
    src = PKG / "__init__.cpp"
    if not force and _newer(out, [src, REPO / "include" / "gemm_sm100.h", LIB]):
        return out
    from torch.utils import cpp_extension as ce

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes = ce.include_paths() + [sysconfig.get_paths()["include"], f"{cuda_home}/include"]
    import torch

    # The macros torch's own extension builder passes: above all the libstdc++ ABI the installed
    # torch was built with (std::string crosses the boundary in error messages and option names).
    cmd = [_cxx(), "-O3", "-Wall", "-Wextra", "-std=c++17", "-fPIC", "-shared",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [str(src), "-o", str(out)]
    for lp in ce.library_paths():
        cmd += [f"-L{lp}", f"-Wl,-rpath,{lp}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
            f"-L{PKG}", "-l:libgemm_sm100.so", "-Wl,-rpath,$ORIGIN", "-Wl,--no-as-needed"]
    _run(cmd, verbose)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernel_library(force, verbose)
    build_torch_binding(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    print(f"built {LIB.name} and {ext_path().name} in {PKG}")
