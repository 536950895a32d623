"""In-tree build of the two shared libraries of the operator.

* ``libpaged_fp8_decode.so`` -- CUDA kernels + C ABI (``include/paged_fp8_decode.h``),
  compiled by ``nvcc`` for sm_100a only, no torch headers.
* ``l20_paged_decode_ops.so`` -- the ``TORCH_LIBRARY(l20_stack)`` dispatcher surface, compiled
  by ``g++`` against the installed torch, linked to the first library through ``$ORIGIN``.
  The file name is the one the reference wrapper loads
  (integrations/vllm/l20_paged_decode.py:11-17).

Both cross-compile on a machine without a GPU.  ``python -m single_gpu_inference_lab_b200.build``
builds whatever is stale.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
CABI_LIB = PKG / "libpaged_fp8_decode.so"
OPS_LIB = PKG / "l20_paged_decode_ops.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return found


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def cabi_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [INCLUDE / "paged_fp8_decode.h"]


def build_cabi(force: bool = False, verbose: bool = False) -> Path:
    sources = cabi_sources()
    if force or _stale(CABI_LIB, sources):
        cmd = [_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-o", str(CABI_LIB)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += [str(s) for s in sources if s.suffix == ".cu"]
        _run(cmd)
    return CABI_LIB


def build_torch_ops(force: bool = False) -> Path:
    src = CSRC / "l20_paged_decode_ops.cpp"
    build_cabi()
    if force or _stale(OPS_LIB, [src, INCLUDE / "paged_fp8_decode.h"]):
        import torch
        from torch.utils import cpp_extension

        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        torch_lib = Path(torch.__file__).parent / "lib"
        cmd = [
            "g++", "-O2", "-std=c++17", "-fPIC", "-shared",
            "-DTORCH_EXTENSION_NAME=l20_paged_decode_ops",
            "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
            *[f"-I{p}" for p in cpp_extension.include_paths()],
            f"-I{cuda_home}/include", f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}",
            str(src), "-o", str(OPS_LIB),
            f"-L{PKG}", "-lpaged_fp8_decode",
            f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-ltorch_python",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
        ]
        _run(cmd)
    return OPS_LIB


def build_all(force: bool = False) -> tuple[Path, Path]:
    return build_cabi(force), build_torch_ops(force)


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv)
    for lib in libs:
        print(lib)
