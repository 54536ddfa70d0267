"""Builds libxb200.so (every kernel, one translation unit, sm_100a) inside the package directory.

Used by ``__graft_entry__.build()`` and by the command-line tools on their first call in a fresh checkout: nvcc
cross-compiles without a GPU, the result is written under a temporary name and renamed, so two processes that
build at once leave one whole library."""
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libxb200.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def find_nvcc() -> str:
  cand = [os.environ.get("NVCC"), os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"]
  for c in cand:
    if c and os.path.exists(c):
      return c
  return "nvcc"


def stale() -> bool:
  if not LIB.exists():
    return True
  t = LIB.stat().st_mtime
  srcs = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "xb200.h"]
  return any(s.stat().st_mtime > t for s in srcs)


def ensure_built(force: bool = False, quiet: bool = False) -> Path:
  if force or stale():
    tmp = PKG / f".libxb200.{os.getpid()}.so"
    cmd = [find_nvcc(), *NVCC_FLAGS, "-o", str(tmp), str(CSRC / "xb_engine.cu")]
    if not quiet:
      print("[build]", " ".join(cmd), file=sys.stderr, flush=True)
    try:
      subprocess.run(cmd, check=True, stdout=sys.stderr)
      os.replace(tmp, LIB)
    finally:
      if tmp.exists():
        tmp.unlink()
  return LIB
