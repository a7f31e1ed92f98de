"""Build the C-ABI shared library (libcache_dit_b200.so) in-tree with nvcc for sm_100a.

    python -m cache_dit_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  cudart is linked statically and the driver API entry point
needed for tensor maps is resolved at run time, so the library loads on a machine with no driver.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_NAME = "libcache_dit_b200.so"
LIB_PATH = os.path.join(PKG, LIB_NAME)
SOURCES = ["lib.cu", "cache_kernels.cu", "fp8_quant.cu", "fp8_gemm.cu", "glue_kernels.cu", "peer_kernels.cu"]
HEADERS = ["common.cuh", os.path.join("..", "..", "include", "cache_dit_b200.h")]
NVCC_FLAGS = [
  "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
  "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not os.path.exists(nvcc):
    raise RuntimeError("nvcc not found: the CUDA kernels of cache_dit_b200 cannot be built")
  return nvcc


def is_stale() -> bool:
  if not os.path.exists(LIB_PATH):
    return True
  built = os.path.getmtime(LIB_PATH)
  deps = [os.path.join(HERE, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
  return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
  if not force and not is_stale():
    return LIB_PATH
  nvcc = find_nvcc()
  objs = []
  build_dir = os.path.join(HERE, "build")
  os.makedirs(build_dir, exist_ok=True)
  procs = []
  for src in SOURCES:
    obj = os.path.join(build_dir, src.replace(".cu", ".o"))
    objs.append(obj)
    cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
    if verbose:
      cmd[1:1] = ["-Xptxas", "-v"]
      print(" ".join(cmd), flush=True)
    procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
  failed = False
  for src, p in procs:
    out, _ = p.communicate()
    if verbose or p.returncode != 0:
      print(out, flush=True)
    failed = failed or p.returncode != 0
  if failed:
    raise RuntimeError("nvcc failed; see output above")
  link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-cudart", "static", "-Xlinker", "--exclude-libs,ALL"]
  r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
  if r.returncode != 0:
    print(r.stdout)
    raise RuntimeError("linking libcache_dit_b200.so failed")
  return LIB_PATH


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--force", action="store_true")
  ap.add_argument("--verbose", action="store_true")
  a = ap.parse_args()
  print(build(force=a.force, verbose=a.verbose))
