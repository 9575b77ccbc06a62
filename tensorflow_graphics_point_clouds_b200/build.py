"""Builds libtfgpc.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python -m tensorflow_graphics_point_clouds_b200.build [--force] [--verbose]
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libtfgpc.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found")


def sources():
  return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
  paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
  paths += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
  return max(os.path.getmtime(p) for p in paths)


def up_to_date():
  return os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime()


def build(force=False, verbose=False):
  if not force and up_to_date():
    return LIB
  nvcc = _nvcc()
  os.makedirs(OBJ_DIR, exist_ok=True)
  extra = ["-Xptxas", "-v"] if verbose else []

  def compile_one(src):
    obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
    cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
    if verbose:
      sys.stderr.write(res.stderr)
    return obj

  with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
    objs = list(ex.map(compile_one, sources()))
  cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
  return LIB


if __name__ == "__main__":
  print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
