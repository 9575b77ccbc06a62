"""Compiles the reference's own CUDA kernels, where they lie under the reference
checkout, behind oracle/ref_kernels_harness.cu into oracle/_ref/ (TEST
INFRASTRUCTURE; git-ignored output).  Only possible where the reference tree is
mounted; on a machine without it the prebuilt library is used if present.

Usage: python oracle/build_ref.py [/path/to/reference]
(default: $TFG_REFERENCE_DIR, else ../reference relative to the repository)
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libtfg_ref_kernels.so")
# Where a checkout of the reference project lies (only needed to rebuild the
# library): TFG_REFERENCE_DIR, else a directory named "reference" beside this
# repository.
DEFAULT_REFERENCE = os.environ.get(
    "TFG_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def build(reference=DEFAULT_REFERENCE, force=False):
  ops_root = os.path.join(reference, "custom_ops")
  sources = sorted(glob.glob(os.path.join(ops_root, "tfg_custom_ops", "*", "cc", "kernels",
                                          "*_kernels.cu.cc")))
  if not sources:
    return LIB if os.path.exists(LIB) else None
  harness = os.path.join(HERE, "ref_kernels_harness.cu")
  if (not force and os.path.exists(LIB)
      and os.path.getmtime(LIB) >= max(os.path.getmtime(p) for p in sources + [harness])):
    return LIB
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  os.makedirs(OUT_DIR, exist_ok=True)
  # the reference's own flags (compute_keys/BUILD:44-45) plus the sm_100a target
  flags = ["-x", "cu", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
           "--expt-relaxed-constexpr", "-ftz=true", "-Xcompiler", "-fPIC", "-I", ops_root, "-w"]

  def compile_one(src):
    obj = os.path.join(OUT_DIR, os.path.basename(src).replace(".cu.cc", ".o").replace(".cu", ".o"))
    res = subprocess.run([nvcc] + flags + ["-c", src, "-o", obj], capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError("nvcc failed for %s:\n%s" % (src, res.stderr))
    return obj

  with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
    objs = list(ex.map(compile_one, sources + [harness]))
  res = subprocess.run([nvcc, "-shared", "-o", LIB] + objs +
                       ["-gencode", "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("link failed:\n%s" % res.stderr)
  for o in objs:
    os.remove(o)
  return LIB


if __name__ == "__main__":
  print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE, force=True))
