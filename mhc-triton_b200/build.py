"""Build libmhc_b200.so (the C-ABI library) for sm_100a with nvcc.

    python mhc-triton_b200/build.py [--force] [--verbose]

The shared object is written next to the Python package (mhc/libmhc_b200.so); it links only
against the CUDA runtime (statically), not against PyTorch.
"""

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "mhc", "libmhc_b200.so")
SOURCES = ["api.cu", "sinkhorn.cu", "stream.cu", "weights.cu", "weights_rows.cu", "weights_rows_tc.cu", "fused.cu", "noalloc.cu"]
HEADERS = ["common.cuh", "launch.h", os.path.join("..", "..", "include", "mhc_b200.h")]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False, defines=(), out=OUT):
    if not force and out == OUT and up_to_date():
        return OUT
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "-cudart", "static"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [f"-D{d}" for d in defines]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        print(res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("-D", dest="defines", action="append", default=[], help="tuning macro, e.g. -D MHC_TPC_MAX=16")
    ap.add_argument("--out", default=OUT)
    a = ap.parse_args()
    print(build(a.force or bool(a.defines) or a.out != OUT, a.verbose, a.defines, a.out))
