"""Builds libmoba_b200.so (sm_100a only) in-tree with nvcc.

Usage: python build.py [--force] [--verbose]
The library lands next to the host package (moba_opt/libmoba_b200.so).
"""
import hashlib
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "moba_opt" / "libmoba_b200.so"
STAMP = HERE / "moba_opt" / ".libmoba_b200.stamp"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "--expt-relaxed-constexpr",
    "-I", str(HERE.parent / "include"), "-I", str(CSRC),
] + os.environ.get("MOBA_NVCC_EXTRA", "").split()


def _digest(sources):
    h = hashlib.sha256()
    for p in sorted(sources + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    sources = sorted(CSRC.glob("*.cu"))
    digest = _digest(sources)
    if not force and OUT.exists() and STAMP.exists() and STAMP.read_text() == digest:
        return OUT
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    procs = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src.name}")
        if verbose or "warning" in out:
            sys.stderr.write(out)
        objs.append(str(obj))
    cmd = [NVCC, "-shared", "-Wno-deprecated-gpu-targets", "-o", str(OUT), *objs, "-lcudart"]
    subprocess.run(cmd, check=True)
    STAMP.write_text(digest)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
