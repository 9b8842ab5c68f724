"""Builds the sm_100a kernel library in-tree: optimi_b200/lib/liboptimi_b200.so.

    python -m optimi_b200.build [--force]

nvcc cross-compiles without a GPU.  Flags that matter for parity: -fmad=false (the kernels fuse
multiply-adds only where they say so with __fmaf_rn), default IEEE division and square root.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc", "optimi_b200.cu")
DEPS = [SRC, os.path.join(PKG, "csrc", "mta_common.cuh"), os.path.join(PKG, "csrc", "optimizer_ops.cuh"),
        os.path.join(os.path.dirname(PKG), "include", "optimi_b200.h")]  # fmt: skip
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "liboptimi_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false", "-prec-div=true",
    "-prec-sqrt=true", "-ftz=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
]  # fmt: skip


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")


STAMP = LIB + ".srchash"


def source_hash() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for d in DEPS:
        with open(d, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def up_to_date() -> bool:
    """True when the library was built from the sources as they are now (content hash, not mtime)."""
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as fh:
        return fh.read().strip() == source_hash()


N_PARTS = 3  # the source compiles as independent translation units (OPTIMI_PART), built in parallel


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library unless it is current.  Safe against several processes arriving at once (the ranks of
    a multi-GPU job importing the package with a stale library): one builds under a file lock, into a private
    directory, and moves the result into place in one step; the others wait and find it current."""
    if not force and up_to_date():
        return LIB
    import fcntl
    import tempfile

    os.makedirs(LIB_DIR, exist_ok=True)
    with open(os.path.join(LIB_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and up_to_date():  # another process built it while this one waited
            return LIB
        nvcc = find_nvcc()
        ccbin = ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []  # the image's CC/CXX point at a wrapper
        compile_flags = [f for f in NVCC_FLAGS if f not in ("-shared", "--use-local-env")]
        with tempfile.TemporaryDirectory(dir=LIB_DIR, prefix=".build-") as tmp:
            objs, procs = [], []
            for part in range(N_PARTS):
                obj = os.path.join(tmp, f"part{part}.o")
                objs.append(obj)
                cmd = [nvcc, *ccbin, *compile_flags, *(["-Xptxas", "-v"] if verbose else []), f"-DOPTIMI_PART={part}", "-c", "-o", obj, SRC]
                procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
            log = ""
            for cmd, p in procs:
                out, err = p.communicate()
                log += out + err
                if p.returncode != 0:
                    raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + out + err)
            fresh = os.path.join(tmp, "liboptimi_b200.so")
            link = [nvcc, *ccbin, "-shared", "-o", fresh, *objs]
            res = subprocess.run(link, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError("link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
            if os.path.exists(STAMP):
                os.remove(STAMP)  # never a current stamp beside an older library
            os.replace(fresh, LIB)
        if verbose:
            print(log)
        with open(STAMP + ".tmp", "w") as fh:
            fh.write(source_hash())
        os.replace(STAMP + ".tmp", STAMP)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
