"""Build the C-ABI shared library (hand-written sm_100a CUDA) in-tree with nvcc.

    python -m sglang_b200.build            # builds sglang_b200/_lib/libb200_blockfp8.so

The library is compiled for sm_100a only; there is no other code path."""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OUT_DIR = os.path.join(PKG, "_lib")
LIB = os.path.join(OUT_DIR, "libb200_blockfp8.so")
SOURCES = ["status.cu", "quant.cu", "align.cu", "gemm.cu", "moe.cu", "topk.cu", "comm.cu", "ep.cu"]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build sglang_b200")


def _stamp(srcs) -> str:
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(os.path.dirname(PKG), "include")):
        for fn in sorted(os.listdir(root)):
            with open(os.path.join(root, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + srcs).encode())
    return h.hexdigest()


def _up_to_date(stamp: str, stamp_file: str) -> bool:
    return os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library unless ``_lib/build.stamp`` already names this exact set of sources and flags
    (a hash of every file under ``csrc/`` and ``include/``), so an edited source never runs with a stale
    library. Several processes may call this at once (one per GPU): an exclusive file lock lets one of
    them compile while the others wait and then find the stamp current; the library is written under a
    temporary name and renamed into place, so a reader never maps a half-written file."""
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    os.makedirs(OUT_DIR, exist_ok=True)
    stamp_file = os.path.join(OUT_DIR, "build.stamp")
    stamp = _stamp(srcs)
    if not force and _up_to_date(stamp, stamp_file):
        return LIB
    with open(os.path.join(OUT_DIR, "build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and _up_to_date(stamp, stamp_file):  # another process built it while this one waited
            return LIB
        nvcc = _nvcc()
        extra = ["-Xptxas", "-v"] if verbose else []

        def compile_one(src):
            obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
            return obj

        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = f"{LIB}.{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
        with open(stamp_file + ".tmp", "w") as f:
            f.write(stamp)
        os.replace(stamp_file + ".tmp", stamp_file)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
