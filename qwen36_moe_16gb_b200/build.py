"""Build ``libb200moe.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import hashlib
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libb200moe.so"
SOURCES = ("api.cu", "routing.cu", "slot_cache.cu", "decode.cu", "prefill.cu", "glue.cu", "dense.cu")
HEADERS = (CSRC / "common.cuh", CSRC / "router.cuh", CSRC / "tc.cuh", HERE.parent / "include" / "b200moe.h")


def source_digest() -> str:
    h = hashlib.sha256()
    for f in [CSRC / s for s in SOURCES] + list(HEADERS):
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    stamp = HERE / ".libb200moe.stamp"
    digest = source_digest()
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", f"-DB200MOE_BUILD_ID=\"b200moe sm_100a {digest}\"", "-o", str(LIB)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    stamp.write_text(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
