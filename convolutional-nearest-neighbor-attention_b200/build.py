"""Build libconvnn_b200.so in-tree with nvcc for sm_100a (no other architecture).

    python convolutional-nearest-neighbor-attention_b200/build.py [--force] [-v]

Each .cu under csrc/ is compiled to an object file (in parallel) and the objects are
linked into one shared library next to this file.  A source is recompiled when it, any
header under csrc/ or include/, or this script is newer than its object.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libconvnn_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", INCLUDE]


def sources() -> list:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> list:
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h")) + [os.path.abspath(__file__)]


def _obj(src: str) -> str:
    return os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")


def _newer(path: str, than: float) -> bool:
    return os.path.getmtime(path) > than


STAMP = LIB + ".srchash"


def source_hash() -> str:
    """Digest of every file the library is built from (content, not timestamps, so a copy
    of the tree with a prebuilt library is not rebuilt)."""
    import hashlib
    h = hashlib.sha256()
    for f in sorted(sources() + _headers()):
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != source_hash()


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what changed and link; return the library path."""
    if not force and not stale():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    hdr_t = max(os.path.getmtime(h) for h in _headers())
    todo = []
    for s in sources():
        o = _obj(s)
        if force or not os.path.exists(o) or _newer(s, os.path.getmtime(o)) or hdr_t > os.path.getmtime(o):
            todo.append(s)

    def compile_one(s: str):
        cmd = [nvcc] + CFLAGS + ["-c", s, "-o", _obj(s)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r.returncode, " ".join(cmd) + "\n" + r.stdout + r.stderr

    logs = []
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as ex:
        for s, rc, log in ex.map(compile_one, todo):
            logs.append(log)
            if rc != 0:
                raise RuntimeError(f"nvcc failed on {os.path.basename(s)}:\n{log[-8000:]}")
    cmd = [nvcc] + ARCH + ["-shared", "-cudart", "static", "-o", LIB + ".tmp"] + [_obj(s) for s in sources()]
    r = subprocess.run(cmd, capture_output=True, text=True)
    logs.append(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    with open(os.path.join(OBJ, "build.log"), "a" if not force else "w") as f:
        f.write("\n".join(logs))
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + logs[-1][-8000:])
    os.replace(LIB + ".tmp", LIB)
    with open(STAMP, "w") as f:
        f.write(source_hash())
    if verbose:
        print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
