"""In-tree nvcc build of libgnk.so (sm_100a only).

`python -m gn_kernels_b200.build` compiles every csrc/*.cu with
`-gencode arch=compute_100a,code=sm_100a` and links one shared library next to this file.
The library has no link-time dependency on libcuda (driver entry points are looked up at
run time) and links the CUDA runtime statically.
"""

from __future__ import annotations

import contextlib
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libgnk.so")
OBJ_DIR = os.path.join(PKG_DIR, "build")
STAMP_PATH = LIB_PATH + ".stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-diag-suppress", "177",
]


def find_nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def source_digest() -> str:
    """Hash of every file the library is built from (file times do not survive a copy)."""
    h = hashlib.sha256()
    files = sources() + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cuh", ".h"))]
    files += [os.path.join(INCLUDE, f) for f in sorted(os.listdir(INCLUDE))]
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(STAMP_PATH):
        return True
    with open(STAMP_PATH) as fh:
        return fh.read().strip() != source_digest()


@contextlib.contextmanager
def _build_lock():
    """Exclusive inter-process lock: ranks started together (torchrun) must not compile into the
    same object files, or load a library another rank is still writing."""
    fh = open(LIB_PATH + ".lock", "w")
    try:
        fcntl.flock(fh, fcntl.LOCK_EX)
        yield
    finally:
        fcntl.flock(fh, fcntl.LOCK_UN)
        fh.close()


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None) -> str:
    if not force and not is_stale():
        return LIB_PATH
    with _build_lock():
        if not force and not is_stale():  # another process built it while this one waited
            return LIB_PATH
        return _build_locked(force, verbose, extra_flags)


def _build_locked(force: bool, verbose: bool, extra_flags: list[str] | None) -> str:
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libgnk.so (set NVCC or add it to PATH)")
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = NVCC_FLAGS + (extra_flags or [])
    hdr_mtime = max(
        os.path.getmtime(os.path.join(d, f))
        for d in (CSRC, INCLUDE)
        for f in os.listdir(d)
        if f.endswith((".cuh", ".h"))
    )

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_mtime):
            return obj
        cmd = [nvcc, *flags, "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr.strip():
            print(r.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources()))) as pool:
        objs = list(pool.map(compile_one, sources()))
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)  # a process that already mapped the old file keeps it
    with open(STAMP_PATH + ".tmp", "w") as fh:
        fh.write(source_digest())
    os.replace(STAMP_PATH + ".tmp", STAMP_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
