"""Build liblf_sm100.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: ``python -m loopfuse_b200.build [--force] [--verbose] [--debug-bounds]``. The build needs
only nvcc; it cross-compiles on hosts without a GPU. The library is written next to this file so
that it travels with the source tree. ``--debug-bounds`` builds the same sources with
``-DLF_DEBUG_BOUNDS`` into ``liblf_sm100_dbg.so`` (index range checks that report through the
status word; loaded instead of the normal library when ``LF_DEBUG_BOUNDS=1`` is set).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "liblf_sm100.so"
STAMP_PATH = PKG_DIR / "csrc" / ".build_stamp"
DBG_LIB_PATH = PKG_DIR / "liblf_sm100_dbg.so"
DBG_STAMP_PATH = PKG_DIR / "csrc" / ".build_stamp_dbg"

PUBLIC_HEADER = PKG_DIR.parent / "include" / "lf_sm100.h"


def _sources() -> list[Path]:
    """Every translation unit under csrc/."""
    return sorted(CSRC.glob("*.cu"))


def fingerprint_files() -> list[Path]:
    """Everything the library is built from: all .cu / .cuh / .h files under csrc/ and the
    public header. A change to any of them forces a rebuild."""
    files = set(CSRC.glob("*.cu")) | set(CSRC.glob("*.cuh")) | set(CSRC.glob("*.h"))
    return sorted(files) + [PUBLIC_HEADER]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: cannot build liblf_sm100.so")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in fingerprint_files():
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_native(force: bool = False, verbose: bool = False,
                 debug_bounds: bool = False) -> Path:
    """Compile every .cu under csrc/ into liblf_sm100.so (or, with ``debug_bounds``, into
    liblf_sm100_dbg.so with -DLF_DEBUG_BOUNDS); skip when sources are unchanged."""
    fp = _fingerprint()
    lib_path, stamp_path = (DBG_LIB_PATH, DBG_STAMP_PATH) if debug_bounds else (LIB_PATH, STAMP_PATH)
    flags = NVCC_FLAGS + (["-DLF_DEBUG_BOUNDS"] if debug_bounds else [])
    suffix = ".dbg.o" if debug_bounds else ".o"
    if not force and lib_path.exists() and stamp_path.exists() and stamp_path.read_text() == fp:
        return lib_path
    nvcc = _nvcc()
    objs = []
    log = []
    procs = []
    for path in _sources():
        src = path.name
        obj = path.with_suffix(suffix)
        cmd = [nvcc, *flags, "-c", str(path), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                 stderr=subprocess.STDOUT, text=True)))
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        log.append(f"== {src}\n{out}")
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        objs.append(str(obj))
    cmd = [nvcc, "-shared", "-o", str(lib_path), *objs, "-lcudart"]
    out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if out.returncode != 0:
        raise RuntimeError(f"link failed:\n{out.stdout}")
    (CSRC / ("build_dbg.log" if debug_bounds else "build.log")).write_text("\n".join(log))
    stamp_path.write_text(fp)
    if verbose:
        print("\n".join(log))
    return lib_path


if __name__ == "__main__":
    path = build_native(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                        debug_bounds="--debug-bounds" in sys.argv)
    print(path)
