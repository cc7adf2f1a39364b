"""Builds the sm_100a kernel library in-tree with nvcc (no JIT cache, no torch headers).

``python -m ksa_b200.csrc.build`` compiles every ``.cu`` next to this file for
``compute_100a/sm_100a`` and links ``ksa_b200/_lib/libksa_b200.so``.  Objects are
rebuilt only when a source or header is newer.  The library exposes plain C
entry points; ``ksa_b200.ops._lib`` binds them with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OBJ_DIR = PKG / "_build"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libksa_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _flags() -> list:
    """Release flags, plus the device-side bounds checks when ``KSA_DEBUG=1`` is set."""
    return NVCC_FLAGS + (["-DKSA_DEBUG_CHECKS"] if os.environ.get("KSA_DEBUG") == "1" else [])


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if not force and obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *_flags(), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    # objects built with other flags (release vs debug checks) are stale whatever their time stamps say
    stamp = OBJ_DIR / "flags.txt"
    flags_text = " ".join(_flags())
    if not stamp.exists() or stamp.read_text() != flags_text:
        force = True
    stamp.write_text(flags_text)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
