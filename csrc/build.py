"""Build the native library ``dart_pytorch_b200/_C/libdptb200.so`` for sm_100a with nvcc.

Every ``csrc/*.cu`` file is compiled to an object in parallel (whole-program device code per file: no device
linking, so the compiler can allocate registers per warp-specialised branch; the device status word is one block per
translation unit, folded on the host) and linked into one shared library.  Objects are rebuilt only when their source
or a header under ``csrc/common`` is newer.

    python csrc/build.py [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ_DIR = ROOT / "build" / "obj"
OUT_DIR = ROOT / "dart_pytorch_b200" / "_C"
LIB = OUT_DIR / "libdptb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    f"-I{CSRC}",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources():
    return sorted(CSRC.glob("*.cu"))


def _newest_header_mtime() -> float:
    hdrs = list((CSRC / "common").glob("*")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile(src: Path, force: bool, verbose: bool, hdr_mtime: float):
    obj = OBJ_DIR / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_mtime):
        return obj, False, ""
    cmd = [nvcc_path(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, True, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose, hdr_mtime), srcs))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if verbose:
        for r in results:
            if r[2]:
                print(r[2])
    stale = (not LIB.exists()) or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs)
    if rebuilt or stale or force:
        cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIB),
               *[str(o) for o in objs], "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    lib = build(args.force, args.verbose)
    print(lib)
    sys.exit(0)
