"""In-tree build of ``libanima_b200.so`` (sm_100a only) with plain ``nvcc``.

``python -m anima_trainer_sm120_b200.build`` compiles every ``csrc/*.cu`` to an
object file (in parallel) and links them into ``libanima_b200.so`` beside this
file. nvcc cross-compiles without a GPU, so this also runs on a CPU-only box.
Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libanima_b200.so"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libanima_b200.so cannot be built")
    return exe


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    hdr_mtime = _newest_header_mtime()

    def compile_one(src: Path) -> tuple[Path, bool]:
        obj = OBJ_DIR / (src.stem + ".o")
        stale = (
            force
            or not obj.exists()
            or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        )
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj, stale

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    objs = [o for o, _ in results]
    if force or not LIB_PATH.exists() or any(s for _, s in results):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-cudart", "static", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libanima_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
