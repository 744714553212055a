"""Compile the CUDA sources under ``csrc/`` into ``libgmb200.so`` for sm_100a.

One ``nvcc`` command per translation unit (run in parallel), then one link.
The library is built in-tree, next to this file, so that it travels with the
source tree; nothing is cached outside the package.  ``nvcc`` cross-compiles,
so no GPU is needed to build.

    python -m gm_attention_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBRARY = HERE / "libgmb200.so"
OBJECTS = HERE / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(source: Path, force: bool, verbose: bool) -> Path:
    obj = OBJECTS / (source.stem + ".o")
    stamp = max(source.stat().st_mtime, _newest_header())
    if obj.exists() and not force and obj.stat().st_mtime >= stamp:
        return obj
    cmd = [NVCC, *ARCH, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(source), "-o", str(obj)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        print(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJECTS.mkdir(exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objects = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    if LIBRARY.exists() and not force and all(LIBRARY.stat().st_mtime >= o.stat().st_mtime for o in objects):
        return LIBRARY
    # link beside the target and rename: a reader (or a snapshot of the tree) never sees a half-written library
    partial = LIBRARY.with_suffix(".so.partial")
    cmd = [NVCC, *ARCH, "-shared", "-o", str(partial), *map(str, objects), "-lcudart", "-ldl"]
    subprocess.run(cmd, check=True)
    os.replace(partial, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build(args.force, args.verbose))
