"""Build recipe for the reference's own CPU drivers (TEST INFRASTRUCTURE, not product).

Compiles the reference's three CPU extension sources *where they lie* in a
read-only checkout of masonfaldet/gm-attention
(``src/gm_attention/nn/fused/{attention,factored,pairs}_cpu.cpp``) with a plain
``g++`` command line into ``oracle/_ref/``.  No reference source is copied; the
reference's own JIT build system (``torch.utils.cpp_extension.load``) is not
run.  The resulting pybind modules expose exactly the reference's extension
functions (``attention_cpu.cpp:256-261``, ``factored_cpu.cpp:223-234``,
``pairs_cpu.cpp:140-148``) and are used

* by ``tests/`` as the checker the CUDA kernels are compared against, and
* by ``bench.py`` as the timed CPU baseline (``cpu_baseline.kind == "reference"``).

Nothing in the shipped package imports this directory.

Usage::

    python oracle/build_ref.py [--reference /path/to/gm-attention] [--force]
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

#: module name -> source file under src/gm_attention/nn/fused/
MODULES = {
    "gm_fused_attention_cpu": "attention_cpu.cpp",
    "gm_factored_cpu": "factored_cpu.cpp",
    "gm_fused_pairs_cpu": "pairs_cpu.cpp",
}


def default_reference() -> Path:
    """``$GM_REFERENCE_ROOT``, else a checkout named ``reference`` next to this repository."""
    return Path(os.environ.get("GM_REFERENCE_ROOT", str(HERE.parent.parent / "reference")))


def compile_one(name: str, source: Path, force: bool) -> Path:
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    target = OUT / f"{name}.so"
    if target.exists() and not force and target.stat().st_mtime >= source.stat().st_mtime:
        return target
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-fopenmp", f"-DTORCH_EXTENSION_NAME={name}",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    for inc in include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-isystem", sysconfig.get_paths()["include"], str(source), "-o", str(target)]
    for lib in library_paths():
        cmd += [f"-L{lib}", f"-Wl,-rpath,{lib}"]
    cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    subprocess.run(cmd, check=True)
    return target


def build(reference: Path | None = None, force: bool = False, modules: tuple[str, ...] | None = None) -> dict[str, Path]:
    """Compile the requested reference CPU drivers; returns name -> .so path.
    Modules whose ``.so`` already exists are kept when the reference checkout
    is absent (the prebuilt files travel with the repository snapshot)."""
    reference = reference or default_reference()
    fused = reference / "src" / "gm_attention" / "nn" / "fused"
    OUT.mkdir(parents=True, exist_ok=True)
    names = modules or tuple(MODULES)
    built: dict[str, Path] = {}
    todo = []
    for name in names:
        source = fused / MODULES[name]
        if source.exists():
            todo.append((name, source))
        elif (OUT / f"{name}.so").exists():
            built[name] = OUT / f"{name}.so"
    with ThreadPoolExecutor(max_workers=3) as pool:
        for (name, _), path in zip(todo, pool.map(lambda item: compile_one(item[0], item[1], force), todo)):
            built[name] = path
    return built


def load(name: str):
    """Import a built reference module from ``oracle/_ref`` (raises if absent)."""
    import importlib.util

    import torch  # noqa: F401  (the module links against libtorch)

    path = OUT / f"{name}.so"
    if not path.exists():
        raise FileNotFoundError(f"{path} is not built; run python oracle/build_ref.py where the reference checkout is mounted")
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[name] = module
    return module


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, default=None)
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    for name, path in build(args.reference, args.force).items():
        print(name, "->", path)
