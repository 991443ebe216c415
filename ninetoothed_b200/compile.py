"""Builds ``libninetoothed_b200.so`` in-tree with nvcc, for sm_100a only.

    python -m ninetoothed_b200.compile [--force] [--verbose]

Each ``csrc/*.cu`` is compiled to an object file (in parallel), then linked with
the static CUDA runtime into ``ninetoothed_b200/lib/libninetoothed_b200.so``.
The library has no link-time dependency on the driver (it looks the one driver
entry point it needs up at run time), so it loads on a GPU-less host.
"""

from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

PACKAGE_DIR = pathlib.Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
INCLUDE_DIR = PACKAGE_DIR.parent / "include"
LIB_DIR = PACKAGE_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIBRARY = LIB_DIR / "libninetoothed_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    f"-I{INCLUDE_DIR}",
]


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and pathlib.Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest_header_mtime() -> float:
    headers = list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h")) + list(INCLUDE_DIR.glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(nvcc: str, source: pathlib.Path, verbose: bool) -> tuple[pathlib.Path, str]:
    obj = OBJ_DIR / (source.stem + ".o")
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr, file=sys.stderr)
    (OBJ_DIR / (source.stem + ".ptxas.txt")).write_text(proc.stderr)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile what is out of date and return the path of the shared library."""
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC_DIR.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC_DIR}")
    header_mtime = _newest_header_mtime()
    stale = []
    for source in sources:
        obj = OBJ_DIR / (source.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(source.stat().st_mtime, header_mtime):
            stale.append(source)
    if stale:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(stale))) as pool:
            list(pool.map(lambda s: _compile(nvcc, s, verbose), stale))
    objects = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if stale or not LIBRARY.exists():
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", str(LIBRARY), *map(str, objects)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
