"""Build libpopcorn_b200.so in-tree with nvcc, for sm_100a only.

    python -m popcorn_b200.build            # rebuild if any source is newer than the library
    python -m popcorn_b200.build --force -v # rebuild everything and print ptxas resource usage

The reference JIT-compiles its one CUDA source through torch.utils.cpp_extension
with no architecture flags (src/popcorn/impls/_cuda.py:17-23); this library is a
plain C-ABI shared object instead, so it needs no ATen headers and is loaded with
ctypes.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIBRARY = PACKAGE_DIR / "libpopcorn_b200.so"
OBJ_DIR = PACKAGE_DIR / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def find_nvcc() -> str:
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home and (Path(home) / "bin" / "nvcc").exists():
            return str(Path(home) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise RuntimeError("nvcc not found: set CUDA_HOME or put nvcc on PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_input() -> float:
    inputs = [*sources(), *CSRC.glob("*.cuh"), *INCLUDE.glob("*.h"), Path(__file__)]
    return max(path.stat().st_mtime for path in inputs)


def is_stale() -> bool:
    return not LIBRARY.exists() or LIBRARY.stat().st_mtime < _newest_input()


def _compile(nvcc: str, source: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (source.stem + ".o")
    command = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(source), "-o", str(obj)]
    if verbose:
        command[1:1] = ["-Xptxas", "-v"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{done.stdout}\n{done.stderr}")
    return obj, done.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every csrc/*.cu for sm_100a and link them into LIBRARY. Returns its path."""
    if not force and not is_stale():
        return LIBRARY
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda src: _compile(nvcc, src, verbose), sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objects = [str(obj) for obj, _ in results]
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIBRARY), *objects, "-lcudart"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIBRARY


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--force", action="store_true", help="rebuild even if the library is up to date")
    parser.add_argument("-v", "--verbose", action="store_true", help="pass -Xptxas -v and print its output")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
