"""Install the UNMODIFIED popcorn package next to this repository, for the checks that run through it.

    python -m oracle.install_reference [--force] [--incumbents] [SOURCE_TREE]

SOURCE_TREE defaults to $POPCORN_SOURCE_TREE, then to a checkout named `reference` beside this repository.

Test infrastructure, like everything under oracle/: the product (popcorn_b200/) never imports the result.
The package is installed with pip into `baseline/_ref/` (ignored by git, so popcorn's sources never enter
this repository's history) from a scratch copy of the source tree, because popcorn's setup.py writes into
its own tree.  `POPCORN_SKIP_REPORTS=1` is popcorn's documented switch (setup.py:13-24 of its tree) for
installing without its benchmark database, which it would otherwise download.  Dependencies are not
resolved (`--no-deps`): popcorn pins torch / triton versions newer than most machines have, and nothing on
the paths used here (the registry, the dispatcher, the comparison harness, the references of the ops, the
first-party SwiGLU CUDA source and Triton rotary / MoMoE kernels) depends on those pins.

`prebuild_incumbents()` additionally compiles popcorn's first-party SwiGLU CUDA source the way popcorn itself does
(torch.utils.cpp_extension.load through popcorn/impls/_cuda.py:17-23, `-O3`, no architecture flags of its own; the
architecture list is the environment's TORCH_CUDA_ARCH_LIST when it is set, as the benchmark run will see it too, else what torch detects on a B200: compute capability 10.0 plus its PTX) into `baseline/_ext/`, so that a
benchmark run on a GPU machine does not spend a minute in nvcc.  ninja keys a build on the absolute paths of source and
output, so both trees are reached through `stable_locations()`: two symlinks under the system temp directory whose
names are the same on every machine.

Users of the installed copy: tests/popcorn_location.py (dispatch, grading and index-pin tests),
`bench.py --impl reference` and the incumbent timings of `bench.py`.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent
TARGET = REPO / "baseline" / "_ref"
EXTENSIONS = REPO / "baseline" / "_ext"


def default_source() -> Path | None:
    """$POPCORN_SOURCE_TREE, else a checkout named `reference` in this repository's parent directory."""
    for candidate in (os.environ.get("POPCORN_SOURCE_TREE"), REPO.parent / "reference"):
        if candidate and (Path(candidate) / "src" / "popcorn").is_dir():
            return Path(candidate)
    return None


def installed() -> bool:
    return (TARGET / "popcorn" / "__init__.py").is_file()


def install(source_tree: str | os.PathLike[str], force: bool = False) -> Path:
    """pip-install the package found at `source_tree` (a checkout with pyproject.toml) into baseline/_ref."""
    source = Path(source_tree)
    if not (source / "pyproject.toml").is_file() or not (source / "src" / "popcorn").is_dir():
        raise FileNotFoundError(f"{source} is not a popcorn checkout (pyproject.toml and src/popcorn expected)")
    if installed() and not force:
        return TARGET
    if TARGET.exists():
        shutil.rmtree(TARGET)
    TARGET.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="popcorn_src_") as scratch:
        copy = Path(scratch) / "popcorn"
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "site", "images", "node_modules"))
        command = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
                   "--target", str(TARGET), str(copy)]
        if Path("/opt/wheelhouse").is_dir():
            command[6:6] = ["--find-links", "/opt/wheelhouse"]
        done = subprocess.run(command, env={**os.environ, "POPCORN_SKIP_REPORTS": "1"}, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"pip could not install popcorn from {source}:\n{done.stdout}\n{done.stderr}")
    if not installed():
        raise RuntimeError(f"pip reported success but {TARGET / 'popcorn'} is missing")
    return TARGET


def stable_locations() -> tuple[Path, Path]:
    """(package directory, torch extension directory) as symlinks <tmp>/popcorn_b200_reference/{ref,ext} onto
    baseline/_ref and baseline/_ext; (re)made on every call, so they always point into this working tree."""
    root = Path(tempfile.gettempdir()) / "popcorn_b200_reference"
    root.mkdir(exist_ok=True)
    EXTENSIONS.mkdir(parents=True, exist_ok=True)
    links = []
    for name, target in (("ref", TARGET), ("ext", EXTENSIONS)):
        link = root / name
        if link.is_symlink() and Path(os.readlink(link)) != target:
            link.unlink()
        if not link.is_symlink():
            try:
                link.symlink_to(target, target_is_directory=True)
            except FileExistsError:  # another rank of the same job was first
                pass
        links.append(link)
    # ninja rebuilds an output whose input looks newer than the build it logged, and a working tree copied to another
    # machine gets fresh modification times: give the one source of the prebuilt extension an old one
    source = TARGET / "popcorn" / "impls" / "swiglu.cu"
    if source.is_file() and (EXTENSIONS / "popcorn_swiglu" / "popcorn_swiglu.so").is_file():
        try:
            os.utime(source, (1_000_000_000, 1_000_000_000))
        except OSError:
            pass
    return links[0], links[1]


def prebuild_incumbents(force: bool = False) -> Path:
    """Build popcorn's swiglu.cu extension into baseline/_ext through popcorn's own loader, in a child process."""
    built = EXTENSIONS / "popcorn_swiglu" / "popcorn_swiglu.so"
    if built.is_file() and not force:
        return built
    package, extensions = stable_locations()
    lock = EXTENSIONS / "popcorn_swiglu" / "lock"
    if lock.is_file():  # left by an interrupted build: torch's loader would wait for it for ever
        lock.unlink()
    env = {**os.environ, "TORCH_EXTENSIONS_DIR": str(extensions), "TORCH_CUDA_ARCH_LIST": os.environ.get("TORCH_CUDA_ARCH_LIST") or "10.0+PTX", "PYTHONPATH": str(package),
           "POPCORN_CACHE_DIR": tempfile.mkdtemp(prefix="popcorn-cache-")}
    done = subprocess.run([sys.executable, "-W", "ignore", "-c", "from popcorn.impls import _cuda; print(_cuda.load('swiglu').__file__)"],
                          env=env, capture_output=True, text=True, timeout=1200)
    if done.returncode != 0 or not built.is_file():
        raise RuntimeError(f"could not build popcorn's swiglu extension:\n{done.stdout}\n{done.stderr}")
    return built


def main() -> None:
    paths = [argument for argument in sys.argv[1:] if not argument.startswith("--")]
    source = paths[0] if paths else default_source()
    if not source:
        raise SystemExit("usage: python -m oracle.install_reference [--force] SOURCE_TREE   (or set POPCORN_SOURCE_TREE)")
    print(install(source, force="--force" in sys.argv))
    if "--incumbents" in sys.argv:
        print(prebuild_incumbents(force="--force" in sys.argv))


if __name__ == "__main__":
    main()
