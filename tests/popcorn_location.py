"""Where the tests find the real popcorn package.

Lookup order: a popcorn already importable in this interpreter, then the unmodified install under
`baseline/_ref/` that `python -m oracle.install_reference` makes (ignored by git, carried to a GPU machine
with the rest of the working tree).  Tests that need popcorn skip with the reason below when neither exists.
"""

from __future__ import annotations

import importlib.util
import sys
import warnings
from pathlib import Path

INSTALL = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
MISSING = "popcorn is neither importable nor installed under baseline/_ref (python -m oracle.install_reference)"


def available() -> bool:
    return importlib.util.find_spec("popcorn") is not None or (INSTALL / "popcorn" / "__init__.py").is_file()


def import_popcorn(cache_dir, monkeypatch=None):
    """Import popcorn with its per-user report cache pointed at `cache_dir`; returns the module.

    popcorn reads POPCORN_CACHE_DIR when a store is first used, so the variable is set before the import."""
    import os

    if monkeypatch is not None:
        monkeypatch.setenv("POPCORN_CACHE_DIR", str(cache_dir))
    else:
        os.environ["POPCORN_CACHE_DIR"] = str(cache_dir)
    if importlib.util.find_spec("popcorn") is None:
        if monkeypatch is not None:
            monkeypatch.syspath_prepend(str(INSTALL))
        else:
            sys.path.insert(0, str(INSTALL))
    warnings.filterwarnings("ignore")
    import popcorn
    import popcorn.kernels  # noqa: F401  (fills popcorn.KERNELS)

    return popcorn
