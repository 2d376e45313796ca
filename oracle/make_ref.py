"""Install the UNMODIFIED reference package into ``oracle/_ref/`` (test infrastructure).

The reference (LarocheC/gru-triton, ``gru_qat`` 0.2.0) is pure Python.  Its wheel would contain
exactly the package directory ``src/gru_qat`` (pyproject.toml: ``packages = ["src/gru_qat"]``), but
the wheel's build backend (hatchling) is not installed where this runs, so this recipe produces
the same install tree directly: ``<reference>/src/gru_qat`` -> ``oracle/_ref/gru_qat``.

``oracle/_ref/`` is git-ignored (no reference source enters the history); it is used only as a
checker and CPU baseline: by ``tests/``, by ``bench.py``'s ``cpu_baseline`` / ``--impl reference``
legs, and by ``tests/golden/make_golden_butterfly_gpu.py``.  Nothing in the product imports it.

    python oracle/make_ref.py [reference checkout]     (default: $GRU_QAT_REFERENCE, else DEFAULT_CHECKOUT below)
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_CHECKOUT = "/root/reference"


def ref_path() -> str:
    """Directory to put on sys.path so that ``import gru_qat`` finds the installed reference."""
    return DEST


def available() -> bool:
    return os.path.isfile(os.path.join(DEST, "gru_qat", "__init__.py"))


def install(checkout: str | None = None, quiet: bool = False) -> bool:
    """Copy the package; returns False (and leaves any earlier install alone) if the checkout is absent."""
    checkout = checkout or os.environ.get("GRU_QAT_REFERENCE", DEFAULT_CHECKOUT)
    src = os.path.join(checkout, "src", "gru_qat")
    if not os.path.isfile(os.path.join(src, "__init__.py")):
        if not quiet:
            print(f"reference package not found at {src}; oracle/_ref left as it is", file=sys.stderr)
        return False
    dst = os.path.join(DEST, "gru_qat")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    if not quiet:
        print(f"installed {src} -> {dst}")
    return True


if __name__ == "__main__":
    sys.exit(0 if install(sys.argv[1] if len(sys.argv) > 1 else None) else 1)
