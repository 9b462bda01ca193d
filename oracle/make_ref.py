"""Install the reference implementation into ``oracle/_ref/`` (git-ignored) so that benchmarks can time the
reference's OWN code for the rollout-decode path next to this library, on whatever machine the tree is carried to.

    REFERENCE_ROOT=/path/to/ultraviolet python oracle/make_ref.py

TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing under ``ultraviolet_b200/`` imports ``oracle/`` or ``oracle/_ref``.

The reference is a pure-Python package (``ultraviolet``: model.py, kernels/*), so "installing" it is
``pip install --no-deps --no-index --target oracle/_ref`` of a scratch copy of the checkout (setuptools writes
build files next to the sources, and the checkout may be read-only).  ``scripts/rl_stream.py`` (StreamGen) is not
part of the package; it is placed beside it as a plain module.  No reference file enters the repository history.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_ROOT = os.path.join(os.sep, "root", "reference")


def reference_root() -> str | None:
    root = os.environ.get("REFERENCE_ROOT") or DEFAULT_ROOT
    return root if os.path.isfile(os.path.join(root, "ultraviolet", "model.py")) else None


def make(force: bool = False) -> str | None:
    """Returns the install directory, or None when no reference checkout is reachable (then a previously made
    ``_ref`` is left as it is)."""
    marker = os.path.join(DEST, "ultraviolet", "model.py")
    root = reference_root()
    if root is None:
        return DEST if os.path.isfile(marker) else None
    if os.path.isfile(marker) and not force:
        return DEST
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(root, src, ignore=shutil.ignore_patterns(".git", "__pycache__", "workbench", "docs", "tests"))
        if os.path.isdir(DEST):
            shutil.rmtree(DEST)
        r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                            "--quiet", "--target", DEST, src], capture_output=True, text=True)
        if r.returncode != 0 or not os.path.isfile(marker):
            # no usable pip / setuptools here: the package is pure Python, so its directory is the install
            os.makedirs(DEST, exist_ok=True)
            shutil.copytree(os.path.join(src, "ultraviolet"), os.path.join(DEST, "ultraviolet"), dirs_exist_ok=True)
        for extra in ("rl_stream.py", "rl_sampler.py"):
            p = os.path.join(src, "scripts", extra)
            if os.path.isfile(p):
                shutil.copy(p, os.path.join(DEST, extra))
    return DEST


if __name__ == "__main__":
    out = make(force="--force" in sys.argv)
    print(out or "no reference checkout found (set REFERENCE_ROOT); nothing installed")
