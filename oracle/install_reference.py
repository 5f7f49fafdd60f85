"""Installs the reference project's ``memory_transformer`` package, unmodified, under ``baseline/_ref``.

TEST INFRASTRUCTURE ONLY.  The installed copy is the stock comparator of the drop-in test
(``tests/test_gpu_dropin_model.py``) and of ``bench.py --impl reference``; nothing in ``memory_b200``
imports it.  ``baseline/_ref`` is kept out of version control.

    python oracle/install_reference.py /path/to/Memory

The reference's ``pyproject.toml`` declares no packages and its flat layout holds several top-level
folders, so ``pip install`` of the checkout stops at metadata generation ("multiple top-level
packages discovered").  The recipe therefore copies the checkout to a temporary folder (the original
may be read-only), appends a ``[tool.setuptools] packages = ["memory_transformer"]`` table to the
copy's ``pyproject.toml`` -- packaging metadata only, no source file is touched -- and runs the
offline install from there.  ``memory_transformer`` imports ``omegaconf`` for YAML loading only; where
that module is absent, :func:`import_reference` registers an empty stand-in before importing.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = os.path.join(ROOT, "baseline", "_ref")

PACKAGING = """

[build-system]
requires = ["setuptools"]
build-backend = "setuptools.build_meta"

[tool.setuptools]
packages = ["memory_transformer"]
"""


def install(reference: str, wheelhouse: str = "/opt/wheelhouse") -> str:
    tmp = tempfile.mkdtemp(prefix="moc_ref_")
    try:
        src = os.path.join(tmp, "src")
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns("outputs", "kernels", "idea", "docs", ".git"))
        with open(os.path.join(src, "pyproject.toml"), "a") as f:
            f.write(PACKAGING)
        if os.path.isdir(TARGET):
            shutil.rmtree(TARGET)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", wheelhouse, "--target", TARGET, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("pip install of the reference failed:\n" + r.stdout[-2000:] + r.stderr[-2000:])
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return TARGET


def available() -> bool:
    return os.path.isfile(os.path.join(TARGET, "memory_transformer", "model.py"))


def import_reference():
    """Imports the installed ``memory_transformer`` (from ``baseline/_ref``) and returns the package."""
    if not available():
        raise ImportError("the reference is not installed under baseline/_ref (run oracle/install_reference.py)")
    if "omegaconf" not in sys.modules:
        try:
            import omegaconf  # noqa: F401
        except ImportError:
            stub = types.ModuleType("omegaconf")
            stub.OmegaConf = type("OmegaConf", (), {})
            stub.DictConfig = dict
            sys.modules["omegaconf"] = stub
    if TARGET not in sys.path:
        sys.path.insert(0, TARGET)
    import memory_transformer
    import memory_transformer.memory_block  # noqa: F401  (submodules the package loads lazily)
    import memory_transformer.model  # noqa: F401
    return memory_transformer


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python oracle/install_reference.py /path/to/reference/checkout")
    print(install(sys.argv[1]))
