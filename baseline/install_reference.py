"""Installs the unmodified reference package (pure Python) under baseline/_ref.

    python baseline/install_reference.py [path to a checkout of the reference]

pip builds a wheel in the source tree, so the checkout (which may be read-only)
is copied to a temporary directory first.  Dependencies are not resolved: torch,
triton, transformers, flash-attn and xxhash come from the environment.  Nothing
of the reference is copied into the tracked tree; baseline/_ref is git-ignored.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
DEFAULT_SOURCE = os.environ.get("NANOVLLM_REFERENCE_SRC", "/root/reference")


def installed() -> bool:
    return os.path.isdir(os.path.join(TARGET, "nanovllm"))


def install(source: str = DEFAULT_SOURCE, force: bool = False) -> bool:
    """Returns True when baseline/_ref holds the package afterwards."""
    if installed() and not force:
        return True
    if not os.path.isdir(os.path.join(source, "nanovllm")):
        return False
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "src")
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "assets"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet", "--upgrade",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, copy]
        subprocess.check_call(cmd)
    return installed()


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    ok = install(paths[0] if paths else DEFAULT_SOURCE, force="--force" in sys.argv)
    print("installed" if ok else "reference source not found")
    sys.exit(0 if ok else 1)
