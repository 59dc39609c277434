"""Installs the UNMODIFIED reference package into ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [path of the reference checkout]

The reference (JonasGeiping/linear_cross_entropy_loss) is a pure-Python package: ``linear_cross_entropy``
holds Triton kernels that are compiled on the GPU at the first call. "Building" it therefore means a
``pip install --target`` from the checkout, offline and without its dependencies (torch and triton are
already in the image). pip needs to write build files next to the sources and the checkout is read-only, so
the install runs from a temporary copy that is deleted afterwards; nothing of the reference enters this
repository's history (``oracle/_ref/`` is git-ignored).

What uses the result: ``tests/test_gpu_vs_triton.py`` (live parity of the CUDA path against the reference's
Triton path on the same inputs) and the ``triton_reference`` timing leg of ``bench.py``. Nothing in the shipped
package imports it. When the folder is absent those legs report that the reference is unavailable.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
# where the reference checkout is looked for: LCE_REFERENCE_CHECKOUT, else a folder "reference" beside this repository
DEFAULT_CHECKOUT = Path(os.environ.get("LCE_REFERENCE_CHECKOUT", HERE.parent.parent / "reference"))


def installed() -> bool:
    return (TARGET / "linear_cross_entropy" / "ops.py").exists()


def install(checkout: Path = DEFAULT_CHECKOUT, force: bool = False) -> bool:
    """True when ``oracle/_ref`` holds the reference afterwards; False when there is no checkout to install from."""
    checkout = Path(checkout)
    if installed() and not force:
        return True
    if not (checkout / "pyproject.toml").exists():
        return False
    with tempfile.TemporaryDirectory(prefix="lce_ref_src_") as tmp:
        src = Path(tmp) / "src"
        shutil.copytree(checkout, src, ignore=shutil.ignore_patterns(".git", "*.png", "*.csv", "variants"))
        if TARGET.exists():
            shutil.rmtree(TARGET)
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(TARGET), str(src)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("pip install of the reference failed:\n" + proc.stdout + proc.stderr)
    return installed()


if __name__ == "__main__":
    ok = install(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT, force=True)
    print(f"reference {'installed into ' + str(TARGET) if ok else 'checkout not found: nothing installed'}")
