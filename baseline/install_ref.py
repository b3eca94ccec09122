"""Places the reference's MoBA package where the GPU tests and the benchmark can load it.

    python baseline/install_ref.py [/path/to/reference-checkout]

Copies the five Python files the inference path needs of `backends/_mthreads/ops/moba/` of a
czy1101/BaselineBenchmark checkout, unmodified, into `baseline/_ref/moba/`.  That folder is
ignored by git: the reference's sources never become part of this repository's history; they
only travel with a working copy to the machine that has the GPU.  The reference ships no
build metadata (no setup.py / pyproject.toml), so there is nothing for pip to install; this
copy is the whole installation.

Nothing in the product imports the copy.  `baseline/ref_triton.py` loads it for
  * tests/test_gpu_reference_triton.py (routing and outputs of the CUDA path against the
    reference's own Triton kernels on the same GPU and inputs), and
  * the informational `reference_triton_b200` timings of bench.py.
Both skip when the folder is absent.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

FILES = ("__init__.py", "attention.py", "native_moba.py", "parallel.py", "routing.py")
DEST = Path(__file__).resolve().parent / "_ref" / "moba"


def default_root() -> Path:
    """$MOBA_REFERENCE_ROOT, else a checkout named `reference` next to this repository."""
    env = os.environ.get("MOBA_REFERENCE_ROOT")
    return Path(env) if env else Path(__file__).resolve().parents[2] / "reference"


def install(reference_root: str | Path | None = None) -> Path | None:
    src = Path(reference_root or default_root()) / "backends" / "_mthreads" / "ops" / "moba"
    if not src.is_dir():
        return None
    DEST.mkdir(parents=True, exist_ok=True)
    for name in FILES:
        if (src / name).exists():
            shutil.copyfile(src / name, DEST / name)
    return DEST


if __name__ == "__main__":
    where = install(sys.argv[1] if len(sys.argv) > 1 else None)
    print(where if where else "reference checkout not found: nothing installed")
