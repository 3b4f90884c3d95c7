"""Recipe that puts the UNMODIFIED reference package beside the oracle, as `oracle/_ref/` (test infrastructure).

    python oracle/build_ref.py <reference root>        # or HYDRA_REFERENCE_ROOT=<reference root>

The reference is pure Python + PyTorch with a setuptools `setup.py`, so "building" it is an offline
`pip install --no-index --no-deps --target oracle/_ref` of a scratch copy of its tree (setuptools writes an egg-info
directory next to setup.py, and the reference tree itself is read-only).  The result holds the reference's `hydra`,
`diagnostics` and `tests` packages exactly as its own installer lays them out.  `oracle/_ref/` is never committed
(it is in .gitignore); it is used only by

  * `bench.py --impl reference`   to time the reference's own `HydraModel.forward` on the host cores,
  * `bench.py`'s `library_baseline` leg   to time the reference's CUDA eager path (cuBLAS / SDPA / cuDNN) beside ours,
  * the `-m gpu` tests that build the reference `HydraModel`, apply `hydra_b200.install.install()` and compare.

Nothing under `hydra_b200/` imports it.  When `oracle/_ref/` is absent, those users fall back to the CPU restatement
(`oracle/hydra_oracle.py`) or skip, and say so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def ref_available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "hydra", "__init__.py"))


def add_ref_to_path() -> bool:
    """Put `oracle/_ref` at the END of sys.path (it also holds the reference's own `tests` package, which must not
    shadow this repository's); False when it has not been built."""
    if not ref_available():
        return False
    if REF_DIR not in sys.path:
        sys.path.append(REF_DIR)
    return True


def build_ref(reference_root: str, force: bool = False) -> str:
    """pip-install the reference tree at `reference_root` into oracle/_ref (offline, no dependencies resolved)."""
    if ref_available() and not force:
        return REF_DIR
    if not os.path.isfile(os.path.join(reference_root, "setup.py")):
        raise FileNotFoundError(f"{reference_root} does not look like the reference tree (no setup.py)")
    tmp = tempfile.mkdtemp(prefix="hydra_ref_src_")
    try:
        src = os.path.join(tmp, "src")
        shutil.copytree(reference_root, src, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.pt", "checkpoints"))
        if os.path.isdir(REF_DIR):
            shutil.rmtree(REF_DIR)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
               "--target", REF_DIR, src]
        r = subprocess.run(cmd, cwd=tmp, capture_output=True, text=True)
        if r.returncode != 0 or not ref_available():
            raise RuntimeError(f"pip install of the reference failed:\n{r.stdout}\n{r.stderr}")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return REF_DIR


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HYDRA_REFERENCE_ROOT", "")
    if not root:
        sys.exit("usage: python oracle/build_ref.py <reference root>")
    print(build_ref(root, force="--force" in sys.argv))
