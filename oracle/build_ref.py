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


def reference_model(*, vocab_size: int, dim: int, n_mor_blocks: int, recursions_per_block: int, n_heads: int,
                    n_kv_heads: int, max_seq_len: int, mod_capacity: float, compression_factor: int = 4, seed: int = 0,
                    **extra):
    """The reference's HydraModel, seeded, in eval mode with MoD hard routing switched on (its warm-up passed), the
    way the reference's own inference benchmarks build it.  Needs add_ref_to_path() first."""
    import torch
    from hydra.model.framework.model import HydraModel
    torch.manual_seed(seed)
    m = HydraModel(vocab_size=vocab_size, dim=dim, n_mor_blocks=n_mor_blocks, recursions_per_block=recursions_per_block,
                   n_heads=n_heads, n_kv_heads=n_kv_heads, compression_factor=compression_factor,
                   max_seq_len=max_seq_len, mod_capacity=mod_capacity, **extra)
    m.eval()
    m.set_global_step(10 ** 6)
    return m


def reference_forward(model, ids):
    """model(ids) under no_grad.  On a CUDA device the reference routes RoPE / SwiGLU / RMSNorm through its Triton
    kernels; if those cannot be compiled on the box, they are switched off with the reference's own switch
    (hydra.kernels.set_use_triton_kernels) and the call is repeated on its PyTorch path."""
    import torch
    with torch.no_grad():
        try:
            return model(ids)
        except Exception:
            if not ids.is_cuda:
                raise
            from hydra.kernels import fused_ops
            fused_ops.set_use_triton_kernels(False)
            return model(ids)


def reference_kernel_status() -> dict:
    from hydra.kernels import fused_ops
    st = fused_ops.get_kernel_status()
    return {k: st.get(k) for k in ("triton_available", "use_triton_kernels", "fused_rope", "fused_swiglu", "fused_rms_norm")}


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HYDRA_REFERENCE_ROOT", "")
    if not root:
        sys.exit("usage: python oracle/build_ref.py <reference root>")
    print(build_ref(root, force="--force" in sys.argv))
