"""hydra_b200 - B200 (sm_100a) implementation of HYDRA's inference forward hot path.

Public surface (mirrors the reference's names for this path):

* ``hydra_b200.kernels``   - ``fused_rope``, ``fused_qk_norm``, ``fused_swiglu``, ``fused_rms_norm`` and the
  kernel-status helpers (reference: ``hydra.kernels``)
* ``hydra_b200.attention`` - ``build_hybrid_attention_module``, registry helpers, ``CCGQAAttention``
  (reference: ``hydra.attention``)
* ``hydra_b200.model``     - ``HydraB200Model`` (whole-model eval forward from a reference ``state_dict``,
  generation by re-forward or with a latent-space KV cache - greedy or sampled -, evaluation loss),
  ``HydraB200BaseModel`` (the routing-free baseline), ``load_checkpoint``, and the reference's factories
  (``create_hydra_model``, ``create_base_model``) with seeded random weights
* ``hydra_b200.routing``   - ``mod_select``, ``mor_depths``: the routers' eval-mode index arithmetic
* ``hydra_b200.sampling``  - ``sample_rows`` (temperature / top-k / top-p), ``cross_entropy_rows``
* ``hydra_b200.parallel``  - sequence sharding across one-process-per-GPU replicas
* ``hydra_b200.install``   - ``install()`` rebinds the reference's module-level names to this package

All compute runs in the CUDA extension ``libhydra_b200.so`` (C ABI in ``include/hydra_b200.h``); there is no
CPU or PyTorch fallback.
"""
__version__ = "0.1.0"

__all__ = ["kernels", "attention", "model", "routing", "sampling", "parallel", "install", "__version__"]
