"""CPU-side checks of the drop-in boundary: the C-ABI library loads and exports every declared symbol, the
registry / factory behave like the reference's (tests/test_attention_{registry,factory}.py semantics), the
product path refuses CPU tensors instead of falling back, and install() rebinds the reference's names."""
import ctypes
import os
import re
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from hydra_b200 import _lib, build
    with open(os.path.join(ROOT, "include", "hydra_b200.h")) as f:
        declared = sorted(set(re.findall(r"\b(hb200_[a-z0-9_]+)\s*\(", f.read())))
    assert len(declared) >= 20
    handle = _lib.lib()
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/hydra_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(declared)
    assert handle.hb200_version() >= 100
    assert os.path.dirname(build.LIB_PATH).endswith("hydra_b200"), "the extension must live in-tree"


def test_struct_layouts_match_header_sizes():
    from hydra_b200 import _lib
    assert ctypes.sizeof(_lib.BlockWeights) == 16 * 8 + 8 + 2 * 8      # 16 pointers, one float (padded), 2 pointers
    assert ctypes.sizeof(_lib.Model) == 12 * 4 + 4 * 4 + 7 * 8 + 16  # trailing int32, float, int32 + padding: two slots
    assert ctypes.sizeof(_lib.Taps) == 6 * 8 + 8
    assert ctypes.sizeof(_lib.LaunchRecord) == 24
    assert ctypes.sizeof(_lib.DecodeState) == 2 * 4 + 8 * 8    # batch, capacity, eight device pointers
    assert [f[0] for f in _lib.DecodeState._fields_] == ["batch", "capacity", "kcache", "vcache", "halo", "vshift",
                                                         "scores", "pos", "tokens", "history"]


def test_host_side_argument_validation_without_a_gpu():
    """Argument checks run before any CUDA call, so they can be exercised on a CPU-only machine."""
    from hydra_b200 import _lib
    L = _lib.lib()
    assert L.hb200_rms_norm(None, None, None, 4, 8, 1e-6, 1, 0, None) == -1
    assert b"null" in L.hb200_last_error()
    assert L.hb200_mod_topk_select(None, 1, 8, 4, None, None, 0, None, None, None) == -1
    assert L.hb200_gemm_bf16(None, None, None, 1, 1, 1, 8, 8, 8, 0, None, 1.0, None, None, 0, None, None) == -1
    assert L.hb200_model_workspace_bytes(None, 1, 1) == 0
    assert L.hb200_profile_reset(None) == -1
    assert L.hb200_sample_rows(None, 1, 8, 8, 0.8, 50, 0.9, None, None, None) == -1
    assert L.hb200_cross_entropy_rows(None, None, 1, 8, 8, -100, None, None) == -1
    assert L.hb200_argmax_rows(None, 1, 8, 8, None, None) == -1
    assert L.hb200_gemm_skinny_bf16(None, None, None, 1, 8, 8, 8, 8, 8, 0, None, 1.0, None, None, None, None) == -1
    assert L.hb200_decode_workspace_bytes(None, 1) == 0


def test_registry_matches_reference_semantics():
    from hydra_b200.attention import (HybridAttentionBackend, available_hybrid_attention_backends,
                                      is_hybrid_attention_backend_available, resolve_hybrid_attention_backend)
    assert available_hybrid_attention_backends() == ("ccqa",)
    for name in ("ccqa", "CCGQA", "  ccgqa ", "CcQa"):
        assert is_hybrid_attention_backend_available(name)
        assert resolve_hybrid_attention_backend(name) == HybridAttentionBackend("ccqa")
    assert resolve_hybrid_attention_backend(None).name == "ccqa"
    assert not is_hybrid_attention_backend_available("lla3")
    for bad in ("lla3", "flash", ""):
        with pytest.raises(ValueError):
            resolve_hybrid_attention_backend(bad)


def test_factory_builds_module_with_reference_parameter_layout(monkeypatch):
    from hydra_b200.attention import CCGQAAttention, build_hybrid_attention_module
    m = build_hybrid_attention_module("ccgqa", dim=1024, n_heads=8, n_kv_heads=2, max_seq_len=128, compression_factor=4,
                                      attention_kwargs={"mod_mlp_capacity": 0.5, "mor_warmup": 10, "use_fused_kernel": True})
    assert isinstance(m, CCGQAAttention)
    assert (m.latent_dim, m.head_dim, m.kv_dim, m.n_groups) == (256, 32, 64, 4)
    shapes = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert shapes == {
        "key_temperature": (1,), "qkv_proj.weight": (384, 1024), "o_proj.weight": (1024, 256),
        "q_conv.conv1.weight": (256, 32, 3), "q_conv.conv2.weight": (256, 256, 3),
        "k_conv.conv1.weight": (64, 32, 3), "k_conv.conv2.weight": (64, 64, 3)}
    assert float(m.key_temperature) == pytest.approx(32 ** 0.5)
    assert m.cos_cached.shape == (1, 1, 128, 16) and m.cos_cached.dtype == torch.float32
    m._init_rope(256)
    assert m.cos_cached.shape[2] == 256
    with pytest.raises(ValueError):
        build_hybrid_attention_module("lla3", dim=1024, n_heads=8, n_kv_heads=2, max_seq_len=128,
                                      compression_factor=4, attention_kwargs={})
    monkeypatch.setenv("HYDRA_CCQA_USE_FUSED_KERNEL", "0")
    m2 = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=64, compression_factor=4,
                                       attention_kwargs={})
    assert m2.use_fused_kernel is False
    # the ablation switches: a module without convolutions has no conv parameters, as in the reference
    m3 = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=64, compression_factor=4,
                                       attention_kwargs={"use_convs": False, "use_rope": False})
    assert not hasattr(m3, "q_conv") and m3.use_convs is False and m3.use_rope is False and m3.use_qk_norm is True
    assert set(m3.state_dict()) == {"qkv_proj.weight", "o_proj.weight", "key_temperature"}
    with pytest.raises(NotImplementedError):
        build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=64, compression_factor=4,
                                      attention_kwargs={"conv_kernel_size": 9})
    m4 = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=64, compression_factor=4,
                                       attention_kwargs={"conv_kernel_size": 5})
    assert tuple(m4.q_conv.conv1.weight.shape) == (128, 16, 5) and tuple(m4.k_conv.conv2.weight.shape) == (32, 32, 5)


def test_legacy_checkpoint_layouts_are_remapped():
    """Older reference checkpoints (hydra/attention/backends/ccgqa/attention.py:333-383): separate down projections and
    flat conv names load into the fused layout; compile / wrapper prefixes are stripped."""
    from hydra_b200.attention import build_hybrid_attention_module
    from hydra_b200.model import normalize_state_dict
    m = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=32, compression_factor=4,
                                      attention_kwargs={})
    g = torch.Generator().manual_seed(0)
    lat, kvd, hd = 128, 32, 16
    legacy = {
        "q_down.weight": torch.randn(lat, 512, generator=g), "k_down.weight": torch.randn(kvd, 512, generator=g),
        "v_down.weight": torch.randn(kvd // 2, 512, generator=g), "v_shift_down.weight": torch.randn(kvd // 2, 512, generator=g),
        "o_proj.weight": torch.randn(512, lat, generator=g), "key_temperature": torch.tensor([3.0]),
        "q_conv1.weight": torch.randn(lat, hd, 3, generator=g), "q_conv2.weight": torch.randn(lat, lat, 3, generator=g),
        "k_conv1.weight": torch.randn(kvd, hd, 3, generator=g), "k_conv2.weight": torch.randn(kvd, kvd, 3, generator=g),
    }
    m.load_state_dict(dict(legacy), strict=True)
    want = torch.cat([legacy["q_down.weight"], legacy["k_down.weight"], legacy["v_down.weight"], legacy["v_shift_down.weight"]])
    assert torch.equal(m.qkv_proj.weight, want)
    assert torch.equal(m.q_conv.conv2.weight, legacy["q_conv2.weight"]) and torch.equal(m.k_conv.conv1.weight, legacy["k_conv1.weight"])
    payload = {"model": {"_orig_mod.layers.0.attention." + k: v for k, v in legacy.items()}, "step": 7}
    emb = torch.randn(6, 4, generator=g)
    payload["model"]["_orig_mod.tok_emb.weight"] = emb
    payload["model"]["_orig_mod.output.weight"] = emb.clone()            # a tied projection saved twice
    payload["model"]["_orig_mod.layers.0.mod_mlp_wrapper.mod_router._aux_loss"] = torch.zeros(())
    sd = normalize_state_dict(payload)
    assert "layers.0.attention.qkv_proj.weight" in sd and torch.equal(sd["layers.0.attention.qkv_proj.weight"], want)
    assert "layers.0.attention.q_conv.conv1.weight" in sd and "output.weight" not in sd
    assert not any("_aux_loss" in k or "q_down" in k or "_orig_mod" in k for k in sd)
    payload["model"]["_orig_mod.output.weight"] = emb + 1.0              # tie_weights=False: kept
    assert torch.equal(normalize_state_dict(payload)["output.weight"], emb + 1.0)


def test_product_path_refuses_cpu_tensors():
    import hydra_b200.kernels as K
    from hydra_b200.attention import build_hybrid_attention_module
    x = torch.randn(2, 8)
    for call in (lambda: K.fused_rms_norm(x, torch.ones(8)), lambda: K.fused_swiglu(x, x),
                 lambda: K.fused_qk_norm(x.view(1, 1, 2, 8), x.view(1, 1, 2, 8), 1.0),
                 lambda: K.fused_rope(x.view(1, 1, 2, 8), torch.ones(2, 4), torch.zeros(2, 4))):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()
    m = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=64, compression_factor=4,
                                      attention_kwargs={})
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.randn(1, 4, 512))
    from hydra_b200.model import HydraB200Model
    with pytest.raises(RuntimeError, match="CUDA"):
        HydraB200Model({}, n_heads=8, n_kv_heads=2, device="cpu")
    from hydra_b200.sampling import cross_entropy_rows, sample_rows
    with pytest.raises(RuntimeError, match="CUDA"):
        sample_rows(torch.zeros(2, 8, dtype=torch.bfloat16), 0.8, 5, 0.9)
    with pytest.raises(RuntimeError, match="CUDA"):
        cross_entropy_rows(torch.zeros(2, 8, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.int64))
    st = K.get_kernel_status()
    for key in ("triton_available", "use_triton_kernels", "fused_rope", "fused_qk_norm", "fused_swiglu",
                "fused_rms_norm", "liger_ce_available", "use_liger_ce"):
        assert key in st


def test_nothing_in_the_package_imports_the_oracle():
    pkg = os.path.join(ROOT, "hydra_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                with open(os.path.join(dirpath, f)) as fh:
                    text = fh.read()
                assert "hydra_oracle" not in text and "import oracle" not in text and "from oracle" not in text, f


class _FakeHydra:
    """A stand-in for the reference package layout, enough for install() to patch."""


def test_install_rebinds_reference_names_and_uninstall_restores(monkeypatch):
    import types
    mods = {}
    def mk(name, **attrs):
        m = types.ModuleType(name)
        for k, v in attrs.items():
            setattr(m, k, v)
        mods[name] = m
        monkeypatch.setitem(sys.modules, name, m)
        return m
    orig = lambda *a, **k: "reference"
    mk("hydra")
    mk("hydra.kernels", fused_rope=orig, fused_qk_norm=orig, fused_swiglu=orig, fused_rms_norm=orig)
    mk("hydra.kernels.fused_ops", fused_rope=orig, fused_qk_norm=orig, fused_swiglu=orig, fused_rms_norm=orig)
    mk("hydra.layers"); mk("hydra.layers.common", fused_swiglu=orig, fused_rms_norm=orig, FUSED_KERNELS_AVAILABLE=False)
    mk("hydra.attention", build_hybrid_attention_module=orig, resolve_hybrid_attention_backend=orig,
       available_hybrid_attention_backends=orig, is_hybrid_attention_backend_available=orig)
    mk("hydra.attention.factory", build_hybrid_attention_module=orig)
    mk("hydra.attention.backends"); mk("hydra.attention.backends.ccgqa", build_ccqa_attention=orig)
    mk("hydra.attention.backends.ccgqa.backend", build_ccqa_attention=orig, CCGQAAttention=orig)
    mk("hydra.attention.backends.ccgqa.attention", fused_rope=orig, FUSED_KERNELS_AVAILABLE=False)
    mk("hydra.model"); mk("hydra.model.framework")
    mk("hydra.model.framework.blocks", build_hybrid_attention_module=orig, CCGQAAttention=orig)
    from hydra_b200 import install as I, kernels as K, attention as A
    done = I.install()
    assert mods["hydra.layers.common"].fused_swiglu is K.fused_swiglu
    assert mods["hydra.layers.common"].FUSED_KERNELS_AVAILABLE is True
    assert mods["hydra.attention.backends.ccgqa.attention"].fused_rope is K.fused_rope
    assert mods["hydra.model.framework.blocks"].build_hybrid_attention_module is A.build_hybrid_attention_module
    assert "hydra.kernels" in done and "hydra.attention.factory" in done
    assert mods["hydra.model.framework.blocks"].CCGQAAttention is A.CCGQAAttention       # HydraBlock builds it by name
    assert mods["hydra.attention.backends.ccgqa"].build_ccqa_attention is A.build_ccqa_attention
    assert mods["hydra.attention.backends.ccgqa.backend"].CCGQAAttention is A.CCGQAAttention
    I.uninstall()
    assert mods["hydra.model.framework.blocks"].CCGQAAttention is orig
    assert mods["hydra.layers.common"].fused_swiglu is orig
    assert mods["hydra.model.framework.blocks"].build_hybrid_attention_module is orig
    assert mods["hydra.layers.common"].FUSED_KERNELS_AVAILABLE is False


def test_end_of_text_padding_of_generated_sequences():
    """generate(eos_token_id=...): the reference's helper stops its sequence at the first end-of-text token
    (eval_checkpoint.py:158-160); in a batch, what follows a row's first one is overwritten with it.  The prompt is
    never touched, even if it holds the token."""
    from hydra_b200.model import _pad_after_eos
    s = torch.tensor([[9, 2, 3, 9, 4, 5], [1, 2, 7, 7, 9, 3], [1, 2, 3, 4, 5, 6]])
    out = _pad_after_eos(s.clone(), 2, 9)
    assert out.tolist() == [[9, 2, 3, 9, 9, 9], [1, 2, 7, 7, 9, 9], [1, 2, 3, 4, 5, 6]]
    assert torch.equal(_pad_after_eos(s.clone(), 2, None), s)
    assert torch.equal(_pad_after_eos(s.clone(), 6, 9), s)


def _tiny_state_dict():
    from oracle import hydra_oracle as O
    cfg = O.HydraConfig(vocab_size=32, dim=64, n_mor_blocks=3, recursions_per_block=2, n_heads=2, n_kv_heads=1,
                        max_seq_len=16, mod_capacity=0.5)
    return O.init_params(cfg, seed=0)


def test_weights_that_no_kernel_reads_are_refused():
    """A reference model built with moe_enabled runs its moe_layers inside the forward (model.py:431-503); this backend has
    no such layers, so a state_dict that carries them - or any other tensor it would drop - is refused, not half-loaded."""
    from hydra_b200.model import check_state_dict_is_consumed, normalize_state_dict
    sd = normalize_state_dict(_tiny_state_dict())
    check_state_dict_is_consumed(sd)                                            # a plain model passes
    ok = dict(sd)
    ok["layers.1.mod_mlp_wrapper.mod_router._aux_loss"] = torch.zeros(())       # bookkeeping buffers are not weights
    ok["loss_baseline._ema"] = torch.zeros(())
    ok["layers.0.attention.cos_cached"] = torch.zeros(1, 1, 16, 16)
    check_state_dict_is_consumed(ok)
    moe = dict(sd)
    moe["moe_layers.0.moe.experts.0.gate_up.weight"] = torch.zeros(8, 64)
    with pytest.raises(NotImplementedError, match="mixture-of-experts"):
        check_state_dict_is_consumed(moe)
    stray = dict(sd)
    stray["layers.0.adapter.weight"] = torch.zeros(4, 4)
    with pytest.raises(KeyError, match="adapter"):
        check_state_dict_is_consumed(stray)


def test_reference_instance_with_moe_layers_is_refused():
    from hydra_b200.model import HydraB200Model

    class FakeRef:
        moe_enabled = True
        moe_layers = [object(), object()]
        layers = []

    with pytest.raises(NotImplementedError, match="moe_enabled"):
        HydraB200Model.reference_kwargs(FakeRef())
    with pytest.raises(NotImplementedError, match="moe_enabled"):
        HydraB200Model.from_reference(FakeRef())


def test_attention_module_refuses_a_training_call():
    """The module's kernels are forward-only; an input that carries a gradient would silently get none back."""
    from hydra_b200.attention import build_hybrid_attention_module
    m = build_hybrid_attention_module("ccqa", dim=512, n_heads=8, n_kv_heads=2, max_seq_len=16, compression_factor=4,
                                      attention_kwargs={})
    x = torch.zeros(1, 4, 512, requires_grad=True)
    with pytest.raises(RuntimeError, match="inference only"):
        m(x)
    with torch.no_grad():                       # under no_grad the refusal that applies is the CPU one
        with pytest.raises(RuntimeError, match="CUDA"):
            m(x)
