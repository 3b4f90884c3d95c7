"""GPU parity of the exported fused ops (through torch custom ops -> C ABI -> sm_100a kernels) against the
CPU oracle and the golden fixtures generated from the reference.  fp32 tolerances follow the reference's own
tests (tests/test_optimizations.py:191-231: 1e-5 swiglu, 1e-4 rms_norm / rope); bf16: 2 bf16 ulps."""
import numpy as np
import pytest
import torch

from oracle import hydra_oracle as O
from tests import golden_io as G
from tests.gpu_util import assert_close_bf16, bf16_round, max_abs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    import hydra_b200.kernels as k
    return k


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_library_is_loaded_and_reports_backend(K):
    st = K.get_kernel_status()
    assert "sm_100a" in st["backend"] and st["fused_rope"] and st["fused_swiglu"]


def test_fused_ops_fp32_match_reference_fixtures(K):
    fx = G.load("fused_ops.npz")
    for hd in (16, 32):
        y = K.fused_rope(cu(fx[f"rope{hd}_x"]), cu(fx[f"rope{hd}_cos"]), cu(fx[f"rope{hd}_sin"]))
        assert y.is_contiguous() and max_abs(y, torch.from_numpy(fx[f"rope{hd}_y"])) <= 1e-4
    K.QK_NORM_MODE = "normalize"
    qo, ko = K.fused_qk_norm(cu(fx["qkn_q"]), cu(fx["qkn_k"]), 5.0, 1.7)
    assert max_abs(qo, torch.from_numpy(fx["qkn_qo"])) <= 1e-5 and max_abs(ko, torch.from_numpy(fx["qkn_ko"])) <= 1e-5
    K.QK_NORM_MODE = "rsqrt"
    q2, k2 = K.fused_qk_norm(cu(fx["qkn_q"]), cu(fx["qkn_k"]), 5.0, 1.7)
    r2q, r2k = O.qk_norm_rsqrt(torch.from_numpy(fx["qkn_q"]), torch.from_numpy(fx["qkn_k"]), 5.0, 1.7)
    assert max_abs(q2, r2q) <= 1e-5 and max_abs(k2, r2k) <= 1e-5
    assert max_abs(K.fused_swiglu(cu(fx["swiglu_gate"]), cu(fx["swiglu_up"])), torch.from_numpy(fx["swiglu_y"])) <= 1e-5
    assert max_abs(K.fused_rms_norm(cu(fx["rms_x"]), cu(fx["rms_w"]), 1e-6), torch.from_numpy(fx["rms_y"])) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rms_norm_config3_shape(K, dtype):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(16384, 1024, generator=g).to(dtype)
    w = (1.0 + 0.02 * torch.randn(1024, generator=g))
    ref = O.rms_norm(x.float(), w, 1e-6)
    y = K.fused_rms_norm(x.cuda(), w.cuda(), 1e-6)
    assert y.dtype == dtype and y.shape == x.shape
    if dtype == torch.float32:
        assert max_abs(y, ref) <= 1e-4
    else:
        assert_close_bf16(y, ref, ulps=1.0 if dtype == torch.bfloat16 else 0.25, what="rms_norm")
    # weight in the activation dtype (a module cast with .to(bfloat16)), odd dims (generic kernel), 3-D input
    y2 = K.fused_rms_norm(x[:64].cuda().view(4, 16, 1024), w.to(dtype).cuda(), 1e-6)
    assert y2.shape == (4, 16, 1024)
    x3 = torch.randn(5, 1001, generator=g)
    w3 = torch.randn(1001, generator=g)
    assert max_abs(K.fused_rms_norm(x3.cuda(), w3.cuda(), 1e-5), O.rms_norm(x3, w3, 1e-5)) <= 1e-4
    x4 = torch.randn(3, 4096, generator=g)   # longer than the register-cached variants
    assert max_abs(K.fused_rms_norm(x4.cuda(), torch.ones(4096).cuda(), 1e-6), O.rms_norm(x4, torch.ones(4096))) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_config3_shape_and_strided_view(K, dtype):
    g = torch.Generator().manual_seed(2)
    B, H, S, hd = 8, 8, 2048, 32
    cos, sin = O.rope_tables(S, hd)
    base = torch.randn(B, S, H, hd, generator=g).to(dtype)      # [B,S,H,hd]; the module rotates a transposed view
    xv = base.cuda().transpose(1, 2)
    assert not xv.is_contiguous()
    y = K.fused_rope(xv, cos.cuda()[None, None], sin.cuda()[None, None])
    ref = O.rope(base.float().transpose(1, 2), cos, sin)
    assert y.is_contiguous() and y.dtype == dtype
    if dtype == torch.float32:
        assert max_abs(y, ref) <= 1e-4
    else:
        assert_close_bf16(y, ref, ulps=1.0, what="rope")
    # 2-D tables longer than S, bf16 tables (module cast), odd head_dim multiple (scalar path)
    y2 = K.fused_rope(xv[:, :, :100], cos.cuda().to(torch.bfloat16), sin.cuda().to(torch.bfloat16))
    ref2 = O.rope(base.float().transpose(1, 2)[:, :, :100], cos.to(torch.bfloat16).float(), sin.to(torch.bfloat16).float())
    assert max_abs(y2.float(), ref2) <= (1e-4 if dtype == torch.float32 else 0.05)
    x6 = torch.randn(2, 3, 7, 6, generator=g)
    c6, s6 = O.rope_tables(7, 6)
    assert max_abs(K.fused_rope(x6.cuda(), c6.cuda(), s6.cuda()), O.rope(x6, c6, s6)) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_chunk_views(K, dtype):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(4, 96, 2 * 2816, generator=g) * 2).to(dtype)
    gate, up = gu.cuda().chunk(2, dim=-1)                      # strided views, as SwiGLUMLPFused passes them
    y = K.fused_swiglu(gate, up)
    ref = O.swiglu(gu.float()[..., :2816], gu.float()[..., 2816:])
    assert y.shape == ref.shape and y.is_contiguous()
    if dtype == torch.float32:
        assert max_abs(y, ref) <= 1e-5
    else:
        assert_close_bf16(y, ref, ulps=1.0, what="swiglu")
    a = torch.randn(3, 7, generator=g)
    b = torch.randn(3, 7, generator=g)
    assert max_abs(K.fused_swiglu(a.cuda(), b.cuda()), O.swiglu(a, b)) <= 1e-6


def test_qk_norm_bf16_and_head_dims(K):
    g = torch.Generator().manual_seed(3)
    for hd in (16, 32, 64, 24):
        q = torch.randn(2, 8, 50, hd, generator=g).to(torch.bfloat16)
        k = torch.randn(2, 2, 50, hd, generator=g).to(torch.bfloat16)
        K.QK_NORM_MODE = "normalize"
        qo, ko = K.fused_qk_norm(q.cuda(), k.cuda(), float(hd) ** 0.5, 0.7)
        rq, rk = O.qk_norm(q.float(), k.float(), float(hd) ** 0.5, 0.7)
        assert_close_bf16(qo, rq, ulps=1.0, what=f"q hd{hd}")
        assert_close_bf16(ko, rk, ulps=1.0, what=f"k hd{hd}")
    K.QK_NORM_MODE = "rsqrt"
    z = torch.zeros(1, 1, 4, 16).cuda()
    qo, ko = K.fused_qk_norm(z, z, 4.0, 1.0)
    assert float(qo.abs().max()) == 0.0 and torch.isfinite(ko).all()    # zero vectors stay zero, no NaN


def test_empty_inputs_and_errors(K):
    e = torch.empty(0, 1024, device="cuda", dtype=torch.bfloat16)
    assert K.fused_rms_norm(e, torch.ones(1024, device="cuda"), 1e-6).shape == (0, 1024)
    assert K.fused_swiglu(e, e).shape == (0, 1024)
    c, s = O.rope_tables(4, 16)
    assert K.fused_rope(torch.empty(0, 2, 4, 16, device="cuda"), c.cuda(), s.cuda()).shape == (0, 2, 4, 16)
    with pytest.raises(RuntimeError):
        K.fused_rms_norm(torch.randn(2, 8), torch.ones(8), 1e-6)             # CPU tensor: no fallback
    with pytest.raises((ValueError, RuntimeError)):
        K.fused_rms_norm(torch.randn(2, 8).cuda(), torch.ones(9).cuda(), 1e-6)
    with pytest.raises((TypeError, RuntimeError)):
        K.fused_swiglu(torch.zeros(2, 8, dtype=torch.float64).cuda(), torch.zeros(2, 8, dtype=torch.float64).cuda())
