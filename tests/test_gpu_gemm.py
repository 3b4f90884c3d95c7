"""tcgen05 GEMM (product path) against an fp32 matmul of the same bf16 inputs, for every epilogue, ragged
shapes, the device-side row count, and against the independent mma.sync kernel.  Tolerance: 2 bf16 ulps of the
fp32 reference (inputs are identical bf16 values; only accumulation order and the final rounding differ)."""
import ctypes as C

import pytest
import torch

from tests.gpu_util import assert_close_bf16, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from hydra_b200 import _lib
    return _lib


def gemm(L, A, W, *, epi=0, resid=None, alpha=1.0, rows=None, m_dev=None, impl=0, C_out=None, n_out=None):
    M, K = A.shape
    N = W.shape[0]
    n_out = n_out if n_out is not None else (N // 2 if epi == L.EPI_SWIGLU else N)
    ldc = (n_out + 7) // 8 * 8
    if C_out is None:
        C_out = torch.zeros((M, ldc), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    L.check(L.lib().hb200_gemm_bf16(
        A.data_ptr(), W.data_ptr(), C_out.data_ptr(), M, N, K, A.stride(0), W.stride(0), C_out.stride(0), epi,
        resid.data_ptr() if resid is not None else None, alpha, rows.data_ptr() if rows is not None else None,
        m_dev.data_ptr() if m_dev is not None else None, impl, err.data_ptr(), st), "gemm")
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "a bounded wait inside the GEMM ran out"
    return C_out[:, :n_out]


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


SHAPES = [
    (128, 256, 64), (128, 128, 64), (256, 512, 256), (1000, 384, 1024), (4096, 1024, 256), (300, 1000, 192),
    (77, 50257, 256), (2048, 5632, 1024), (1, 256, 64), (129, 136, 72), (513, 1024, 2816),
]


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_store(L, M, N, K, impl):
    A, W = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05)
    ref = A.float() @ W.float().T
    out = gemm(L, A, W, impl=impl)
    assert_close_bf16(out, ref, what=f"store {M}x{N}x{K} impl{impl}")


@pytest.mark.parametrize("impl", [0, 1])
def test_residual_epilogue(L, impl):
    M, N, K = 1500, 1024, 256
    A, W, X = rnd(M, K, seed=3), rnd(N, K, seed=4, scale=0.05), rnd(M, N, seed=5)
    ref = X.float() + 0.5 * (A.float() @ W.float().T)
    out = gemm(L, A, W, epi=L.EPI_RESID, resid=X, alpha=0.5, impl=impl)
    assert_close_bf16(out, ref, what="resid")


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("F", [2816, 1536, 256, 264])
def test_swiglu_epilogue_with_interleaved_weight(L, F, impl):
    M, K = 700, 512
    A = rnd(M, K, seed=6)
    Wgu = rnd(2 * F, K, seed=7, scale=0.05)                   # [gate rows | up rows], as gate_up.weight
    Wil = torch.empty_like(Wgu)
    L.check(L.lib().hb200_interleave_gate_up(Wgu.data_ptr(), Wil.data_ptr(), F, K, torch.cuda.current_stream().cuda_stream))
    gu = A.float() @ Wgu.float().T
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    out = gemm(L, A, Wil, epi=L.EPI_SWIGLU, impl=impl)
    assert out.shape == (M, F)
    assert_close_bf16(out, ref, what=f"swiglu F={F}")


@pytest.mark.parametrize("impl", [0, 1])
def test_scatter_add_with_device_row_count(L, impl):
    T, N, K, live = 2000, 1024, 512, 777
    A, W = rnd(T, K, seed=8), rnd(N, K, seed=9, scale=0.05)
    cur = rnd(T, N, seed=10)
    g = torch.Generator().manual_seed(11)
    rows = torch.randperm(T, generator=g)[:T].to(torch.int32).cuda()          # each target row at most once
    m_dev = torch.tensor([live], dtype=torch.int32, device="cuda")
    ref = cur.float().clone()
    ref[rows[:live].long()] += (A.float() @ W.float().T)[:live]
    out = gemm(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=m_dev, impl=impl, C_out=cur.clone())
    assert_close_bf16(out, ref, what="scatter_add")
    untouched = torch.ones(T, dtype=torch.bool)
    untouched[rows[:live].long().cpu()] = False
    assert torch.equal(out[untouched.cuda()], cur[untouched.cuda()]), "rows beyond the live count must not change"
    # live count zero: nothing is written
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    out0 = gemm(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=z, impl=impl, C_out=cur.clone())
    assert torch.equal(out0, cur)


def test_tcgen05_agrees_with_mma_sync_kernel(L):
    """Two independent implementations of the same contraction: fp32 accumulation order differs, the bf16
    results may differ by one rounding step at most."""
    A, W = rnd(777, 1024, seed=12), rnd(1000, 1024, seed=13, scale=0.05)
    a = gemm(L, A, W, impl=0).float()
    b = gemm(L, A, W, impl=1).float()
    assert rel_l2(a, b) < 2e-3
    assert_close_bf16(a, b, ulps=1.01, what="tcgen05 vs mma.sync")


def test_full_size_linearity_property(L):
    """The 250M prefill's MLP contraction (65536 x 5632 x 1024 is too slow for a CPU oracle): check the
    size-independent property (A1 + A2) W^T == A1 W^T + A2 W^T on rows sampled across all tiles, and that
    duplicated rows give identical outputs wherever they sit in the M dimension."""
    M, N, K = 65536, 5632, 1024
    A = rnd(M, K, seed=14)
    W = rnd(N, K, seed=15, scale=0.03)
    A[40000:40128] = A[:128]                                        # same rows in two different tiles
    out = gemm(L, A, W)
    assert torch.equal(out[40000:40128], out[:128]), "a row's result must not depend on its tile position"
    idx = torch.randint(0, M, (512,), generator=torch.Generator().manual_seed(16)).cuda()
    ref = A[idx].float() @ W.float().T
    assert_close_bf16(out[idx], ref, what="full-size sampled rows")


def test_argument_errors_are_reported_not_faulted(L):
    A, W = rnd(64, 64), rnd(64, 64)
    Cb = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    f = L.lib().hb200_gemm_bf16
    assert f(None, W.data_ptr(), Cb.data_ptr(), 64, 64, 64, 64, 64, 64, 0, None, 1.0, None, None, 0, None, st) == -1
    assert f(A.data_ptr(), W.data_ptr(), Cb.data_ptr(), 64, 64, 60, 64, 64, 64, 0, None, 1.0, None, None, 0, None, st) == -1
    assert f(A.data_ptr() + 2, W.data_ptr(), Cb.data_ptr(), 64, 64, 64, 64, 64, 64, 0, None, 1.0, None, None, 0, None, st) == -1
    assert f(A.data_ptr(), W.data_ptr(), Cb.data_ptr(), 64, 64, 64, 64, 64, 64, 3, None, 1.0, None, None, 0, None, st) == -1
    assert b"rows" in L.lib().hb200_last_error()


# ---- skinny-M split-K kernel (decode) ---------------------------------------------------------------------------
def skinny(L, A, W, *, epi=0, resid=None, alpha=1.0, rows=None, m_dev=None, C_out=None):
    M, K = A.shape
    N = W.shape[0]
    n_out = N // 2 if epi == L.EPI_SWIGLU else N
    ldc = (n_out + 7) // 8 * 8
    if C_out is None:
        C_out = torch.zeros((M, ldc), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(L.lib().hb200_gemm_skinny_bf16(
        A.data_ptr(), W.data_ptr(), C_out.data_ptr(), M, N, K, A.stride(0), W.stride(0), C_out.stride(0), epi,
        resid.data_ptr() if resid is not None else None, alpha, rows.data_ptr() if rows is not None else None,
        m_dev.data_ptr() if m_dev is not None else None, err.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "gemm_skinny")
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "a bounded wait inside the skinny GEMM ran out"
    return C_out[:, :n_out]


SKINNY_SHAPES = [(64, 2048, 5632), (64, 640, 2048), (8, 64, 192), (37, 512, 1536), (128, 2048, 512), (1, 256, 64),
                 (77, 50257, 256), (64, 136, 72), (5, 11264, 2048), (100, 384, 1024),
                 (129, 512, 256), (256, 2048, 5632), (300, 640, 2048), (512, 1000, 192)]      # several 128-row tiles


@pytest.mark.parametrize("M,N,K", SKINNY_SHAPES)
def test_skinny_store(L, M, N, K):
    A, W = rnd(M, K, seed=21), rnd(N, K, seed=22, scale=0.05)
    ref = A.float() @ W.float().T
    out = skinny(L, A, W)
    assert_close_bf16(out, ref, what=f"skinny store {M}x{N}x{K}")
    assert torch.equal(out, skinny(L, A, W))          # fixed summation order: bit-reproducible


def test_skinny_epilogues_and_device_row_count(L):
    M, D, F = 64, 2048, 5632
    # residual
    A, W, X = rnd(M, 512, seed=23), rnd(D, 512, seed=24, scale=0.05), rnd(M, D, seed=25)
    out = skinny(L, A, W, epi=L.EPI_RESID, resid=X, alpha=0.5)
    assert_close_bf16(out, X.float() + 0.5 * (A.float() @ W.float().T), what="skinny resid")
    # SwiGLU with the interleaved weight
    A = rnd(M, D, seed=26)
    Wgu = rnd(2 * F, D, seed=27, scale=0.02)
    Wil = torch.empty_like(Wgu)
    L.check(L.lib().hb200_interleave_gate_up(Wgu.data_ptr(), Wil.data_ptr(), F, D, torch.cuda.current_stream().cuda_stream))
    gu = A.float() @ Wgu.float().T
    out = skinny(L, A, Wil, epi=L.EPI_SWIGLU)
    assert out.shape == (M, F)
    assert_close_bf16(out, torch.nn.functional.silu(gu[:, :F]) * gu[:, F:], what="skinny swiglu")
    # scatter-add of the first `live` compact rows into their target rows
    live = 23
    A, W = rnd(M, F, seed=28), rnd(D, F, seed=29, scale=0.02)
    cur = rnd(M, D, seed=30)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(31)).to(torch.int32).cuda()
    m_dev = torch.tensor([live], dtype=torch.int32, device="cuda")
    ref = cur.float().clone()
    ref[rows[:live].long()] += (A.float() @ W.float().T)[:live]
    out = skinny(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=m_dev, C_out=cur.clone())
    assert_close_bf16(out, ref, what="skinny scatter_add")
    untouched = torch.ones(M, dtype=torch.bool)
    untouched[rows[:live].long().cpu()] = False
    assert torch.equal(out[untouched.cuda()], cur[untouched.cuda()])
    # zero live rows: nothing is written
    m_dev.zero_()
    out = skinny(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=m_dev, C_out=cur.clone())
    assert torch.equal(out, cur)


def test_skinny_row_tiles_with_read_modify_write_epilogues(L):
    """200 rows = two 128-row tiles: residual, and scatter-add with a device-side row count that ends inside the
    second tile, inside the first one (the second tile's CTAs find no live rows), and at zero."""
    M, D, F = 200, 1024, 1408
    A, W, X = rnd(M, 512, seed=41), rnd(D, 512, seed=42, scale=0.05), rnd(M, D, seed=43)
    out = skinny(L, A, W, epi=L.EPI_RESID, resid=X, alpha=0.5)
    assert_close_bf16(out, X.float() + 0.5 * (A.float() @ W.float().T), what="skinny resid, 2 tiles")
    A, W = rnd(M, F, seed=44), rnd(D, F, seed=45, scale=0.02)
    cur = rnd(M, D, seed=46)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(47)).to(torch.int32).cuda()
    for live in (171, 60, 128, 0):
        m_dev = torch.tensor([live], dtype=torch.int32, device="cuda")
        ref = cur.float().clone()
        ref[rows[:live].long()] += (A.float() @ W.float().T)[:live]
        out = skinny(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=m_dev, C_out=cur.clone())
        assert_close_bf16(out, ref, what=f"skinny scatter_add, {live} live rows")
        untouched = torch.ones(M, dtype=torch.bool)
        untouched[rows[:live].long().cpu()] = False
        assert torch.equal(out[untouched.cuda()], cur[untouched.cuda()])


def test_skinny_agrees_with_the_large_kernel(L):
    A, W = rnd(64, 2048, seed=33), rnd(640, 2048, seed=34, scale=0.05)
    assert rel_l2(skinny(L, A, W).float(), gemm(L, A, W).float()) < 2e-3


def test_skinny_argument_errors(L):
    A, W = rnd(513, 64), rnd(128, 64)
    with pytest.raises(L.Hb200Error):
        skinny(L, A, W)                                # more than four 128-row tiles


def _pair_cases(L):
    """Outputs of the shapes that run as CTA pairs (256- and 384-column tiles, >= 256 rows), every epilogue, odd row and
    column counts, a device-side row count: a dict of CPU tensors."""
    out = {}
    for (M, N, K) in [(513, 1024, 2816), (2048, 5632, 1024), (1000, 384, 1024), (300, 1000, 192), (777, 50257, 256)]:
        A, W = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05)
        out[f"store {M}x{N}x{K}"] = gemm(L, A, W).cpu()
    A, W = rnd(1300, 1024, seed=3), rnd(2 * 2816, 1024, seed=4, scale=0.05)
    out["swiglu"] = gemm(L, A, W, epi=L.EPI_SWIGLU).cpu()
    A, W = rnd(900, 2816, seed=5), rnd(1024, 2816, seed=6, scale=0.05)
    cur = rnd(4000, 1024, seed=7)
    rows = torch.randperm(4000, generator=torch.Generator().manual_seed(8))[:900].to(torch.int32).cuda()
    m_dev = torch.tensor([700], dtype=torch.int32, device="cuda")
    out["scatter"] = gemm(L, A, W, epi=L.EPI_SCATTER_ADD, rows=rows, m_dev=m_dev, C_out=cur.clone()).cpu()
    out["resid"] = gemm(L, rnd(640, 256, seed=9), rnd(768, 256, seed=10, scale=0.05), epi=L.EPI_RESID,
                        resid=rnd(640, 768, seed=11), alpha=0.5).cpu()
    return out


def test_cta_pair_form_gives_the_bits_of_the_single_cta_form(L, tmp_path):
    """256- and 384-column tiles run as CTA pairs (tcgen05.mma.cta_group::2) unless HB200_GEMM_PAIR=0.  Both forms add the
    same products in the same order, so their outputs agree bit for bit.  The switch is read once per process, so the
    single-CTA form runs in a child process."""
    import os
    import subprocess
    import sys
    here = _pair_cases(L)
    out = tmp_path / "single_cta.pt"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys, torch\n"
            f"sys.path.insert(0, {root!r})\n"
            "from hydra_b200 import _lib\n"
            "from tests.test_gpu_gemm import _pair_cases\n"
            f"torch.save(_pair_cases(_lib), {str(out)!r})\n")
    env = dict(os.environ, HB200_GEMM_PAIR="0", HB200_NO_REBUILD="1")
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    there = torch.load(out)
    assert set(here) == set(there)
    for k in here:
        assert torch.equal(here[k], there[k]), k
