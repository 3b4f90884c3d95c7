"""The allocation-free attention entry point (hb200_ccgqa_forward_static) against the regular one.

Some callers cannot ask the driver for device memory at the moment they need attention to run - a serving process
whose HBM already belongs to another allocator's pool, a host runtime that forbids cudaMalloc on its worker threads,
a loop that cannot pay for cudaMalloc's device synchronisation.  They cannot build the workspace hb200_ccgqa_forward
wants, so the library keeps an 8 MiB scratch array of its own for them.  This test drives that entry point through the C ABI, twice in a row
(the array keeps the first call's contents, the second call must not be disturbed by them), and requires the output
to be bit-identical to the workspace-based entry point: both run the same four kernels on the same inputs.

This file sorts last on purpose: a run that stops at the first failure has by then run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _module(dim, H, KV, S):
    from hydra_b200.attention import build_hybrid_attention_module
    torch.manual_seed(11)
    m = build_hybrid_attention_module("ccgqa", dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S, compression_factor=4,
                                      attention_kwargs={})
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                torch.nn.init.xavier_uniform_(p)
    return m.cuda()


def _run_static(L, pm, x, B, S, check_device_free=False):
    y = torch.full_like(x, float("nan"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    st = L.lib().hb200_ccgqa_forward_static(C.byref(pm.struct), 0, x.data_ptr(), y.data_ptr(), B, S,
                                           pm.err_flag.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert torch.cuda.memory_allocated() == before, "the call must not allocate through torch either"
    L.check(st, "ccgqa_forward_static")
    torch.cuda.synchronize()
    if check_device_free:
        # what the driver itself reports as free: neither cudaMalloc nor a lazily loaded module may have taken any
        # (the first call on a device is the set-up call and is allowed to; this is asked of the calls after it)
        assert torch.cuda.mem_get_info()[0] == free_before, "a call after the set-up call took device memory"
    return y


@pytest.mark.parametrize("dim,H,KV,B,S", [(1024, 8, 2, 2, 2048), (512, 8, 2, 3, 100)])
def test_static_scratch_entry_point_matches_workspace_entry_point(dim, H, KV, B, S):
    from hydra_b200 import _lib as L
    m = _module(dim, H, KV, S)
    g = torch.Generator(device="cuda").manual_seed(5)
    x1 = torch.randn(B, S, dim, generator=g, device="cuda").to(torch.bfloat16)
    x2 = torch.randn(B, S, dim, generator=g, device="cuda").to(torch.bfloat16)
    ref1, ref2 = m(x1).clone(), m(x2).clone()          # hb200_ccgqa_forward with a torch-allocated workspace
    pm = m._packed
    y1 = _run_static(L, pm, x1, B, S)                  # first call on this device also resolves the array address
    y2 = _run_static(L, pm, x2, B, S, check_device_free=True)   # second call: the array still holds the first call's data
    pm.check_device_errors()
    assert torch.isfinite(y1.float()).all() and torch.isfinite(y2.float()).all()
    assert torch.equal(y1, ref1), "first call differs from the workspace-based entry point"
    assert torch.equal(y2, ref2), "second call differs from the workspace-based entry point"
    assert not torch.equal(y1, y2)


def test_static_scratch_entry_point_rejects_oversized_requests():
    from hydra_b200 import _lib as L
    m = _module(1024, 8, 2, 4096)
    x = torch.zeros(4, 4096, 1024, dtype=torch.bfloat16, device="cuda")
    m(x[:1, :64])                                      # builds the packed weights
    pm = m._packed
    cap = L.lib().hb200_ccgqa_forward_static_max_bytes()
    assert cap == 8 << 20
    y = torch.zeros_like(x)
    st = L.lib().hb200_ccgqa_forward_static(C.byref(pm.struct), 0, x.data_ptr(), y.data_ptr(), 4, 4096,
                                           pm.err_flag.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == -3                                    # HB200_ERR_WORKSPACE, nothing launched
    msg = L.lib().hb200_last_error().decode()
    assert "scratch" in msg and "hb200_ccgqa_forward" in msg
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0
    # exactly at the limit (4096 tokens at dim 1024, 8q/2kv) is accepted
    st = L.lib().hb200_ccgqa_forward_static(C.byref(pm.struct), 0, x.data_ptr(), y.data_ptr(), 1, 4096,
                                           pm.err_flag.data_ptr(), torch.cuda.current_stream().cuda_stream)
    L.check(st, "ccgqa_forward_static at the limit")
    torch.cuda.synchronize()
    pm.check_device_errors()
