"""Single-kernel microbenchmarks on the shapes of the two microbenchmark configurations (CCGQA block; RMSNorm / RoPE / SwiGLU FFN)
and on the GEMM shapes of the 250M model.  Run through ``python bench.py --micro NAME`` (one JSON line each) - also
the small, self-terminating command lines used for ``ncu`` captures.

Timing: CUDA events on the launching stream around ITERS launches after warm-up.  Bandwidth-bound kernels rotate
through input/output buffer sets whose total size exceeds twice the 126 MB L2, so every launch reads from HBM;
tensor-bound cases state their working set.
"""
from __future__ import annotations

import ctypes as C
import json
import math
import os
from typing import Callable, Dict

import torch

from hydra_b200 import _lib, kernels
from hydra_b200._pack import PackedBlock, PackedModel, interleave_gate_up, repack_conv, rope_tables

L2_BYTES = 126 * 1024 * 1024


def _peaks(root: str) -> tuple[dict, str]:
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def _time(fn: Callable[[int], None], iters: int, warmup: int = 3) -> float:
    """Average milliseconds per call of fn(i)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _sets(bytes_per_set: int) -> int:
    return max(2, int(math.ceil(2.2 * L2_BYTES / max(1, bytes_per_set))))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _rand_bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------------------------
def gemm(args) -> dict:
    M, N, K = args.m, args.n, args.k
    epi = {"store": 0, "resid": 1, "swiglu": 2, "scatter": 3}[args.epilogue]
    n_out = N // 2 if epi == 2 else N
    ldc = (n_out + 7) // 8 * 8
    per_set = M * K * 2 + M * ldc * 2
    ns = min(_sets(per_set), 4)
    A = [_rand_bf16(M, K, seed=i) for i in range(ns)]
    W = _rand_bf16(N, K, scale=0.03, seed=99)
    Cs = [torch.zeros(M, ldc, dtype=torch.bfloat16, device="cuda") for _ in range(ns)]
    X = _rand_bf16(M, ldc, seed=7) if epi == 1 else None
    rows = torch.randperm(M, device="cuda").to(torch.int32) if epi == 3 else None
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = _lib.lib()

    def run(i):
        j = i % ns
        _lib.check(lib.hb200_gemm_bf16(A[j].data_ptr(), W.data_ptr(), Cs[j].data_ptr(), M, N, K, K, K, ldc, epi,
                                       X.data_ptr() if X is not None else None, 0.5,
                                       rows.data_ptr() if rows is not None else None, None, args.impl,
                                       err.data_ptr(), _stream()))

    ms = _time(run, args.iters)
    assert int(err.item()) == 0
    flops = 2.0 * M * N * K
    return {"kernel": f"gemm_{'tcgen05' if args.impl == 0 else 'mma'} {args.epilogue}", "shape": [M, N, K], "ms": ms,
            "bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "algorithmic_flops": flops, "working_set_mb": (per_set * ns + N * K * 2) / 1e6}


def gemm_skinny(args) -> dict:
    """The decode contraction (M <= 128 rows) with weight sets rotated so that every call streams W from HBM:
    achieved = bytes of W (+ A and C) per call / time, against the HBM peak."""
    M, N, K = min(args.m, 128), args.n, args.k
    epi = {"store": 0, "resid": 1, "swiglu": 2, "scatter": 3}[args.epilogue]
    n_out = N // 2 if epi == 2 else N
    ldc = (n_out + 7) // 8 * 8
    ns = _sets(N * K * 2)
    W = [_rand_bf16(N, K, scale=0.03, seed=90 + i) for i in range(ns)]
    A = _rand_bf16(M, K, seed=1)
    Cm = torch.zeros(M, ldc, dtype=torch.bfloat16, device="cuda")
    X = _rand_bf16(M, ldc, seed=7) if epi == 1 else None
    rows = torch.randperm(M, device="cuda").to(torch.int32) if epi == 3 else None
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = _lib.lib()

    def run(i):
        _lib.check(lib.hb200_gemm_skinny_bf16(A.data_ptr(), W[i % ns].data_ptr(), Cm.data_ptr(), M, N, K, K, K, ldc, epi,
                                              X.data_ptr() if X is not None else None, 0.5,
                                              rows.data_ptr() if rows is not None else None, None, err.data_ptr(),
                                              _stream()))

    ms = _time(run, args.iters)
    assert int(err.item()) == 0
    nbytes = 2.0 * (N * K + M * K + M * n_out * (2 if epi in (1, 3) else 1))
    return {"kernel": f"gemm_skinny {args.epilogue}", "shape": [M, N, K], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes,
            "working_set_mb": ns * N * K * 2 / 1e6}


def _attention_module(dim=1024, H=8, KV=2, S=2048, temperature=1.0):
    from hydra_b200.attention import build_hybrid_attention_module
    torch.manual_seed(1)
    m = build_hybrid_attention_module("ccgqa", dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S, compression_factor=4,
                                      attention_kwargs={})
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                torch.nn.init.xavier_uniform_(p)
        if temperature is not None:
            m.key_temperature.fill_(temperature)
    return m.cuda()


def ccgqa_block(args) -> dict:
    """One CCGQA attention block, B=8 x S=2048 x dim 1024, 8q/2kv heads of 32, bf16, causal,
    Xavier-uniform weights (seed 1), key temperature 1.0.  46.51 GFLOP and 68.9 MB of minimum traffic per call."""
    B, S, D = args.batch, 2048, 1024
    m = _attention_module()
    ns = _sets(B * S * D * 2 * 2)
    xs = [_rand_bf16(B, S, D, seed=i) for i in range(ns)]
    m(xs[0])
    pm = m._packed
    prof = _lib.lib().hb200_profile_create(64)
    pm.struct.profile = prof
    ms = _time(lambda i: m(xs[i % ns]), args.iters)
    _lib.lib().hb200_profile_reset(prof)
    m(xs[0])
    torch.cuda.synchronize()
    recs = (_lib.LaunchRecord * 64)()
    t = (C.c_float * 64)()
    n = _lib.lib().hb200_profile_read(prof, recs, t, 64)
    parts = {_lib.KERNEL_KINDS[recs[i].kind]: float(t[i]) for i in range(n)}
    pm.struct.profile = None
    _lib.lib().hb200_profile_destroy(prof)
    pm.check_device_errors()
    T, lat, kvd, hd = B * S, 256, 64, 32
    flops = T * (2 * D * (lat + 2 * kvd) + 6 * (lat * hd + lat * lat + kvd * hd + kvd * kvd) + 4 * lat * (S + 1) / 2 + 2 * lat * D)
    return {"kernel": "ccgqa_block (qkv GEMM + fused pre-attention + attention + o_proj GEMM)", "shape": [B, S, D],
            "ms": ms, "bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "algorithmic_flops": flops, "parts_ms": parts}


def pre_attention(args) -> dict:
    """Fused pre-attention kernel at config-2 shapes: reads qkv once, writes q,k,v once: 1536 B/token + 0.47 MB."""
    B, S, H, KV, hd = args.batch, 2048, 8, 2, 32
    lat, kvd = H * hd, KV * hd
    m = _attention_module()
    sd = m.state_dict()
    dev = torch.device("cuda", torch.cuda.current_device())
    w1 = torch.cat([repack_conv(sd["q_conv.conv1.weight"], dev), repack_conv(sd["k_conv.conv1.weight"], dev)], 0).contiguous()
    w2q, w2k = repack_conv(sd["q_conv.conv2.weight"], dev), repack_conv(sd["k_conv.conv2.weight"], dev)
    cos, sin = rope_tables(S, hd, dev)
    temp = torch.ones(1, device="cuda")
    per_set = B * S * (lat + 2 * kvd) * 2 * 2
    ns = _sets(per_set)
    qkv = [_rand_bf16(B, S, lat + 2 * kvd, seed=i) for i in range(ns)]
    q = [torch.empty(B, H, S, hd, dtype=torch.bfloat16, device="cuda") for _ in range(ns)]
    k = [torch.empty(B, KV, S, hd, dtype=torch.bfloat16, device="cuda") for _ in range(ns)]
    v = [torch.empty(B, KV, S, hd, dtype=torch.bfloat16, device="cuda") for _ in range(ns)]
    lib = _lib.lib()

    def run(i):
        j = i % ns
        _lib.check(lib.hb200_ccgqa_pre_attention(qkv[j].data_ptr(), w1.data_ptr(), w2q.data_ptr(), w2k.data_ptr(),
                                                 cos.data_ptr(), sin.data_ptr(), temp.data_ptr(), q[j].data_ptr(),
                                                 k[j].data_ptr(), v[j].data_ptr(), B, S, H, KV, hd,
                                                 err.data_ptr(), _stream()))

    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ms = _time(run, args.iters)
    assert int(err.item()) == 0
    T = B * S
    nbytes = 4.0 * T * (lat + 2 * kvd) + 6.0 * (lat * hd + lat * lat + kvd * hd + kvd * kvd)
    flops = 6.0 * T * (lat * hd + lat * lat + kvd * hd + kvd * kvd)
    return {"kernel": "ccgqa_pre_tc_kernel<32>", "shape": [B, S, lat + 2 * kvd], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes,
            "conv_tflops": flops / (ms * 1e-3) / 1e12}


def attention(args) -> dict:
    B, S, H, KV, hd = args.batch, 2048, 8, 2, 32
    q = _rand_bf16(B, H, S, hd)
    q = torch.nn.functional.normalize(q.float(), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(_rand_bf16(B, KV, S, hd, seed=1).float(), dim=-1).to(torch.bfloat16)
    v = _rand_bf16(B, KV, S, hd, seed=2)
    o = torch.empty(B, S, H * hd, dtype=torch.bfloat16, device="cuda")
    lib = _lib.lib()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    bound = 0.0 if args.impl == 1 else 1.02 / math.sqrt(hd)     # q, k are unit vectors here
    ms = _time(lambda i: _lib.check(lib.hb200_attention_causal_gqa(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                                    B, S, H, KV, hd, 1.0 / math.sqrt(hd), bound,
                                                                    err.data_ptr(), _stream())),
               args.iters)
    assert int(err.item()) == 0
    flops = 4.0 * B * S * H * hd * (S + 1) / 2
    return {"kernel": "attention_tcgen05_kernel<32>" if args.impl == 0 else "attention_causal_gqa_kernel<32> (mma.sync)",
            "shape": [B, H, S, hd], "ms": ms, "bound": "tensor",
            "achieved": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "algorithmic_flops": flops,
            "note": "exp-throughput limited at head_dim 32: one ex2 per 128 MMA FLOPs"}


def rms_norm(args) -> dict:
    """Config 3: RMSNorm on 16384 x 1024 bf16, gain ~ N(1, 0.02): 4 B/element moved."""
    T, D = 16384, 1024
    ns = _sets(T * D * 4)
    xs = [_rand_bf16(T, D, seed=i) for i in range(ns)]
    w = (1 + 0.02 * torch.randn(D, device="cuda")).float()
    ys = [torch.empty_like(x) for x in xs]
    lib = _lib.lib()
    ms = _time(lambda i: _lib.check(lib.hb200_rms_norm(xs[i % ns].data_ptr(), w.data_ptr(), ys[i % ns].data_ptr(), T, D,
                                                       1e-6, 1, 0, _stream())), args.iters)
    nbytes = 4.0 * T * D + 4 * D
    return {"kernel": "rms_norm_vec_kernel<bf16,float,4>", "shape": [T, D], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes}


def rope(args) -> dict:
    """Config 3: RoPE theta 1e4, head_dim 32, positions 0..2047, q-shaped [8,8,2048,32] bf16: 4 B/element moved."""
    B, H, S, hd = 8, 8, 2048, 32
    n = B * H * S * hd
    ns = _sets(n * 4)
    xs = [_rand_bf16(B, H, S, hd, seed=i) for i in range(ns)]
    ys = [torch.empty_like(x) for x in xs]
    cos, sin = rope_tables(S, hd, torch.device("cuda"))
    lib = _lib.lib()
    ms = _time(lambda i: _lib.check(lib.hb200_rope(xs[i % ns].data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                                   ys[i % ns].data_ptr(), B, H, S, hd, H * S * hd, S * hd, hd, hd // 2, 1,
                                                   _stream())), args.iters)
    nbytes = 4.0 * n
    return {"kernel": "rope_kernel<bf16,vec>", "shape": [B, H, S, hd], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes}


def swiglu_ffn(args) -> dict:
    """Config 3: SwiGLU FFN 1024 -> 2816 -> 1024 on 16384 tokens, weights N(0, 0.02): 283.5 GFLOP; the activation is
    fused into the gate_up GEMM epilogue, so the [T, 2*2816] intermediate never reaches HBM."""
    T, D, F = 16384, 1024, 2816
    x = _rand_bf16(T, D)
    wgu = interleave_gate_up(_rand_bf16(2 * F, D, scale=0.02, seed=1), torch.device("cuda", torch.cuda.current_device()))
    wd = _rand_bf16(D, F, scale=0.02, seed=2)
    act = torch.empty(T, F, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = _lib.lib()

    def run(i):
        _lib.check(lib.hb200_gemm_bf16(x.data_ptr(), wgu.data_ptr(), act.data_ptr(), T, 2 * F, D, D, D, F, 2, None, 1.0,
                                       None, None, 0, err.data_ptr(), _stream()))
        _lib.check(lib.hb200_gemm_bf16(act.data_ptr(), wd.data_ptr(), y.data_ptr(), T, D, F, F, F, D, 0, None, 1.0,
                                       None, None, 0, err.data_ptr(), _stream()))

    ms = _time(run, args.iters)
    assert int(err.item()) == 0
    flops = 6.0 * T * D * F
    return {"kernel": "swiglu_ffn (gate_up GEMM + SwiGLU epilogue, down GEMM)", "shape": [T, D, F], "ms": ms,
            "bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "algorithmic_flops": flops}


def swiglu_act(args) -> dict:
    """The exported fused_swiglu op alone (6*F bytes per token when left unfused)."""
    T, F = 16384, 2816
    ns = _sets(T * F * 6)
    gu = [_rand_bf16(T, 2 * F, seed=i) for i in range(ns)]
    ms = _time(lambda i: kernels.fused_swiglu(*gu[i % ns].chunk(2, dim=-1)), args.iters)
    nbytes = 6.0 * T * F
    return {"kernel": "swiglu_kernel<bf16,vec>", "shape": [T, F], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes,
            "note": "includes the torch custom-op dispatch and output allocation"}


def model_hidden(args) -> dict:
    """The 250M model without the output projection (forward_hidden), batch x 2048: a few GB on the device, every
    block kernel at its full-size shape - the command used to capture the row / routing kernels under ncu."""
    from hydra_b200.model import HydraB200Model, random_state_dict
    arch = dict(vocab_size=50257, dim=1024, n_mor_blocks=10, recursions_per_block=4, n_heads=8, n_kv_heads=2,
                compression_factor=4, mlp_ratio=2.67, mod_capacity=0.75)
    sd = random_state_dict(seed=0, device="cuda", **arch)
    m = HydraB200Model(sd, n_heads=8, n_kv_heads=2, max_seq_len=2048, mod_capacity=0.75, device="cuda")
    B = args.batch
    ids = torch.randint(0, 50257, (B, 2048), generator=torch.Generator().manual_seed(1)).cuda()
    ms = _time(lambda i: m.forward_hidden(ids), args.iters, warmup=1)
    m.check_device_errors()
    return {"kernel": "HydraB200Model.forward_hidden (10 blocks, no lm_head)", "shape": [B, 2048, 1024], "ms": ms,
            "bound": "tensor", "achieved": B * 2048 / (ms * 1e-3) / 1e6, "unit": "Mtok/s"}


def decode(args) -> dict:
    """Cached greedy decode at the 1.5B shape (dim 2048, 22 blocks x 4 recursions, 32 query / 4 KV heads of 16,
    F 5632, MoD 0.75): `batch` sequences per GPU, prompt of 1024 uniform-random tokens, 256 new tokens.  Reports the
    decode phase (steps replayed from one CUDA graph) against the weight-streaming bound: every step reads each
    weight once (the activations of `batch` rows are negligible) plus the cached keys / values of every position."""
    from hydra_b200.model import HydraB200Model, random_state_dict
    arch = dict(vocab_size=50257, dim=2048, n_mor_blocks=args.blocks, recursions_per_block=4, n_heads=32, n_kv_heads=4,
                compression_factor=4, mlp_ratio=2.67, mod_capacity=0.75)
    sd = random_state_dict(seed=0, device="cuda", **arch)
    P, n_new = args.prompt, args.new_tokens
    m = HydraB200Model(sd, n_heads=32, n_kv_heads=4, max_seq_len=P + n_new, mod_capacity=0.75, device="cuda")
    weight_bytes = 2.0 * sum(v.numel() for k, v in sd.items() if v.dim() >= 2 and "router" not in k and "recursion" not in k)
    del sd
    B = args.batch
    prompt = torch.randint(0, 50257, (B, P), generator=torch.Generator().manual_seed(1)).cuda()
    sess = m.new_decode_session(B, P + n_new)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    sess.prefill(prompt)                      # warm-up of the prefill kernels
    torch.cuda.synchronize()
    ev[0].record()
    sess.prefill(prompt)
    ev[1].record()
    graph = os.environ.get("HB200_DECODE_GRAPH", "1") != "0"
    sess.step(use_graph=False)                # direct launch (one-time kernel setup), then the graph is captured
    sess.step(use_graph=graph)
    torch.cuda.synchronize()
    ev[2].record()
    steps = n_new - 3
    for _ in range(steps):
        sess.step(use_graph=graph)
    ev[3].record()
    torch.cuda.synchronize()
    m.check_device_errors()
    prefill_ms, decode_ms = ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])
    # positions cached while the timed steps ran: P+2 .. P+2+steps-1, keys and values of 4 KV heads x 16
    mean_pos = P + 2 + (steps - 1) / 2.0
    kv_bytes = 2.0 * 2.0 * B * 4 * 16 * mean_pos * args.blocks
    step_ms = decode_ms / steps
    nbytes = weight_bytes + kv_bytes
    return {"kernel": "hb200_model_decode_step (%s)" % ("CUDA graph replay" if graph else "direct launches"), "shape": [B, P, n_new], "ms": step_ms,
            "bound": "hbm", "achieved": nbytes / (step_ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes,
            "decode_tok_per_s": B / (step_ms * 1e-3), "timed_steps": steps,
            "note": "prefill of the prompt measured separately: %.1f ms; weights %.2f GB + cache reads %.3f GB per step"
                    % (prefill_ms, weight_bytes / 1e9, kv_bytes / 1e9)}


def sample_rows(args) -> dict:
    """Next-token sampling (temperature 0.8, top-k 50, top-p 0.9: the reference sampler's defaults) and the greedy
    argmax on --batch logit rows of 50257 bf16 columns: one read of the rows is the algorithmic traffic."""
    from hydra_b200.sampling import sample_rows as sample
    B, V, ld = int(args.batch), 50257, 50264
    ns = _sets(B * ld * 2)
    xs = [_rand_bf16(B, ld, scale=2.5, seed=i) for i in range(ns)]
    u = torch.rand(B, device="cuda")
    out = torch.empty(B, dtype=torch.int64, device="cuda")
    lib = _lib.lib()
    sample(xs[0], 0.8, 50, 0.9, uniforms=u, vocab=V, out=out)           # the public wrapper once; timed below without it

    def call(i, t, k, p):
        _lib.check(lib.hb200_sample_rows(xs[i % ns].data_ptr(), B, V, ld, t, k, p, u.data_ptr(), out.data_ptr(), _stream()))
    ms = _time(lambda i: call(i, 0.8, 50, 0.9), args.iters)
    ms_nuc = _time(lambda i: call(i, 1.0, 0, 0.9), args.iters)
    ms_arg = _time(lambda i: _lib.check(lib.hb200_argmax_rows(xs[i % ns].data_ptr(), B, V, ld, out.data_ptr(), _stream())),
                   args.iters)
    nbytes = 2.0 * B * V
    return {"kernel": "sample_rows_kernel", "shape": [B, V], "ms": ms, "bound": "hbm",
            "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "algorithmic_bytes": nbytes,
            "ms_nucleus_only": ms_nuc, "ms_argmax_rows": ms_arg}


# ------------------------------------------------------------------------------------------------------------
def _time_us(fn: Callable[[int], None], iters: int = 10, warmup: int = 3) -> float:
    return _time(fn, iters, warmup) * 1e3


def library_baseline(gemm_rows: int, root: str, ref_model_args: dict | None = None, iters: int = 10) -> dict:
    """The library calls the reference makes on a CUDA device, timed on this GPU beside this package's kernels at the
    same shapes (CUDA events, same process): ``F.linear`` (cuBLAS) for the five contractions of the 250M model
    (hydra/layers/common.py:221-230, attention.py:122-124), ``F.scaled_dot_product_attention(is_causal=True,
    enable_gqa=True)`` at the CCGQA-block microbenchmark shape (attention.py:288-299), the four ``Conv1d`` calls with
    their transposes and pads as the reference issues them (kernels/fused_conv.py:39-62; compared with the whole fused
    pre-attention kernel, which also does the QK-mean, L2 norm, RoPE and value shift), and - when the reference
    package is present under oracle/_ref - the reference's own bf16 eager model at the prefill workload.
    ``gemm_rows``: rows of the gate_up / down contractions (the average number of rows routed to them per launch)."""
    import torch.nn.functional as F
    T, D, Fh, V = 65536, 1024, 2816, 50257
    lib = _lib.lib()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out: dict = {"method": f"CUDA events, {iters} launches after 3 warm-up launches, one process, operands larger than L2"}

    def ours_gemm(A, W, Cm, M, N, K, epi, ldc):
        return lambda i: _lib.check(lib.hb200_gemm_bf16(A.data_ptr(), W.data_ptr(), Cm.data_ptr(), M, N, K, K, K, ldc, epi,
                                                        None, 1.0, None, None, 0, err.data_ptr(), _stream()))

    gemms = {}
    Mr = max(128, (int(gemm_rows) + 127) // 128 * 128)
    for name, (M, N, K) in {"qkv": (T, 384, D), "o_proj": (T, D, 256), "gate_up": (Mr, 2 * Fh, D), "down": (Mr, D, Fh),
                            "lm_head": (T, V, D)}.items():
        A = _rand_bf16(M, K, seed=3)
        W = _rand_bf16(N, K, scale=0.03, seed=4)
        ldc = (N + 63) // 64 * 64                 # rows on 128-byte boundaries, as the model lays its logits out
        Cm = torch.empty(M, ldc, dtype=torch.bfloat16, device="cuda")
        flops = 2.0 * M * N * K
        t_lib = _time_us(lambda i: F.linear(A, W), iters)
        if name == "gate_up":
            # ours fuses the SwiGLU activation into the epilogue; the library side is the bare contraction plus the
            # reference's separate activation pass over the [M, 2F] result (common.py:224-230)
            Wi = interleave_gate_up(W, torch.device("cuda", torch.cuda.current_device()))
            act = torch.empty(M, Fh, dtype=torch.bfloat16, device="cuda")
            t_ours = _time_us(ours_gemm(A, Wi, act, M, N, K, 2, Fh), iters)

            def lib_mlp(i):
                gu = F.linear(A, W)
                g, u = gu.chunk(2, dim=-1)
                return F.silu(g) * u
            t_lib_act = _time_us(lib_mlp, iters)
            gemms[name] = {"shape": [M, N, K], "torch_us": t_lib, "torch_with_activation_us": t_lib_act, "ours_us": t_ours,
                           "torch_tflops": flops / t_lib / 1e6, "ours_tflops": flops / t_ours / 1e6,
                           "note": "ours includes the SwiGLU epilogue"}
        else:
            t_ours = _time_us(ours_gemm(A, W, Cm, M, N, K, 0, ldc), iters)
            gemms[name] = {"shape": [M, N, K], "torch_us": t_lib, "ours_us": t_ours,
                           "torch_tflops": flops / t_lib / 1e6, "ours_tflops": flops / t_ours / 1e6}
        del A, W, Cm
    assert int(err.item()) == 0
    out["gemm"] = gemms

    # attention core, config 2
    B, S, H, KV, hd = 8, 2048, 8, 2, 32
    q = torch.nn.functional.normalize(_rand_bf16(B, H, S, hd).float(), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(_rand_bf16(B, KV, S, hd, seed=1).float(), dim=-1).to(torch.bfloat16)
    v = _rand_bf16(B, KV, S, hd, seed=2)
    o = torch.empty(B, S, H * hd, dtype=torch.bfloat16, device="cuda")
    t_sdpa = _time_us(lambda i: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True), iters)
    t_att = _time_us(lambda i: _lib.check(lib.hb200_attention_causal_gqa(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, S, H, KV, hd, 1.0 / math.sqrt(hd),
        1.02 / math.sqrt(hd), err.data_ptr(), _stream())), iters)
    out["attention"] = {"shape": [B, H, S, hd], "torch_sdpa_us": t_sdpa, "ours_us": t_att}

    # the reference's conv path at config 2: [B,S,C] -> transpose -> pad -> grouped conv -> pad -> dense conv -> transpose
    lat, kvd = H * hd, KV * hd
    xq, xk = _rand_bf16(B, S, lat, seed=5), _rand_bf16(B, S, kvd, seed=6)
    wq1, wq2 = _rand_bf16(lat, hd, 3, scale=0.05, seed=7), _rand_bf16(lat, lat, 3, scale=0.05, seed=8)
    wk1, wk2 = _rand_bf16(kvd, hd, 3, scale=0.05, seed=9), _rand_bf16(kvd, kvd, 3, scale=0.05, seed=10)

    def conv_seq(x, w1, w2, groups):
        y = x.transpose(1, 2).contiguous()
        y = F.conv1d(F.pad(y, (2, 0)), w1, groups=groups)
        y = F.conv1d(F.pad(y, (2, 0)), w2)
        return y.transpose(1, 2).contiguous()

    def convs(i):
        conv_seq(xq, wq1, wq2, H)
        conv_seq(xk, wk1, wk2, KV)
    t_conv = _time_us(convs, iters)
    ns = argparse_like(batch=B, iters=iters)
    out["convs"] = {"shape": [B, S, lat + kvd], "torch_conv1d_x4_us": t_conv,
                    "ours_whole_pre_attention_us": pre_attention(ns)["ms"] * 1e3,
                    "note": "ours is the whole fused pre-attention kernel (value shift, both conv pairs, QK-mean, L2 norm, "
                            "temperature, RoPE); the library side is the two conv pairs only"}

    if ref_model_args is not None:
        out["reference_eager_bf16"] = reference_eager_on_gpu(ref_model_args, root)
    return out


class argparse_like:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def reference_eager_on_gpu(ref_model_args: dict, root: str) -> dict:
    """The reference's own HydraModel (unmodified package under oracle/_ref), bf16, eager, on this GPU at the prefill
    workload (diagnostics/benchmark_hydra_models.py:133-143 times it this way): tokens/s of its forward."""
    import sys
    sys.path.insert(0, root) if root not in sys.path else None
    from oracle import build_ref
    if not build_ref.add_ref_to_path():
        return {"unavailable": "oracle/_ref has not been built"}
    try:
        model = build_ref.reference_model(**ref_model_args).cuda().bfloat16()
    except Exception as e:   # pragma: no cover - depends on the box
        return {"unavailable": f"building the reference model failed: {type(e).__name__}: {e}"[:300]}
    S = ref_model_args["max_seq_len"]
    res = {}
    for B in (32, 8):
        try:
            ids = torch.randint(0, ref_model_args["vocab_size"], (B, S), device="cuda")
            with torch.no_grad():
                ms = _time(lambda i: build_ref.reference_forward(model, ids), 3, warmup=2)
            res = {"batch": B, "seq_len": S, "ms": ms, "tok_per_s": B * S / (ms * 1e-3),
                   "kernels": build_ref.reference_kernel_status()}
            break
        except torch.cuda.OutOfMemoryError:
            torch.cuda.empty_cache()
            res = {"unavailable": f"out of memory at batch {B}"}
        except Exception as e:   # pragma: no cover
            res = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
            break
    del model
    torch.cuda.empty_cache()
    return res


CASES: Dict[str, Callable] = {
    "decode": decode, "gemm_skinny": gemm_skinny, "sample_rows": sample_rows,
    "gemm": gemm, "ccgqa_block": ccgqa_block, "pre_attention": pre_attention, "attention": attention,
    "rms_norm": rms_norm, "rope": rope, "swiglu_ffn": swiglu_ffn, "swiglu_act": swiglu_act,
    "model_hidden": model_hidden,
}


def run(name: str, args, root: str) -> dict:
    peaks, src = _peaks(root)
    res = CASES[name](args)
    if res["bound"] == "hbm":
        peak = float(peaks["hbm_gbs"])
    else:
        peak = float(peaks["bf16_tflops"])   # burst figure: the kernel is timed alone
    res.update({"micro": name, "peak": peak, "frac": res["achieved"] / peak, "peak_source": src, "iters": args.iters})
    return res
