"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Usage (only where the reference tree is available):

    PYTHONPATH=<reference root> python tests/golden/make_golden.py          # every fixture
    PYTHONPATH=<reference root> python tests/golden/make_golden.py base     # only base_model_hd16.npz

The reference (pure Python + PyTorch) is imported, its modules are built on CPU
with a fixed seed, weights are rounded to bf16-representable values (so that a
bf16 device path can start from identical bits; they are stored as raw bf16 bit
patterns, uint16), the reference's own fp32 eval forward is run, and inputs,
weights and outputs are written as ``.npz`` files.  Nothing here is imported by
the package; the fixtures are read by ``tests/``.

No dataset or public benchmark is involved: inputs are seeded synthetic tensors,
as in the reference's own benchmarks.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_round_(t: torch.Tensor) -> torch.Tensor:
    t.data.copy_(t.data.to(torch.bfloat16).to(t.dtype))
    return t


def to_bits(t: torch.Tensor) -> np.ndarray:
    """fp32 tensor holding bf16-representable values -> uint16 bit patterns."""
    b = t.detach().to(torch.bfloat16).contiguous().view(torch.int16).numpy().astype(np.uint16)
    return b


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).contiguous().numpy()


def save(name: str, **arrs) -> None:
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrs)
    print(f"wrote {path}: {os.path.getsize(path) / 1e6:.2f} MB")


# ----------------------------------------------------------------------------
def gen_fused_ops() -> None:
    from hydra.kernels import fused_ops as fo
    from hydra.layers.common import AdaRMSNorm, RMSNorm

    g = torch.Generator().manual_seed(2)
    out = {}
    # RoPE, head_dim 32 and 16, 4-D tables as the attention module passes them
    for hd in (16, 32):
        x = torch.randn(2, 3, 40, hd, generator=g)
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
        ang = torch.outer(torch.arange(64, dtype=torch.float32), inv)
        cos, sin = ang.cos()[None, None], ang.sin()[None, None]
        out[f"rope{hd}_x"] = f32(x)
        out[f"rope{hd}_cos"] = f32(cos)
        out[f"rope{hd}_sin"] = f32(sin)
        out[f"rope{hd}_y"] = f32(fo._rope_pytorch(x, cos, sin))
    q = torch.randn(2, 8, 24, 32, generator=g)
    k = torch.randn(2, 2, 24, 32, generator=g)
    qn, kn = fo._qk_norm_pytorch(q, k, 5.0, 1.7)
    out.update(qkn_q=f32(q), qkn_k=f32(k), qkn_qo=f32(qn), qkn_ko=f32(kn))
    gate = torch.randn(37, 264, generator=g) * 3
    up = torch.randn(37, 264, generator=g)
    out.update(swiglu_gate=f32(gate), swiglu_up=f32(up), swiglu_y=f32(fo._swiglu_pytorch(gate, up)))
    x = torch.randn(19, 1024, generator=g)
    w = 1.0 + 0.02 * torch.randn(1024, generator=g)
    out.update(rms_x=f32(x), rms_w=f32(w), rms_y=f32(fo._rms_norm_pytorch(x, w, 1e-6)))
    n1 = RMSNorm(1024)
    n1.weight.data.copy_(w)
    out["rms_module_y"] = f32(n1(x))
    n2 = AdaRMSNorm(1024)
    n2.weight.data.copy_(w)
    out["ada_y"] = f32(n2(x))
    save("fused_ops.npz", **out)


# ----------------------------------------------------------------------------
def gen_attention_ablated(name: str, dim: int, H: int, KV: int, B: int, S: int, seed: int) -> None:
    """The reference module built with each of its ablation switches off in turn, two off, all of them off, and with conv
    kernel sizes 2 and 5 (attention.py:74-160): one variant per entry, each with its own weights (`v{i}:w:` keys), the
    same input."""
    from hydra.attention import build_hybrid_attention_module

    stages = ["rope", "qk_norm", "convs", "qk_mean", "value_shift"]
    variants = [[s_] for s_ in stages] + [["convs", "qk_mean"], stages, ["ksize=2"], ["ksize=5"]]
    g = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(B, S, dim, generator=g).to(torch.bfloat16).to(torch.float32)
    arrs = dict(meta=np.array([dim, H, KV, B, S], dtype=np.int64), x=to_bits(x),
                variants=np.array([",".join(v) for v in variants]))
    for i, off in enumerate(variants):
        torch.manual_seed(seed + i)
        kw = {f"use_{s_}": (s_ not in off) for s_ in stages}
        for tag in off:
            if tag.startswith("ksize="):                  # a variant with another conv kernel size, every stage on
                kw["conv_kernel_size"] = int(tag[6:])
        m = build_hybrid_attention_module("ccgqa", dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S,
                                          compression_factor=4, attention_kwargs=kw)
        with torch.no_grad():
            for p in m.parameters():
                if p.dim() >= 2:
                    torch.nn.init.xavier_uniform_(p)
            for p in m.parameters():
                bf16_round_(p)
        m.eval()
        for s_ in stages:
            assert getattr(m, f"use_{s_}") == (s_ not in off)
        with torch.no_grad():
            arrs[f"v{i}:y"] = f32(m(x))
        for kname, t in m.state_dict().items():
            arrs[f"v{i}:w:" + kname] = to_bits(t) if t.dim() >= 2 else f32(t)
    save(name, **arrs)


# ----------------------------------------------------------------------------
def gen_attention_masked(name: str, dim: int, H: int, KV: int, S: int, seed: int) -> None:
    """CCGQAAttention.forward(x, mask) as the reference computes it (attention.py:269-283): one sequence per mask
    pattern - all valid, right-padded, left-padded, holes, all padded.  `y` is the reference's output as it is; the
    boolean mask it hands to SDPA is True for future and padded keys, which SDPA reads as "take part"."""
    from hydra.attention import build_hybrid_attention_module

    torch.manual_seed(seed)
    m = build_hybrid_attention_module("ccgqa", dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S,
                                      compression_factor=4, attention_kwargs={})
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                torch.nn.init.xavier_uniform_(p)
        for p in m.parameters():
            bf16_round_(p)
    m.eval()
    g = torch.Generator().manual_seed(seed + 100)
    mask = torch.ones(5, S, dtype=torch.int64)
    mask[1, S - 7:] = 0                                   # right padding
    mask[2, :5] = 0                                       # left padding
    mask[3] = (torch.rand(S, generator=g) > 0.3).long()   # holes
    mask[4] = 0                                           # nothing valid
    x = torch.randn(5, S, dim, generator=g).to(torch.bfloat16).to(torch.float32)
    with torch.no_grad():
        y = m(x, mask)
        y_plain = m(x)
    arrs = dict(meta=np.array([dim, H, KV, 5, S], dtype=np.int64), x=to_bits(x), mask=mask.numpy(), y=f32(y),
                y_plain=f32(y_plain))
    for kname, t in m.state_dict().items():
        arrs["w:" + kname] = to_bits(t) if t.dim() >= 2 else f32(t)
    save(name, **arrs)


# ----------------------------------------------------------------------------
def gen_attention(name: str, dim: int, H: int, KV: int, B: int, S: int, seed: int,
                  temperature: float | None = None) -> None:
    from hydra.attention import build_hybrid_attention_module
    import hydra.attention.backends.ccgqa.attention as attn_mod

    torch.manual_seed(seed)
    m = build_hybrid_attention_module("ccgqa", dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S,
                                      compression_factor=4, attention_kwargs={})
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                torch.nn.init.xavier_uniform_(p)
        if temperature is not None:
            m.key_temperature.fill_(temperature)
        for p in m.parameters():
            bf16_round_(p)
    m.eval()
    g = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(B, S, dim, generator=g).to(torch.bfloat16).to(torch.float32)

    captured = {}
    real_sdpa = F.scaled_dot_product_attention

    def tap(q, k, v, *a, **kw):
        captured["q"], captured["k"], captured["v"] = q.clone(), k.clone(), v.clone()
        o = real_sdpa(q, k, v, *a, **kw)
        captured["o"] = o.clone()
        return o

    attn_mod.F.scaled_dot_product_attention = tap
    try:
        with torch.no_grad():
            y = m(x)
            qkv = m.qkv_proj(x)
    finally:
        attn_mod.F.scaled_dot_product_attention = real_sdpa
    G = H // KV
    arrs = dict(
        meta=np.array([dim, H, KV, B, S], dtype=np.int64),
        x=to_bits(x), y=f32(y), qkv=f32(qkv),
        q=f32(captured["q"]), k=f32(captured["k"][:, ::G]), v=f32(captured["v"][:, ::G]),
        o=f32(captured["o"]),
    )
    for kname, t in m.state_dict().items():
        arrs["w:" + kname] = to_bits(t) if t.dim() >= 2 else f32(t)
    save(name, **arrs)


# ----------------------------------------------------------------------------
def gen_model(name: str, *, vocab: int, dim: int, NB: int, R: int, H: int, KV: int, mlp_ratio: float,
              B: int, S: int, cap: float, seed: int, tie: bool = True, static: bool = False,
              rampup: float = 1.0, fresh: bool = False) -> None:
    from hydra.model.framework import HydraModel

    torch.manual_seed(seed)
    m = HydraModel(vocab_size=vocab, dim=dim, n_mor_blocks=NB, recursions_per_block=R, n_heads=H,
                   n_kv_heads=KV, compression_factor=4, mlp_ratio=mlp_ratio, max_seq_len=S,
                   mod_capacity=cap, tie_weights=tie, static_routing_mode=static)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("norm1.weight") or n.endswith("norm2.weight") or n.endswith("final_norm.weight") \
                    or n == "norm.weight":
                p.mul_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            if "recursion_bias" in n:
                p.copy_(0.05 * torch.randn(p.shape, generator=g))
            if "router.weight" in n:
                p.mul_(10.0)
        for p in m.parameters():
            bf16_round_(p)
    m.eval()
    if rampup < 1.0:             # MoR curriculum in the middle of its ramp: scale = steps since enable / ramp steps
        m.set_mor_curriculum(enable_step=10 ** 6 - int(round(rampup * 1000)) + 1, rampup_steps=1000)
    if not fresh:                # fresh: the model as constructed - MoD still in its warm-up, every token through the MLP
        m.set_global_step(10 ** 6)   # MoD hard routing is off in eval until the step passes its warm-up
    if rampup < 1.0:
        assert abs(m.layers[0].get_mor_rampup_scale() - rampup) < 1e-9
    ids = torch.randint(0, vocab, (B, S), generator=torch.Generator().manual_seed(seed + 2))
    ids[0, 0] = vocab + 5        # out-of-range ids are clamped by the reference
    ids[0, 1] = -3

    mod_calls = []
    hooks = []
    for li, layer in enumerate(m.layers):
        if layer.mod_mlp_wrapper is not None:
            def hook(_mod, _inp, outp, li=li):
                mod_calls.append((li, outp[1].clone(), outp[2].clone()))
            hooks.append(layer.mod_mlp_wrapper.mod_router.register_forward_hook(hook))
    block_out = []
    for layer in m.layers:
        hooks.append(layer.register_forward_hook(lambda _m, _i, o: block_out.append(o.clone())))
    with torch.no_grad():
        logits = m(ids)
    depths = [layer._last_depths.clone() for layer in m.layers]
    rlogits = [layer._last_router_logits.clone() for layer in m.layers]
    for h in hooks:
        h.remove()

    arrs = dict(
        meta=np.array([vocab, dim, NB, R, H, KV, B, S], dtype=np.int64),
        cap=np.array([cap], dtype=np.float64),
        ffn_hidden=np.array([m.layers[0].mlp.down.weight.shape[1]], dtype=np.int64),
        ids=ids.numpy(), logits=f32(logits), static=np.array([int(static)], dtype=np.int64),
        rampup=np.array([rampup], dtype=np.float64),
    )
    # what HydraB200Model.from_reference would read off this instance (checked on the GPU against the logits above)
    import json
    from hydra_b200.model import HydraB200Model
    arrs["reference_kwargs"] = np.frombuffer(json.dumps(HydraB200Model.reference_kwargs(m)).encode(), dtype=np.uint8)
    for i, d in enumerate(depths):
        arrs[f"depths:{i}"] = d.numpy().astype(np.int32)
        arrs[f"router_logits:{i}"] = f32(rlogits[i])
        arrs[f"block_out:{i}"] = f32(block_out[i])
    per_layer = {}
    for li, idx, sc in mod_calls:
        r = per_layer.get(li, 0)
        per_layer[li] = r + 1
        arrs[f"mod_idx:{li}:{r}"] = torch.sort(idx, dim=1)[0].numpy().astype(np.int32)
        arrs[f"mod_scores:{li}:{r}"] = f32(sc)
    for kname, t in m.state_dict().items():
        if (kname == "output.weight" and tie) or "_aux_loss" in kname or ".mod_mlp_wrapper.mlp." in kname:
            continue   # tied / alias / bookkeeping tensors
        arrs["w:" + kname] = to_bits(t) if t.dim() >= 2 and t.numel() > 4096 else f32(t)

    # fixed-depth path (adaptive=False) and min_depth=1 on the same weights
    for layer in m.layers:
        layer.adaptive = False
    with torch.no_grad():
        arrs["logits_fixed"] = f32(m(ids))
    for layer in m.layers:
        layer.adaptive = True
        object.__setattr__(layer.mor_router.config, "min_depth", 1)   # frozen dataclass
    with torch.no_grad():
        arrs["logits_min1"] = f32(m(ids))
    for i, layer in enumerate(m.layers):
        arrs[f"depths_min1:{i}"] = layer._last_depths.numpy().astype(np.int32)
    # the reference's own bf16 path (whole module cast, as its bf16 benchmark does) on the same inputs
    for layer in m.layers:
        object.__setattr__(layer.mor_router.config, "min_depth", 0)
    mb = m.to(torch.bfloat16)   # in place, after every fp32 run (its routers do not survive deepcopy)
    mb.eval()
    mb.set_global_step(10 ** 6)
    with torch.no_grad():
        lb = mb(ids).float()
    err = (lb - logits)
    arrs["ref_bf16_maxabs"] = np.array([float(err.abs().max())])
    arrs["ref_bf16_rel_l2"] = np.array([float(err.norm() / logits.norm())])
    agree = [float((mb.layers[i]._last_depths == depths[i]).float().mean()) for i in range(NB)]
    arrs["ref_bf16_depth_agree"] = np.array(agree)

    save(name, **arrs)


def gen_base_model(name: str, *, vocab: int, dim: int, n_layers: int, H: int, KV: int, mlp_ratio: float, B: int, S: int,
                   seed: int) -> None:
    """HydraBaseModel (no routing): logits, every block's output and the reference's own bf16 error."""
    from hydra.model.framework import HydraBaseModel

    torch.manual_seed(seed)
    m = HydraBaseModel(vocab_size=vocab, dim=dim, n_layers=n_layers, n_heads=H, n_kv_heads=KV, compression_factor=4,
                       mlp_ratio=mlp_ratio, max_seq_len=S)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("norm1.weight") or n.endswith("norm2.weight") or n == "norm.weight":
                p.mul_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
        for p in m.parameters():
            bf16_round_(p)
    m.eval()
    ids = torch.randint(0, vocab, (B, S), generator=torch.Generator().manual_seed(seed + 2))
    ids[0, 0] = vocab + 5
    ids[0, 1] = -3
    block_out = []
    hooks = [layer.register_forward_hook(lambda _m, _i, o: block_out.append(o.clone())) for layer in m.layers]
    with torch.no_grad():
        logits = m(ids)
    for h in hooks:
        h.remove()
    arrs = dict(meta=np.array([vocab, dim, n_layers, 1, H, KV, B, S], dtype=np.int64),
                cap=np.array([1.0], dtype=np.float64),
                ffn_hidden=np.array([m.layers[0].mlp.down.weight.shape[1]], dtype=np.int64),
                ids=ids.numpy(), logits=f32(logits))
    for i, bo in enumerate(block_out):
        arrs[f"block_out:{i}"] = f32(bo)
    for kname, t in m.state_dict().items():
        if kname == "output.weight":
            continue   # tied to tok_emb.weight
        arrs["w:" + kname] = to_bits(t) if t.dim() >= 2 and t.numel() > 4096 else f32(t)
    mb = m.to(torch.bfloat16)
    mb.eval()
    with torch.no_grad():
        lb = mb(ids).float()
    err = lb - logits
    arrs["ref_bf16_maxabs"] = np.array([float(err.abs().max())])
    arrs["ref_bf16_rel_l2"] = np.array([float(err.norm() / logits.norm())])
    import json
    from hydra_b200.model import HydraB200BaseModel
    arrs["reference_kwargs"] = np.frombuffer(json.dumps(HydraB200BaseModel.reference_kwargs(m)).encode(), dtype=np.uint8)
    save(name, **arrs)


def gen_sampler(name: str = "sampler.npz") -> None:
    """The filtered next-token distribution of the reference's generation helper (diagnostics/eval_checkpoint.py:
    111-166).  generate_text is run with a stand-in model that returns prepared logits and a stand-in tokenizer, and
    torch.multinomial is replaced for the call by a recorder that keeps the probabilities it is handed (and returns the
    most probable token), so what is stored is exactly what the reference would draw from."""
    import diagnostics.eval_checkpoint as E

    V = 1024
    g = torch.Generator().manual_seed(31)
    settings = [(0.8, 50, 0.9), (1.0, 0, 0.9), (0.7, 20, 1.0), (1.3, 0, 1.0), (0.5, 5, 0.5), (1.0, 200, 0.95),
                (2.0, 1000, 0.99), (0.25, 3, 0.1)]
    rows_per = 3
    logits, probs, used = [], [], []
    for (temp, k, p) in settings:
        rows = bf16_round_(torch.randn(rows_per, V, generator=g) * 3.0)
        rows[1, :40] = rows[1, 40]                       # a block of equal logits (ties at the thresholds)
        rec = []

        class Model(torch.nn.Module):
            calls = 0

            def forward(self, ids):
                r = rows[Model.calls]
                Model.calls += 1
                return r.view(1, 1, V).expand(1, ids.shape[1], V).clone()

        class Tok:
            eos_token_id = -1

            def encode(self, prompt, return_tensors="pt"):
                return torch.zeros(1, 1, dtype=torch.int64)

            def decode(self, ids, skip_special_tokens=True):
                return ""

        def recorder(pr, num_samples=1):
            rec.append(pr.clone())
            return pr.argmax(dim=-1, keepdim=True)

        keep = torch.multinomial
        torch.multinomial = recorder
        try:
            E.generate_text(Model(), Tok(), "x", max_new_tokens=rows_per, temperature=temp, top_k=k, top_p=p, device="cpu")
        finally:
            torch.multinomial = keep
        assert len(rec) == rows_per
        logits.append(rows)
        probs.append(torch.cat(rec, dim=0))
        used.extend([(temp, k, p)] * rows_per)
    save(name, logits=f32(torch.cat(logits)), probs=f32(torch.cat(probs)), settings=np.array(used, dtype=np.float64))


if __name__ == "__main__":
    try:
        import hydra  # noqa: F401
    except Exception as e:  # pragma: no cover
        sys.exit(f"the reference package 'hydra' must be importable (set PYTHONPATH): {e}")
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    if len(sys.argv) > 1 and sys.argv[1] == "base":     # only the routing-free baseline model
        gen_base_model("base_model_hd16.npz", vocab=384, dim=256, n_layers=3, H=4, KV=2, mlp_ratio=1.0, B=2, S=112, seed=8)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "sampler":  # only the sampler's filtered distributions
        gen_sampler()
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "fresh":    # only the freshly constructed model (MoD warm-up not passed)
        gen_model("model_fresh.npz", vocab=200, dim=256, NB=3, R=2, H=4, KV=2, mlp_ratio=1.0,
                  B=2, S=48, cap=0.5, seed=29, fresh=True)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "ablate":   # only the attention module with its ablation switches off
        gen_attention_ablated("ccgqa_ablated.npz", 256, 4, 2, 2, 24, seed=37)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "mask":     # only the attention module called with a padding mask
        gen_attention_masked("ccgqa_mask.npz", 256, 4, 2, 40, seed=31)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "rampup":   # only the model in the middle of its MoR ramp-up
        gen_model("model_rampup.npz", vocab=200, dim=256, NB=3, R=3, H=4, KV=2, mlp_ratio=1.0,
                  B=2, S=64, cap=0.75, seed=27, rampup=0.4)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "static":   # only the static-routing model
        gen_model("model_static.npz", vocab=200, dim=256, NB=3, R=3, H=4, KV=2, mlp_ratio=1.0,
                  B=2, S=64, cap=0.75, seed=23, static=True)
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "untied":   # only the model with its own output projection
        gen_model("model_untied.npz", vocab=200, dim=256, NB=3, R=2, H=4, KV=2, mlp_ratio=1.0,
                  B=2, S=64, cap=0.75, seed=21, tie=False)
        sys.exit(0)
    gen_fused_ops()
    # config-2 shapes (dim 1024, 8q/2kv, hd 32) at a short sequence; temperature 1.0 as in the CCGQA block microbenchmark
    gen_attention("ccgqa_hd32.npz", 1024, 8, 2, 1, 80, seed=1, temperature=1.0)
    # config-1 shapes (dim 512, 8q/2kv, hd 16), default temperature sqrt(hd)
    gen_attention("ccgqa_hd16.npz", 512, 8, 2, 2, 72, seed=3)
    # odd KV count: the value-shift split falls inside a head (100M preset: 12q/3kv)
    gen_attention("ccgqa_kv3.npz", 768, 12, 3, 1, 40, seed=4)
    # n_groups == 1 branch of the QK-mean coupling (H == KV)
    gen_attention("ccgqa_mha.npz", 256, 4, 4, 1, 33, seed=6)
    gen_attention_masked("ccgqa_mask.npz", 256, 4, 2, 40, seed=31)
    # whole model, 4 blocks so that blocks 1 and 2 carry MoD
    gen_model("model_hd16.npz", vocab=384, dim=256, NB=4, R=3, H=4, KV=2, mlp_ratio=1.0,
              B=2, S=128, cap=0.75, seed=0)
    gen_model("model_hd32.npz", vocab=384, dim=256, NB=3, R=4, H=2, KV=1, mlp_ratio=1.0,
              B=2, S=96, cap=0.5, seed=5)
    gen_base_model("base_model_hd16.npz", vocab=384, dim=256, n_layers=3, H=4, KV=2, mlp_ratio=1.0, B=2, S=112, seed=8)
    # tie_weights=False: the output projection is a matrix of its own
    gen_model("model_untied.npz", vocab=200, dim=256, NB=3, R=2, H=4, KV=2, mlp_ratio=1.0,
              B=2, S=64, cap=0.75, seed=21, tie=False)
    gen_sampler()
    # static_routing_mode=True: dense compute, soft routing weights (also honoured in eval)
    gen_model("model_static.npz", vocab=200, dim=256, NB=3, R=3, H=4, KV=2, mlp_ratio=1.0,
              B=2, S=64, cap=0.75, seed=23, static=True)
    # MoR curriculum mid-ramp: every block returns 0.4 * adaptive + 0.6 * fixed-depth
    gen_model("model_rampup.npz", vocab=200, dim=256, NB=3, R=3, H=4, KV=2, mlp_ratio=1.0,
              B=2, S=64, cap=0.75, seed=27, rampup=0.4)
    # a model as constructed (no set_global_step): MoD is still in its warm-up, so every token goes through the MLP
    gen_model("model_fresh.npz", vocab=200, dim=256, NB=3, R=2, H=4, KV=2, mlp_ratio=1.0,
              B=2, S=48, cap=0.5, seed=29, fresh=True)
