"""Pins the CPU oracle to the reference: every function of oracle/hydra_oracle.py is
checked against outputs of the reference's own code (fixtures in tests/golden/, made by
tests/golden/make_golden.py).  fp32, tolerance 2e-6 relative to the output scale; routing
index lists and depths must be identical."""
import numpy as np
import pytest
import torch

from oracle import hydra_oracle as O
from tests import golden_io as G


def close(a: torch.Tensor, b: np.ndarray, tol=2e-6):
    b = torch.from_numpy(b)
    scale = max(1.0, float(b.abs().max()))
    err = float((a - b).abs().max())
    assert err <= tol * scale, f"max abs err {err:.3e} (scale {scale:.3g})"


def test_fused_op_semantics():
    fx = G.load("fused_ops.npz")
    t = lambda k: torch.from_numpy(fx[k])
    for hd in (16, 32):
        close(O.rope(t(f"rope{hd}_x"), t(f"rope{hd}_cos"), t(f"rope{hd}_sin")), fx[f"rope{hd}_y"])
        c2, s2 = O.rope_tables(64, hd)
        close(c2, fx[f"rope{hd}_cos"][0, 0], 1e-7)
        close(s2, fx[f"rope{hd}_sin"][0, 0], 1e-7)
    qo, ko = O.qk_norm(t("qkn_q"), t("qkn_k"), 5.0, 1.7)
    close(qo, fx["qkn_qo"]); close(ko, fx["qkn_ko"])
    q2, k2 = O.qk_norm_rsqrt(t("qkn_q"), t("qkn_k"), 5.0, 1.7)   # device formula differs only by its eps
    close(q2, fx["qkn_qo"], 1e-5); close(k2, fx["qkn_ko"], 1e-5)
    close(O.swiglu(t("swiglu_gate"), t("swiglu_up")), fx["swiglu_y"])
    close(O.rms_norm(t("rms_x"), t("rms_w")), fx["rms_y"])
    close(O.rms_norm(t("rms_x"), t("rms_w")), fx["rms_module_y"])
    close(O.ada_rms_norm(t("rms_x"), t("rms_w")), fx["ada_y"])


@pytest.mark.parametrize("name", ["ccgqa_hd32.npz", "ccgqa_hd16.npz", "ccgqa_kv3.npz", "ccgqa_mha.npz"])
def test_ccgqa_attention(name):
    fx, cfg, w = G.attention_fixture(name)
    x = G.tensor(fx["x"])
    B, S, _ = x.shape
    qkv = x @ w["attn.qkv_proj.weight"].T
    close(qkv, fx["qkv"])
    cos, sin = O.rope_tables(S, cfg.head_dim)
    q, k, v = O.ccgqa_pre_attention(torch.from_numpy(fx["qkv"]), w, "attn.", cfg, cos, sin)
    close(q, fx["q"]); close(k, fx["k"]); close(v, fx["v"])
    o = O.causal_gqa_attention(torch.from_numpy(fx["q"]), torch.from_numpy(fx["k"]), torch.from_numpy(fx["v"]))
    close(o, fx["o"])
    close(O.ccgqa_forward(x, w, "attn.", cfg), fx["y"])


def test_ccgqa_attention_with_stages_switched_off():
    """The module's ablation switches (use_rope / use_qk_norm / use_convs / use_qk_mean / use_value_shift), each off in
    turn, two off, all off, and conv kernel sizes 2 and 5: the oracle against the reference module built that way."""
    fx, cfg, variants = G.ablated_attention_fixture("ccgqa_ablated.npz")
    x = G.tensor(fx["x"])
    assert len(variants) == 9 and [v[1]["attn.q_conv.conv1.weight"].shape[-1] for v in variants[-2:]] == [2, 5]
    for off, w, y in variants:
        assert ("attn.q_conv.conv1.weight" in w) == ("convs" not in off)      # no conv parameters without convolutions
        close(O.ccgqa_forward(x, w, "attn.", cfg, off=off), y.numpy())
    full = O.ccgqa_forward(x, variants[0][1], "attn.", cfg)
    assert float((full - variants[0][2]).abs().max()) > 1e-3                  # the switch does change the result


def test_ccgqa_attention_with_a_padding_mask():
    """CCGQAAttention.forward(x, mask) as the reference computes it (five mask patterns, run on the reference module):
    the "reference" semantics reproduce it - a query uses the keys after it and the padded ones, a query without any
    gives zeros -; the "intended" semantics are causal attention over the valid keys: an all-ones mask then changes
    nothing, and a sequence without a valid token gives zeros."""
    fx, cfg, w = G.attention_fixture("ccgqa_mask.npz")
    x, mask = G.tensor(fx["x"]), torch.from_numpy(fx["mask"])
    assert mask[0].all() and not mask[4].any()
    close(O.ccgqa_forward(x, w, "attn.", cfg, mask=mask), fx["y"])
    close(O.ccgqa_forward(x, w, "attn.", cfg), fx["y_plain"])
    assert float(torch.from_numpy(fx["y"])[0, -1].abs().max()) == 0.0
    yi = O.ccgqa_forward(x, w, "attn.", cfg, mask=mask, mask_semantics="intended")
    close(yi[0], fx["y_plain"][0])
    assert float(yi[4].abs().max()) == 0.0 and float(yi[2, :5].abs().max()) == 0.0
    # right padding: the valid prefix does not see the padding at all
    n = int(mask[1].sum())
    close(yi[1, :n], O.ccgqa_forward(x[1:2, :n], w, "attn.", cfg)[0].numpy())
    with pytest.raises(ValueError):
        O.ccgqa_forward(x, w, "attn.", cfg, mask=mask, mask_semantics="other")


@pytest.mark.parametrize("name", ["model_hd16.npz", "model_hd32.npz", "model_untied.npz"])
def test_model_forward_and_routing(name):
    fx, cfg, w = G.model_fixture(name)
    # model_untied.npz was made with tie_weights=False: the output projection is a matrix of its own
    assert ("output.weight" in w) == (name == "model_untied.npz")
    if "output.weight" in w:
        assert not torch.equal(w["output.weight"], w["tok_emb.weight"])
    ids = torch.from_numpy(fx["ids"])
    taps = O.RoutingTaps()
    logits = O.model_forward(ids, w, cfg, taps=taps)
    close(logits, fx["logits"], 5e-6)
    n_mod = 0
    for i in range(cfg.n_mor_blocks):
        assert np.array_equal(taps.depths[i].numpy().astype(np.int32), fx[f"depths:{i}"]), f"depths block {i}"
        # the reference keeps the squashed logit 3*tanh(l/2) (mixture_of_recursions.py:268-269)
        close(torch.tanh(taps.router_logits[i] / 2.0) * 3.0, fx[f"router_logits:{i}"], 5e-6)
        close(taps.block_out[i], fx[f"block_out:{i}"], 5e-6)
        for r in range(cfg.recursions_per_block):
            key = f"mod_idx:{i}:{r}"
            if cfg.block_has_mod(i):
                assert np.array_equal(taps.mod_indices[(i, r)].numpy().astype(np.int32), fx[key]), key
                close(taps.mod_scores[(i, r)], fx[f"mod_scores:{i}:{r}"], 5e-6)
                n_mod += 1
            else:
                assert key not in fx
    assert n_mod == (cfg.n_mor_blocks - 2) * cfg.recursions_per_block
    # depth spread: the fixture exercises more than one exit depth
    assert len(np.unique(np.concatenate([fx[f"depths:{i}"].ravel() for i in range(cfg.n_mor_blocks)]))) >= 2


@pytest.mark.parametrize("name", ["model_hd16.npz", "model_hd32.npz", "model_untied.npz"])
def test_model_fixed_depth_and_min_depth(name):
    fx, cfg, w = G.model_fixture(name)
    ids = torch.from_numpy(fx["ids"])
    cfg.adaptive = False
    close(O.model_forward(ids, w, cfg), fx["logits_fixed"], 5e-6)
    cfg.adaptive = True
    cfg.mor_min_depth = 1
    taps = O.RoutingTaps()
    close(O.model_forward(ids, w, cfg, taps=taps), fx["logits_min1"], 5e-6)
    for i in range(cfg.n_mor_blocks):
        assert np.array_equal(taps.depths[i].numpy().astype(np.int32), fx[f"depths_min1:{i}"])


def test_forced_routing_replay_is_identity():
    """Replaying a run's own routing decisions reproduces it exactly."""
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    ids = torch.from_numpy(fx["ids"])
    taps = O.RoutingTaps()
    a = O.model_forward(ids, w, cfg, taps=taps)
    b = O.model_forward(ids, w, cfg, forced=taps)
    assert torch.equal(a, b)


def test_mod_k_and_select_edges():
    assert O.mod_k(2048, 0.75) == 1536 and O.mod_k(512, 0.75) == 384
    assert O.mod_k(3, 0.0) == 1 and O.mod_k(5, 2.0) == 5 and O.mod_k(1, 0.75) == 1
    s = torch.tensor([[0.1, 0.9, -1.0, 0.5, 0.7]])
    assert O.mod_select(s, 0.6).tolist() == [[1, 3, 4]]


def test_mor_depths_rounding_half_even():
    # sigmoid(0) * 3 = 1.5 -> 2 (half to even); probs*2 = 1.0 stays
    d, p = O.mor_depths(torch.tensor([0.0, -50.0, 50.0]), 4)
    assert d.tolist() == [2, 0, 3]
    d1, _ = O.mor_depths(torch.tensor([-50.0, 50.0]), 4, min_depth=1)
    assert d1.tolist() == [1, 3]


def test_base_model_without_routing_matches_reference():
    """HydraBaseModel (HydraBlock layers, no routers, no exit norms): logits and every block output."""
    fx, cfg, w = G.model_fixture("base_model_hd16.npz")
    ids = torch.from_numpy(fx["ids"])
    taps = []
    lg = O.base_model_forward(ids, w, cfg, taps=taps)
    ref = torch.from_numpy(fx["logits"])
    assert float((lg - ref).abs().max()) <= 5e-6 * max(1.0, float(ref.abs().max()))
    for i, bo in enumerate(taps):
        r = torch.from_numpy(fx[f"block_out:{i}"])
        assert float((bo - r).abs().max()) <= 5e-6 * max(1.0, float(r.abs().max())), f"block {i}"


def test_sampler_filter_matches_the_reference_distributions():
    """tests/golden/sampler.npz holds the probabilities the reference's generate_text handed to torch.multinomial
    (diagnostics/eval_checkpoint.py:133-153) for prepared logits.  The oracle's filter must keep the same number of
    tokens with the same probabilities; which of several equal logits straddling the nucleus edge stays is the one
    thing the reference leaves to its sort, so membership may differ there and only there."""
    fx = G.load("sampler.npz")
    lg, pr, st = torch.from_numpy(fx["logits"]), torch.from_numpy(fx["probs"]), fx["settings"]
    differing = 0
    for r in range(lg.shape[0]):
        t, k, p = float(st[r, 0]), int(st[r, 1]), float(st[r, 2])
        q = torch.softmax(O.sample_filter(lg[r:r + 1], t, k, p), dim=-1)[0]
        assert int((q > 0).sum()) == int((pr[r] > 0).sum()), f"row {r}: kept-token count"
        close(q.sort().values, pr[r].sort().values.numpy(), 1e-6)
        diff = (q > 0) != (pr[r] > 0)
        if diff.any():
            differing += 1
            assert len(set(lg[r][diff].tolist())) == 1, f"row {r}: membership differs beyond one tied logit value"
        else:
            close(q, pr[r].numpy(), 1e-6)
    assert differing < lg.shape[0] // 2


def test_sampler_draw_is_the_inverse_cdf():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, 50, generator=g)
    # u -> 0 picks the most probable token, u -> 1 the least probable kept one
    lo = O.sample_next_token(x, 1.0, 10, 1.0, torch.zeros(3))
    assert torch.equal(lo, x.argmax(-1))
    hi = O.sample_next_token(x, 1.0, 10, 1.0, torch.full((3,), 0.9999999))
    assert torch.equal(hi, x.topk(10).indices[:, -1])
    # greedy limits
    assert torch.equal(O.sample_next_token(x, 0.0, 0, 1.0, torch.rand(3)), x.argmax(-1))
    assert torch.equal(O.sample_next_token(x, 0.8, 1, 0.9, torch.rand(3)), x.argmax(-1))
    # frequencies over many uniforms follow softmax(filtered)
    row = torch.randn(1, 30, generator=g)
    n = 20000
    draws = O.sample_next_token(row.expand(n, -1), 0.8, 8, 0.9, torch.rand(n, generator=g))
    probs = torch.softmax(O.sample_filter(row, 0.8, 8, 0.9), -1)[0]
    freq = torch.bincount(draws, minlength=30).double() / n
    assert float(freq[probs == 0].sum()) == 0.0 and float((freq - probs).abs().max()) < 0.02


def test_static_routing_mode_matches_reference():
    """HydraModel(static_routing_mode=True) in eval: dense compute, MoD mixes mlp(u) with u by the router probability,
    MoR weights every recursion's state by soft depth weights.  Logits, block outputs, router logits, and the
    fixed-depth variant (adaptive=False: MoD mixing only) against the reference's run."""
    fx, cfg, w = G.model_fixture("model_static.npz")
    assert cfg.static_routing
    ids = torch.from_numpy(fx["ids"])
    taps = O.RoutingTaps()
    close(O.model_forward(ids, w, cfg, taps=taps), fx["logits"], 5e-6)
    for i in range(cfg.n_mor_blocks):
        close(taps.block_out[i], fx[f"block_out:{i}"], 5e-6)
        close(torch.tanh(taps.router_logits[i] / 2.0) * 3.0, fx[f"router_logits:{i}"], 5e-6)
    assert all(v == ids.numel() for v in taps.mlp_rows.values())
    assert not any(k.startswith("mod_idx") for k in fx)          # nothing is selected in this mode
    cfg.adaptive = False
    close(O.model_forward(ids, w, cfg), fx["logits_fixed"], 5e-6)
    # the mode matters: hard routing on the same weights gives other logits
    cfg.adaptive, cfg.static_routing = True, False
    assert float((O.model_forward(ids, w, cfg) - torch.from_numpy(fx["logits"])).abs().max()) > 1e-2


def test_eval_loss_is_cross_entropy_of_the_forward():
    """eval_checkpoint.py:168-193: F.cross_entropy(model(tokens[:, :-1]), tokens[:, 1:]), summed, divided by the count."""
    fx, cfg, w = G.model_fixture("model_hd32.npz")
    ids = torch.from_numpy(fx["ids"]).clamp(0, cfg.vocab_size - 1)[:, :40]
    logits = O.model_forward(ids[:, :-1], w, cfg)
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, cfg.vocab_size), ids[:, 1:].reshape(-1), reduction="sum")
    assert float(O.eval_loss(ids, w, cfg, reduction="sum")) == pytest.approx(float(want), rel=1e-6)
    assert float(O.eval_loss(ids, w, cfg)) == pytest.approx(float(want) / ids[:, 1:].numel(), rel=1e-6)
    # an untrained model scores near the uniform loss
    assert abs(float(O.eval_loss(ids, w, cfg)) - float(torch.log(torch.tensor(float(cfg.vocab_size))))) < 1.5


def test_mor_rampup_blend_matches_reference():
    """MoR curriculum in the middle of its ramp (blocks.py:645-657, 731-745): every block returns
    0.4 * adaptive + 0.6 * fixed-depth.  Logits, block outputs and the adaptive pass's depths against the reference."""
    fx, cfg, w = G.model_fixture("model_rampup.npz")
    assert cfg.mor_rampup_scale == pytest.approx(0.4)
    ids = torch.from_numpy(fx["ids"])
    taps = O.RoutingTaps()
    close(O.model_forward(ids, w, cfg, taps=taps), fx["logits"], 5e-6)
    for i in range(cfg.n_mor_blocks):
        close(taps.block_out[i], fx[f"block_out:{i}"], 5e-6)
        assert np.array_equal(taps.depths[i].numpy().astype(np.int32), fx[f"depths:{i}"])
    # the end points of the ramp are the two plain paths
    import dataclasses
    full = O.model_forward(ids, w, dataclasses.replace(cfg, mor_rampup_scale=1.0))
    fixed = O.model_forward(ids, w, dataclasses.replace(cfg, adaptive=False, mor_rampup_scale=1.0))
    close(O.model_forward(ids, w, dataclasses.replace(cfg, mor_rampup_scale=0.0)), fixed.numpy(), 1e-6)
    close(fixed, fx["logits_fixed"], 5e-6)
    assert float((full - torch.from_numpy(fx["logits"])).abs().max()) > 1e-3


def reference_kwargs(fx):
    import json
    return json.loads(bytes(fx["reference_kwargs"]).decode())


def test_freshly_constructed_model_runs_every_token_through_the_mlp():
    """A HydraModel right after construction (no set_global_step): MoD is still in its warm-up (blocks.py:140,162-186),
    i.e. capacity 1.0 whatever capacity it was built with - which is what from_reference reads off such an instance."""
    fx, cfg, w = G.model_fixture("model_fresh.npz")
    kw = reference_kwargs(fx)
    assert cfg.mod_capacity == 0.5 and kw["mod_capacity"] == 1.0 and kw["mor_rampup_scale"] == 1.0
    ids = torch.from_numpy(fx["ids"])
    cfg.mod_capacity = kw["mod_capacity"]
    close(O.model_forward(ids, w, cfg), fx["logits"], 5e-6)
    cfg.mod_capacity = 0.5
    assert float((O.model_forward(ids, w, cfg) - torch.from_numpy(fx["logits"])).abs().max()) > 1e-3
