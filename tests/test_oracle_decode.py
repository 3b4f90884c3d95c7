"""The cached-decode restatement of the oracle against the full re-forward (the reference's own generation semantics):
with MoD capacity 1.0 they are the same computation and must agree to fp32 rounding; with capacity 0.75 cached decode
is an approximation whose greedy tokens are compared step by step."""
import torch

from oracle import hydra_oracle as O
from tests import golden_io as G


def test_cached_decode_equals_reforward_at_full_capacity():
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    cfg.mod_capacity = 1.0
    prompt = torch.from_numpy(fx["ids"])[:, :9].clamp(0, cfg.vocab_size - 1)
    n = 7
    seq_c, logits_c = O.cached_generate(prompt, w, cfg, n, return_logits=True)
    seq_r = prompt.clone()
    for step in range(n):
        full = O.model_forward(seq_r, w, cfg)[:, -1]
        err = float((full - logits_c[:, step]).abs().max())
        assert err < 2e-4, f"step {step}: cached vs re-forward logits differ by {err:.2e}"
        seq_r = torch.cat([seq_r, full.argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(seq_c, seq_r)


def test_cached_decode_short_prompt_and_fixed_depth():
    """Prompt shorter than the conv halo (zero-filled history) and the fixed-depth (non-adaptive) path."""
    fx, cfg, w = G.model_fixture("model_hd32.npz")
    cfg.mod_capacity = 1.0
    for adaptive in (True, False):
        cfg.adaptive = adaptive
        prompt = torch.from_numpy(fx["ids"])[:, 2:4].clamp(0, cfg.vocab_size - 1)     # 2 tokens
        seq_c, logits_c = O.cached_generate(prompt, w, cfg, 5, return_logits=True)
        seq_r = prompt.clone()
        for step in range(5):
            full = O.model_forward(seq_r, w, cfg)[:, -1]
            assert float((full - logits_c[:, step]).abs().max()) < 2e-4
            seq_r = torch.cat([seq_r, full.argmax(-1, keepdim=True)], dim=1)
        assert torch.equal(seq_c, seq_r)


def test_cached_decode_with_mod_is_a_close_approximation():
    fx, cfg, w = G.model_fixture("model_hd16.npz")          # capacity 0.75
    prompt = torch.from_numpy(fx["ids"])[:, :24].clamp(0, cfg.vocab_size - 1)
    n = 8
    seq_c, logits_c = O.cached_generate(prompt, w, cfg, n, return_logits=True)
    ref = O.model_forward(prompt, w, cfg)[:, -1]
    assert float((ref - logits_c[:, 0]).abs().max()) < 2e-4     # the prefill itself is exact
    seq_r = O.greedy_generate(prompt, w, cfg, n)
    agree = float((seq_c[:, 24:] == seq_r[:, 24:]).float().mean())
    assert agree >= 0.5, f"greedy-token agreement {agree:.2f}"


def test_cached_decode_with_an_untied_output_projection():
    """tie_weights=False: the cached path projects with output.weight, as the forward does."""
    fx, cfg, w = G.model_fixture("model_untied.npz")
    cfg.mod_capacity = 1.0
    prompt = torch.from_numpy(fx["ids"])[:, :11].clamp(0, cfg.vocab_size - 1)
    seq_c, logits_c = O.cached_generate(prompt, w, cfg, 4, return_logits=True)
    seq_r = prompt.clone()
    for step in range(4):
        full = O.model_forward(seq_r, w, cfg)[:, -1]
        assert float((full - logits_c[:, step]).abs().max()) < 2e-4
        seq_r = torch.cat([seq_r, full.argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(seq_c, seq_r)


def test_cached_decode_in_static_routing_mode_equals_the_reforward():
    """static_routing_mode has no top-k over the sequence: every operation is causal, so the cached step must reproduce
    the re-forward of the longer sequence for any MoD capacity (adaptive and fixed-depth blocks)."""
    fx, cfg, w = G.model_fixture("model_static.npz")
    assert cfg.static_routing and cfg.mod_capacity < 1.0
    for adaptive in (True, False):
        cfg.adaptive = adaptive
        prompt = torch.from_numpy(fx["ids"])[:, :13].clamp(0, cfg.vocab_size - 1)
        seq_c, logits_c = O.cached_generate(prompt, w, cfg, 5, return_logits=True)
        seq_r = prompt.clone()
        for step in range(5):
            full = O.model_forward(seq_r, w, cfg)[:, -1]
            assert float((full - logits_c[:, step]).abs().max()) < 2e-4
            seq_r = torch.cat([seq_r, full.argmax(-1, keepdim=True)], dim=1)
        assert torch.equal(seq_c, seq_r)


def test_cached_decode_before_the_mor_ramp_is_the_fixed_depth_path():
    """MoR curriculum scale 0 (HydraMoRBlock.forward, blocks.py:645-649): the block is the fixed-depth path, in the
    cached prefill and step too - same logits as a model built without the depth router; inside the ramp the cached step
    is undefined and refuses."""
    import dataclasses
    import pytest
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    before = dataclasses.replace(cfg, mor_rampup_scale=0.0)
    fixed = dataclasses.replace(cfg, adaptive=False)
    prompt = torch.from_numpy(fx["ids"])[:, :9].clamp(0, cfg.vocab_size - 1)
    seq_a, lg_a = O.cached_generate(prompt, w, before, 5, return_logits=True)
    seq_b, lg_b = O.cached_generate(prompt, w, fixed, 5, return_logits=True)
    assert torch.equal(seq_a, seq_b) and torch.equal(lg_a, lg_b)
    _, lg_c = O.cached_generate(prompt, w, cfg, 5, return_logits=True)
    assert float((lg_c - lg_a).abs().max()) > 1e-3                 # the depth router does change the result
    _, cache = O.cached_prefill(prompt, w, dataclasses.replace(cfg, mor_rampup_scale=0.5))
    with pytest.raises(ValueError):
        O.cached_decode_step(prompt[:, -1], w, dataclasses.replace(cfg, mor_rampup_scale=0.5), cache)
