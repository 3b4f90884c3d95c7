"""hb200_sample_rows (temperature / top-k / top-p sampling on the device) against the oracle's restatement of the
reference's sampler and against the distributions the reference itself produced (tests/golden/sampler.npz).

The draw is a deterministic function of (logits, uniform): the first token, in descending-logit order with equal logits
by ascending id, whose cumulative probability exceeds the uniform number.  The oracle accumulates probabilities in
float64, the kernel in 64-bit fixed point from fp32 exponentials, so a uniform number closer than 2e-5 to a step of the
CDF may land on the neighbouring token; everything else must agree exactly."""
import numpy as np
import pytest
import torch

from oracle import hydra_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
TOL = 2e-5


def gpu_sample(logits_bf16, temperature, top_k, top_p, u):
    from hydra_b200.sampling import sample_rows
    return sample_rows(logits_bf16.cuda(), temperature, top_k, top_p, uniforms=u.cuda()).cpu()


def check_rows(logits, temperature, top_k, top_p, u, label):
    """logits fp32 [B, V] holding bf16-representable values; u fp32 [B]."""
    got = gpu_sample(logits.to(torch.bfloat16), temperature, top_k, top_p, u)
    want = O.sample_next_token(logits, temperature, top_k, top_p, u)
    x = O.sample_filter(logits, temperature, top_k, top_p)
    sx, si = torch.sort(x, descending=True, stable=True)
    cdf = torch.cumsum(torch.softmax(sx.double(), dim=-1), dim=-1)
    rank = torch.empty_like(si).scatter_(1, si, torch.arange(si.shape[1]).expand_as(si))
    exact = int((got == want).sum())
    for b in torch.nonzero(got != want)[:, 0].tolist():
        j = int(rank[b, got[b]])
        assert torch.isfinite(x[b, got[b]]) or abs(float(cdf[b, j - 1]) - top_p) < TOL, f"{label} row {b}: removed token drawn"
        lo = float(cdf[b, j - 1]) if j > 0 else 0.0
        # the kept set may differ by the borderline token, which rescales the CDF by at most its probability
        assert lo - 10 * TOL <= float(u[b]) <= float(cdf[b, j]) + 10 * TOL or not torch.isfinite(x[b, got[b]]), \
            f"{label} row {b}: u {float(u[b]):.6f} outside [{lo:.6f}, {float(cdf[b, j]):.6f}]"
    frac = exact / got.numel()
    print(f"{label}: {exact}/{got.numel()} draws equal to the oracle's")
    assert frac >= 0.995, f"{label}: only {frac:.4f} of the draws equal the oracle's"
    return got


def test_against_the_reference_distributions():
    """Every fixture row (logits and the probabilities the reference's generate_text handed to torch.multinomial):
    256 uniform numbers per row; draws equal the oracle's, and every drawn token carries the probability the reference
    gave to a token of that logit value (its choice among equal logits at the nucleus edge is not pinned)."""
    fx = G.load("sampler.npz")
    lg, pr, st = torch.from_numpy(fx["logits"]), torch.from_numpy(fx["probs"]), fx["settings"]
    g = torch.Generator().manual_seed(0)
    for r in range(lg.shape[0]):
        t, k, p = float(st[r, 0]), int(st[r, 1]), float(st[r, 2])
        u = torch.rand(256, generator=g)
        u[0], u[1] = 0.0, 0.99999994
        rows = lg[r:r + 1].expand(256, -1).contiguous()
        got = check_rows(rows, t, k, p, u, f"fixture row {r} (T={t}, k={k}, p={p})")
        ref_values = set(lg[r][pr[r] > 0].tolist())
        assert set(lg[r][got].tolist()) <= ref_values, f"row {r}: a token outside the reference's kept values was drawn"
        assert int(got[0]) == int(O.sample_next_token(rows[:1], t, k, p, u[:1])[0])


def test_full_vocabulary_rows_with_padding_columns():
    """50257 columns in rows 50264 apart (the model's logits buffer): top-k only, nucleus only, both, neither."""
    V, ld, B = 50257, 50264, 96
    g = torch.Generator().manual_seed(1)
    buf = (torch.randn(B, ld, generator=g) * 2.5).to(torch.bfloat16)
    buf[:, V:] = 100.0                                     # padding must never be drawn
    u = torch.rand(B, generator=g)
    from hydra_b200.sampling import sample_rows
    for (t, k, p) in ((0.8, 50, 0.9), (1.0, 0, 0.9), (0.7, 40, 1.0), (1.0, 0, 1.0), (1.5, 5000, 0.97)):
        got = sample_rows(buf.cuda(), t, k, p, uniforms=u.cuda(), vocab=V).cpu()
        assert int(got.max()) < V and int(got.min()) >= 0
        want = O.sample_next_token(buf[:, :V].float(), t, k, p, u)
        agree = float((got == want).float().mean())
        print(f"V=50257 T={t} k={k} p={p}: agreement {agree:.4f}")
        assert agree >= 0.97
        x = O.sample_filter(buf[:, :V].float(), t, k, p)
        bad = ~torch.isfinite(x.gather(1, got[:, None])[:, 0]) & (got != want)
        assert int(bad.sum()) <= 1                         # at most a nucleus-edge token


def test_greedy_limits_ties_and_unaligned_rows():
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(33, 1001, generator=g) * 3).to(torch.bfloat16)
    x[3, 10] = x[3, 500] = x[3].max() + 1                  # equal maxima: lowest id wins
    x[4, 7] = float("nan")                                 # NaN never wins
    u = torch.rand(33, generator=g)
    ref = O.sample_next_token(torch.nan_to_num(x.float(), nan=-1e30), 0.0, 0, 1.0, u)
    from hydra_b200.sampling import sample_rows
    for (t, k) in ((0.0, 0), (-1.0, 50), (0.8, 1)):
        got = sample_rows(x.cuda(), t, k, 0.9, uniforms=u.cuda() if t > 0 else None).cpu()
        assert torch.equal(got, ref)
    assert int(got[3]) == 10
    # a tiny temperature and a tiny nucleus both collapse to the argmax
    assert torch.equal(sample_rows(x.cuda(), 1e-4, 0, 1.0, uniforms=u.cuda()).cpu(), ref)
    assert torch.equal(sample_rows(x.cuda(), 1.0, 0, 0.0, uniforms=u.cuda()).cpu()[5:], ref[5:])
    # all logits equal: the draw is uniform over the ids, in id order
    flat = torch.zeros(64, 1000, dtype=torch.bfloat16)
    uu = (torch.arange(64, dtype=torch.float32) + 0.5) / 64
    got = sample_rows(flat.cuda(), 1.0, 0, 1.0, uniforms=uu.cuda()).cpu()
    assert torch.equal(got, (uu.double() * 1000).long())
    # signed zeros are one value (they compare equal): ties among them go by token id, and -0 ties with a +0 k-th value
    z = (torch.randn(64, 257, generator=g) * 2).round() / 2
    z[:, ::5] = -0.0
    z[:, 1::7] = 0.0
    uz = torch.rand(64, generator=g)
    for (t, k, p) in ((1.0, 0, 1.0), (5.0, 100, 0.999), (0.8, 20, 0.9)):
        got = sample_rows(z.to(torch.bfloat16).cuda(), t, k, p, uniforms=uz.cuda()).cpu()
        assert torch.equal(got, O.sample_next_token(z, t, k, p, uz)), f"signed zeros, T={t} k={k} p={p}"
    # a row view that starts at an odd element (no 16-byte alignment) and one row only
    wide = (torch.randn(5, 777, generator=g) * 2).to(torch.bfloat16).cuda()
    view = wide[:, 3:]
    got = sample_rows(view, 0.9, 30, 0.8, uniforms=u[:5].cuda()).cpu()
    assert torch.equal(got, O.sample_next_token(view.float().cpu(), 0.9, 30, 0.8, u[:5]))
    got1 = sample_rows(view[2:3], 0.9, 30, 0.8, uniforms=u[2:3].cuda()).cpu()
    assert int(got1[0]) == int(got[2])


def test_draws_follow_the_distribution():
    """One row, 20000 uniform numbers: empirical frequencies of the kept tokens against their probabilities."""
    g = torch.Generator().manual_seed(3)
    row = (torch.randn(1, 4096, generator=g) * 2).to(torch.bfloat16)
    n = 20000
    u = torch.rand(n, generator=g)
    from hydra_b200.sampling import sample_rows
    got = sample_rows(row.expand(n, -1).contiguous().cuda(), 1.0, 20, 0.95, uniforms=u.cuda()).cpu()
    probs = torch.softmax(O.sample_filter(row.float(), 1.0, 20, 0.95), dim=-1)[0]
    freq = torch.bincount(got, minlength=4096).double() / n
    assert float(freq[probs == 0].sum()) == 0.0
    sd = torch.sqrt(probs.double() * (1 - probs.double()) / n)
    assert float(((freq - probs.double()).abs() / (sd + 1e-4)).max()) < 5.0


def test_errors():
    from hydra_b200 import _lib as L
    from hydra_b200.sampling import sample_rows
    x = torch.zeros(2, 70000, dtype=torch.bfloat16).cuda()
    with pytest.raises(L.Hb200Error):
        sample_rows(x, 1.0, 0, 1.0)                        # more than 65535 columns
    assert int(sample_rows(x, 1.0, 0, 1.0, vocab=65535).max()) < 65535
    with pytest.raises(RuntimeError):
        sample_rows(x.cpu(), 1.0, 0, 1.0)
    with pytest.raises(ValueError):
        sample_rows(x.float(), 1.0, 0, 1.0)
    out = torch.empty(2, dtype=torch.int64, device="cuda")
    st = L.lib().hb200_sample_rows(x.data_ptr(), 2, 100, 70000, 0.8, 50, 0.9, None, out.data_ptr(), None)
    assert st == -1                                        # HB200_ERR_INVALID: sampling without uniforms


def test_sampled_generation_in_both_modes():
    """generate(temperature=...) - reproducible from the generator's seed, different seeds differ, every drawn token
    has non-zero probability under the filter applied to the logits it was drawn from, and (cached mode) the logits
    still match the oracle's cached decode fed with the drawn tokens."""
    from tests.test_gpu_decode import build, teacher_forced_oracle
    from tests.gpu_util import rel_l2
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    m = build(w, cfg)
    prompt = torch.from_numpy(fx["ids"])[:, :16].clamp(0, cfg.vocab_size - 1)
    n_new = 10

    def run(seed, mode):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        return m.generate(prompt.cuda(), n_new, mode=mode, temperature=1.0, top_k=40, top_p=0.95, generator=gen).cpu()

    for mode in ("reforward", "cached"):
        a, b, c = run(5, mode), run(5, mode), run(6, mode)
        assert torch.equal(a, b) and not torch.equal(a, c), mode
        assert torch.equal(a[:, :16], prompt) and int(a.max()) < cfg.vocab_size
        assert not torch.equal(a, m.generate(prompt.cuda(), n_new, mode=mode).cpu())      # not the greedy sequence
    # end-of-text handling: what follows a row's first end-of-text token is overwritten with it, in both modes
    greedy = m.generate(prompt.cuda(), n_new, mode="cached").cpu()
    eos = int(greedy[0, 16 + 3])
    for mode in ("reforward", "cached"):
        padded = m.generate(prompt.cuda(), n_new, mode=mode, eos_token_id=eos).cpu()
        first = int((padded[0, 16:] == eos).nonzero()[0])
        assert first <= 3 and bool((padded[0, 16 + first:] == eos).all()) and torch.equal(padded[:, :16], prompt)
    gen = torch.Generator(device="cuda").manual_seed(9)
    seq, lg = m.generate_cached(prompt.cuda(), n_new, return_logits=True, temperature=1.0, top_k=40, top_p=0.95,
                                generator=gen)
    m.check_device_errors()
    seq, lg = seq.cpu(), lg.float().cpu()
    for i in range(n_new):
        x = O.sample_filter(lg[:, i], 1.0, 40, 0.95)
        assert torch.isfinite(x.gather(1, seq[:, 16 + i][:, None])).all(), f"step {i}: a removed token was drawn"
    ref = teacher_forced_oracle(prompt, seq[:, 16:], w, cfg)
    assert rel_l2(lg, ref) <= 1.5e-2
