"""Cached decode on the GPU (hb200_model_prefill_cached / hb200_model_decode_step) against the oracle's cached
decode driven with the GPU's own token choices (so one differing choice cannot make the rest incomparable), against
the GPU's own longer prefill (cache contents), and graph replay against direct launches.

Tolerances: logits are bf16 results of a bf16 pipeline compared with an fp32 oracle; the model fixtures record the
reference's own bf16-vs-fp32 error on the same weights (rel. L2 about 5e-3), and a per-step bound of 3e-2 / overall
bound of 1.5e-2 is used here (a single sequence's routing decision flipping at a threshold moves one row's logits
by more than rounding does)."""
import pytest
import torch

from oracle import hydra_oracle as O
from tests import golden_io as G
from tests.gpu_util import rel_l2

pytestmark = pytest.mark.gpu


def build(w, cfg, **kw):
    from hydra_b200.model import HydraB200Model
    args = dict(n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, max_seq_len=cfg.max_seq_len,
                mod_capacity=cfg.mod_capacity, mor_min_depth=cfg.mor_min_depth, adaptive=cfg.adaptive)
    args.update(kw)
    return HydraB200Model(w, **args)


def teacher_forced_oracle(prompt, tokens, w, cfg):
    """Oracle cached decode consuming `tokens` [B, n] (the GPU's choices): logits [B, n, V] each choice is made from."""
    logits, cache = O.cached_prefill(prompt, w, cfg)
    out = [logits[:, -1]]
    for i in range(tokens.shape[1] - 1):
        out.append(O.cached_decode_step(tokens[:, i], w, cfg, cache))
    return torch.stack(out, dim=1)


def check_against_oracle(m, w, cfg, prompt, n_new, label, use_graph=True, step_tol=3e-2, all_tol=1.5e-2):
    P = prompt.shape[1]
    seq, lg = m.generate_cached(prompt.cuda(), n_new, use_graph=use_graph, return_logits=True)
    seq, lg = seq.cpu(), lg.float().cpu()
    assert seq.shape == (prompt.shape[0], P + n_new) and torch.equal(seq[:, :P], prompt)
    assert torch.isfinite(lg).all()
    assert torch.equal(seq[:, P:], lg.argmax(-1)), "tokens are the argmax of the returned logits"
    ref = teacher_forced_oracle(prompt, seq[:, P:], w, cfg)
    per_step = [rel_l2(lg[:, i], ref[:, i]) for i in range(n_new)]
    print(f"{label}: per-step rel_l2 {['%.2e' % e for e in per_step]} overall {rel_l2(lg, ref):.2e}")
    assert max(per_step) <= step_tol, f"{label}: worst step rel_l2 {max(per_step):.3e}"
    assert rel_l2(lg, ref) <= all_tol
    # greedy choices agree with the oracle's wherever its best-vs-second gap exceeds the bf16 noise on a logit
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 0.06
    assert torch.equal(seq[:, P:][clear], ref.argmax(-1)[clear])
    return seq, lg


@pytest.mark.parametrize("name,cap,P,n_new", [("model_hd16.npz", 1.0, 20, 10), ("model_hd16.npz", 0.75, 33, 12),
                                               ("model_hd32.npz", 0.5, 17, 9), ("model_hd32.npz", 1.0, 64, 6)])
def test_cached_decode_against_teacher_forced_oracle(name, cap, P, n_new):
    fx, cfg, w = G.model_fixture(name)
    cfg.mod_capacity = cap
    prompt = torch.from_numpy(fx["ids"])[:, :P].clamp(0, cfg.vocab_size - 1)
    m = build(w, cfg)
    check_against_oracle(m, w, cfg, prompt, n_new, f"{name} cap {cap}")


def test_short_prompt_fixed_depth_and_single_sequence():
    """Prompts shorter than the conv halo (zero history), the non-adaptive path, batch 1."""
    fx, cfg, w = G.model_fixture("model_hd32.npz")
    for adaptive, P, rows in ((True, 1, 2), (False, 2, 2), (True, 3, 1)):
        cfg.adaptive = adaptive
        prompt = torch.from_numpy(fx["ids"])[:rows, 5:5 + P].clamp(0, cfg.vocab_size - 1)
        check_against_oracle(build(w, cfg), w, cfg, prompt, 7, f"P={P} adaptive={adaptive} B={rows}")


def test_before_the_mor_ramp_decode_runs_the_fixed_depth_path():
    """MoR curriculum scale 0 (what a reference model reports before MoR is enabled): prefill and cached decode are the
    fixed-depth path, bit for bit the model built without the depth router, and match the oracle in that state."""
    import dataclasses
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    prompt = torch.from_numpy(fx["ids"])[:, :21].clamp(0, cfg.vocab_size - 1)
    before = dataclasses.replace(cfg, mor_rampup_scale=0.0)
    m = build(w, cfg, mor_rampup_scale=0.0)
    seq, lg = check_against_oracle(m, w, before, prompt, 8, "ramp-up scale 0")
    cfg.adaptive = False
    seq_f, lg_f = build(w, cfg).generate_cached(prompt.cuda(), 8, return_logits=True)
    assert torch.equal(seq, seq_f.cpu()) and torch.equal(lg, lg_f.float().cpu())


def test_graph_replay_equals_direct_launches():
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    prompt = torch.from_numpy(fx["ids"])[:, :25].clamp(0, cfg.vocab_size - 1).cuda()
    m = build(w, cfg)
    s0, l0 = m.generate_cached(prompt, 9, use_graph=False, return_logits=True)
    s1, l1 = m.generate_cached(prompt, 9, use_graph=True, return_logits=True)
    assert torch.equal(s0, s1) and torch.equal(l0, l1)
    assert torch.equal(m.generate(prompt, 9, mode="cached"), s1)


def test_caches_after_decode_match_a_longer_prefill():
    """Prefill(P) + n steps leaves the same keys / values / conv halo / MoD scores as a prefill of the P + n tokens
    (capacity 1.0: every operation of the forward is causal, so only bf16 rounding differs)."""
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    cfg.mod_capacity = 1.0
    P, n = 30, 11
    m = build(w, cfg)
    prompt = torch.from_numpy(fx["ids"])[:, :P].clamp(0, cfg.vocab_size - 1).cuda()
    a = m.new_decode_session(prompt.shape[0], P + n + 1)
    a.prefill(prompt)
    for _ in range(n):
        a.step(use_graph=True)
    m.check_device_errors()
    assert a.pos == P + n and int(a.pos_dev.item()) == P + n
    full = a.history[:, :P + n].clone()
    b = m.new_decode_session(prompt.shape[0], P + n + 1)
    b.prefill(full)
    T = P + n
    assert rel_l2(a.kcache[:, :, :, :T].float().cpu(), b.kcache[:, :, :, :T].float().cpu()) < 1e-2
    assert rel_l2(a.vcache[:, :, :, :T].float().cpu(), b.vcache[:, :, :, :T].float().cpu()) < 1e-2
    assert rel_l2(a.halo.float().cpu(), b.halo.float().cpu()) < 1e-2
    assert rel_l2(a.vshift.float().cpu(), b.vshift.float().cpu()) < 1e-2
    mod_blocks = [i for i in range(cfg.n_mor_blocks) if cfg.block_has_mod(i)]
    assert mod_blocks
    sa, sb = a.scores[mod_blocks][..., :T].cpu(), b.scores[mod_blocks][..., :T].cpu()
    assert rel_l2(sa, sb) < 2e-2
    # block 0's cache depends only on the embeddings: values are copies of the same projection (bit-equal), keys
    # differ only by the summation order of the two conv implementations
    assert torch.equal(a.vcache[0, :, :, :T], b.vcache[0, :, :, :T])
    assert rel_l2(a.kcache[0, :, :, :T].float().cpu(), b.kcache[0, :, :, :T].float().cpu()) < 3e-3
    # both sessions then choose the same next token where the margin is clear
    la, lb = a.last_logits.float().cpu()[:, :cfg.vocab_size], b.last_logits.float().cpu()[:, :cfg.vocab_size]
    assert rel_l2(la, lb) < 2e-2


def test_1p5b_block_shape_decode():
    """dim 2048, 32 query / 4 KV heads of 16 (latent 512, eight query heads per KV head), 3 blocks x 2 recursions."""
    cfg = O.HydraConfig(vocab_size=512, dim=2048, n_mor_blocks=3, recursions_per_block=2, n_heads=32, n_kv_heads=4,
                        max_seq_len=160, mod_capacity=0.75)
    w = O.init_params(cfg, seed=3, perturb=True)
    prompt = torch.randint(0, 512, (3, 70), generator=torch.Generator().manual_seed(3))
    check_against_oracle(build(w, cfg), w, cfg, prompt, 8, "1.5B block shape")


def test_equal_head_counts_and_batch_beyond_one_row_tile():
    """n_heads == n_kv_heads takes the other QK-mean branch; 37 sequences exercise ragged row kernels."""
    cfg = O.HydraConfig(vocab_size=640, dim=256, n_mor_blocks=3, recursions_per_block=2, n_heads=4, n_kv_heads=4,
                        max_seq_len=64, mod_capacity=0.75)
    w = O.init_params(cfg, seed=11, perturb=True)
    prompt = torch.randint(0, 640, (37, 12), generator=torch.Generator().manual_seed(5))
    check_against_oracle(build(w, cfg), w, cfg, prompt, 5, "MHA, B=37")


def test_odd_kv_head_count_value_shift_split_inside_a_head():
    """12 query / 3 KV heads of 16: the value-shift boundary (kv_dim / 2 = 24 channels) falls inside the second KV head."""
    cfg = O.HydraConfig(vocab_size=500, dim=768, n_mor_blocks=3, recursions_per_block=2, n_heads=12, n_kv_heads=3,
                        max_seq_len=96, mod_capacity=0.75)
    w = O.init_params(cfg, seed=13, perturb=True)
    prompt = torch.randint(0, 500, (2, 41), generator=torch.Generator().manual_seed(6))
    check_against_oracle(build(w, cfg), w, cfg, prompt, 6, "12q/3kv")


@pytest.mark.parametrize("B", [130, 520])
def test_batches_beyond_one_row_tile(B):
    """130 sequences: the decode contractions run as two 128-row tiles of the weight-streaming kernel; 520: beyond its
    four tiles, they fall back to the general GEMM kernel."""
    cfg = O.HydraConfig(vocab_size=320, dim=256, n_mor_blocks=3, recursions_per_block=2, n_heads=4, n_kv_heads=2,
                        max_seq_len=48, mod_capacity=0.75)
    w = O.init_params(cfg, seed=17, perturb=True)
    prompt = torch.randint(0, 320, (B, 9), generator=torch.Generator().manual_seed(8))
    check_against_oracle(build(w, cfg), w, cfg, prompt, 4, f"B={B}")


def test_static_routing_mode_decodes_exactly():
    """static_routing_mode has no top-k over the sequence, so the cached step computes what the re-forward computes for
    the newest position at ANY MoD capacity: against the oracle's cached decode (teacher-forced), against the GPU's own
    re-forward of the generated sequence, adaptive and fixed-depth."""
    fx, cfg, w = G.model_fixture("model_static.npz")
    assert cfg.static_routing and cfg.mod_capacity < 1.0
    for adaptive in (True, False):
        cfg.adaptive = adaptive
        m = build(w, cfg, static_routing_mode=True)
        prompt = torch.from_numpy(fx["ids"])[:, :21].clamp(0, cfg.vocab_size - 1)
        seq, lg = check_against_oracle(m, w, cfg, prompt, 8, f"static routing, adaptive={adaptive}")
        full = m(seq[:, :-1].cuda()).float().cpu()[:, 20:]          # logits each generated token was chosen from
        assert rel_l2(lg, full) < 1e-2
        assert torch.equal(m.generate(prompt.cuda(), 8, mode="cached").cpu(), seq)


def test_session_errors():
    fx, cfg, w = G.model_fixture("model_hd16.npz")
    m = build(w, cfg)
    prompt = torch.from_numpy(fx["ids"])[:, :8].clamp(0, cfg.vocab_size - 1).cuda()
    s = m.new_decode_session(2, 9)
    s.prefill(prompt)
    s.step()
    with pytest.raises(RuntimeError):
        s.step()                                   # cache full
    with pytest.raises(ValueError):
        m.new_decode_session(2, cfg.max_seq_len + 1)
    with pytest.raises(ValueError):
        m.generate(prompt, 2, mode="nope")
    with pytest.raises(RuntimeError):
        m.generate_cached(prompt.cpu(), 2)


def test_cache_longer_than_the_routing_kernels_register_slice():
    """4100 cached positions: the MoD rank of the newest token counts the first 4096 cached scores from registers and the
    rest on demand."""
    cfg = O.HydraConfig(vocab_size=300, dim=256, n_mor_blocks=3, recursions_per_block=2, n_heads=4, n_kv_heads=2,
                        max_seq_len=4120, mod_capacity=0.75, hidden_dim=256)
    w = O.init_params(cfg, seed=19, perturb=True)
    prompt = torch.randint(0, 300, (2, 4100), generator=torch.Generator().manual_seed(9))
    check_against_oracle(build(w, cfg), w, cfg, prompt, 4, "P=4100")
