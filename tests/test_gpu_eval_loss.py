"""hb200_cross_entropy_rows and HydraB200Model.eval_loss: the next-token loss of the reference's evaluation helper
(diagnostics/eval_checkpoint.py:168-193).  Tolerances: the kernel against F.cross_entropy on the same bf16 logits is
fp32 rounding (1e-4); the model's loss against the reference's fp32 logits carries the bf16 rounding of the logits
(per token up to a few 1e-2, mean within 1e-2)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import hydra_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu


def test_kernel_against_torch_on_the_same_logits():
    from hydra_b200.sampling import cross_entropy_rows
    g = torch.Generator().manual_seed(0)
    for (N, V, ld) in ((5, 1000, 1000), (33, 50257, 50264), (7, 777, 790), (1, 16, 16)):
        buf = (torch.randn(N, ld, generator=g) * 4).to(torch.bfloat16)
        buf[:, V:] = 50.0                                           # padding columns must not count
        tgt = torch.randint(0, V, (N,), generator=g)
        if N > 2:
            tgt[1] = -100
        got = cross_entropy_rows(buf.cuda(), tgt.cuda(), vocab=V).cpu()
        want = F.cross_entropy(buf[:, :V].float(), tgt, reduction="none", ignore_index=-100)
        assert float((got - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max())), (N, V)
        if N > 2:
            assert float(got[1]) == 0.0
    # a row view that does not start on a 16-byte boundary
    wide = (torch.randn(4, 300, generator=g) * 3).to(torch.bfloat16)
    view = wide.cuda()[:, 3:]
    tgt = torch.randint(0, 297, (4,), generator=g)
    got = cross_entropy_rows(view, tgt.cuda()).cpu()
    assert float((got - F.cross_entropy(wide[:, 3:].float(), tgt, reduction="none")).abs().max()) < 1e-4
    # extreme rows: one dominant logit, all equal, -inf entries
    x = torch.full((3, 64), -5.0)
    x[0, 7] = 80.0
    x[1] = 2.5
    x[2, :60] = float("-inf")
    t = torch.tensor([7, 3, 61])
    got = cross_entropy_rows(x.to(torch.bfloat16).cuda(), t.cuda()).cpu()
    assert float((got - F.cross_entropy(x.to(torch.bfloat16).float(), t, reduction="none")).abs().max()) < 1e-4
    with pytest.raises(ValueError):
        cross_entropy_rows(x.to(torch.bfloat16).cuda(), torch.tensor([0, 1, 64]).cuda())


@pytest.mark.parametrize("name", ["model_hd16.npz", "model_untied.npz"])
def test_model_loss_against_the_reference_logits(name):
    """The model runs on the fixture's ids; every position but the last is scored against the next token.  The same
    quantity from the reference's own fp32 logits pins it."""
    from tests.test_gpu_model import build
    fx, cfg, w = G.model_fixture(name)
    ids = torch.from_numpy(fx["ids"])
    tgt = torch.cat([ids[:, 1:], torch.full((ids.shape[0], 1), -100)], dim=1).clamp(min=-100, max=cfg.vocab_size - 1)
    tgt[tgt < 0] = -100                                              # the fixture holds out-of-range ids on purpose
    m = build(w, cfg)
    nll = m.eval_loss(ids.cuda(), tgt.cuda(), reduction="none").cpu()
    ref_logits = torch.from_numpy(fx["logits"])
    want = F.cross_entropy(ref_logits.reshape(-1, cfg.vocab_size), tgt.reshape(-1), reduction="none",
                           ignore_index=-100).view(tgt.shape)
    n = int((tgt != -100).sum())
    mean_got, mean_want = float(nll.sum()) / n, float(want.sum()) / n
    print(f"{name}: mean loss {mean_got:.4f} vs reference {mean_want:.4f}; worst token {float((nll - want).abs().max()):.3e}")
    assert abs(mean_got - mean_want) < 1e-2 and float((nll - want).abs().max()) < 0.15
    assert float(m.eval_loss(ids.cuda(), tgt.cuda(), reduction="sum")) == pytest.approx(float(nll.sum()), rel=1e-5)
    assert float(m.eval_loss(ids.cuda(), tgt.cuda())) == pytest.approx(mean_got, rel=1e-5)


def test_default_targets_are_the_next_tokens():
    from tests.test_gpu_model import build
    fx, cfg, w = G.model_fixture("model_hd32.npz")
    cfg.mod_capacity = 1.0                                           # no top-k: the oracle run is comparable token by token
    ids = torch.from_numpy(fx["ids"]).clamp(0, cfg.vocab_size - 1)
    m = build(w, cfg)
    got = m.eval_loss(ids.cuda(), reduction="none").cpu()
    want = O.eval_loss(ids, w, cfg, reduction="none")
    assert got.shape == (ids.shape[0], ids.shape[1] - 1)
    # a depth decision that flips on bf16 noise moves single tokens; the mean stays close
    assert abs(float(got.mean()) - float(want.mean())) < 2e-2
    assert float((got - want).abs().median()) < 2e-2
    with pytest.raises(ValueError):
        m.eval_loss(ids[:, :1].cuda())
