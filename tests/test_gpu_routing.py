"""MoD selection and MoR depth assignment on the GPU: index lists must be identical to the oracle's
(torch.topk + sort on the same fp32 scores)."""
import numpy as np
import pytest
import torch

from oracle import hydra_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from hydra_b200 import _lib
    return _lib


def select(L, scores, k, depth=None, min_active=0):
    B, Ln = scores.shape
    sc = scores.float().cuda().contiguous()
    idx = torch.full((B, k), -1, dtype=torch.int32, device="cuda")
    rows = count = None
    if depth is not None:
        rows = torch.full((B * Ln,), -1, dtype=torch.int32, device="cuda")
        count = torch.zeros(1, dtype=torch.int32, device="cuda")
        depth = depth.to(torch.int32).cuda().contiguous()
    L.check(L.lib().hb200_mod_topk_select(sc.data_ptr(), B, Ln, k, idx.data_ptr(),
                                          depth.data_ptr() if depth is not None else None, min_active,
                                          rows.data_ptr() if rows is not None else None,
                                          count.data_ptr() if count is not None else None,
                                          torch.cuda.current_stream().cuda_stream), "mod_topk_select")
    torch.cuda.synchronize()
    if depth is None:
        return idx.cpu()
    return idx.cpu(), rows.cpu(), int(count.item())


@pytest.mark.parametrize("B,Ln,cap", [(32, 2048, 0.75), (4, 512, 0.75), (3, 2048, 0.5), (2, 8192, 0.75), (5, 1, 0.75),
                                      (2, 7, 0.3), (1, 3000, 1.0), (2, 1000, 0.0001)])
def test_indices_identical_to_oracle(L, B, Ln, cap):
    g = torch.Generator().manual_seed(Ln + B)
    scores = torch.randn(B, Ln, generator=g) * 3
    k = O.mod_k(Ln, cap)
    ref = O.mod_select(scores, cap)
    got = select(L, scores, k)
    assert got.shape == (B, k)
    assert torch.equal(got.long(), ref), "MoD index lists must be bit-identical"


def test_ties_nan_inf_and_signed_zero(L):
    """Tie rule: among scores equal to the k-th largest the lowest positions are taken; the selected set is always
    valid (every strictly larger score is in, exactly k chosen).  NaN ranks above +inf (ATen's order); -0 == +0."""
    s = torch.tensor([[1.0, 2.0, 2.0, 2.0, 0.0, 2.0, 3.0, 2.0]])
    assert select(L, s, 4).tolist() == [[1, 2, 3, 6]]
    s = torch.tensor([[0.5, float("nan"), float("inf"), -float("inf"), 7.0, float("nan")]])
    assert select(L, s, 3).tolist() == [[1, 2, 5]]
    s = torch.tensor([[-0.0, 0.0, -1.0, 0.0, -0.0]])
    assert select(L, s, 2).tolist() == [[0, 1]]
    # heavy ties (bf16-like quantised scores): validity of the set and agreement with torch.topk's VALUES
    g = torch.Generator().manual_seed(9)
    q = (torch.randn(16, 2048, generator=g) * 4).round() / 4
    k = 1536
    got = select(L, q, k).long()
    vals = torch.gather(q, 1, got)
    tv, _ = torch.topk(q, k, dim=-1)
    assert torch.equal(vals.sort(dim=1, descending=True)[0], tv)
    assert (got[:, 1:] > got[:, :-1]).all(), "ascending and unique"


def test_tie_order_beside_torch_topk_on_the_same_device(L, capsys):
    """What CUDA torch.topk does with tie-heavy scores (the reference's bf16 path produces bf16-quantised scores,
    mixture_of_depths.py:187): its choice among equal scores is not specified, so this reports how often it picks the
    same positions as the lowest-index-first rule used here, and asserts only what any valid top-k must satisfy -
    the same multiset of selected VALUES."""
    g = torch.Generator().manual_seed(9)
    q = (torch.randn(32, 2048, generator=g) * 3).to(torch.bfloat16).float()
    k = 1536
    got = select(L, q, k).long()
    tv, ti = torch.topk(q.cuda(), k, dim=-1)
    ti = ti.sort(dim=-1)[0].cpu()
    assert torch.equal(torch.gather(q, 1, got).sort(dim=1, descending=True)[0], tv.cpu())
    rows_equal = int((got == ti).all(dim=1).sum())
    pos_equal = float((got == ti).float().mean())
    kth = tv[:, -1].cpu()
    tied_at_cut = [(int((q[b] == kth[b]).sum()), int(((q[b] == kth[b]) & (torch.zeros(2048, dtype=torch.bool).scatter_(0, ti[b], True))).sum()))
                   for b in range(32)]
    # among the scores equal to the k-th value, does torch keep the lowest positions too?
    lowest_first = 0
    for b in range(32):
        eq = torch.nonzero(q[b] == kth[b]).flatten()
        kept = torch.isin(eq, ti[b])
        n_kept = int(kept.sum())
        lowest_first += int(bool(kept[:n_kept].all()))
    with capsys.disabled():
        print(f"\n[tie report] rows with identical index lists: {rows_equal}/32; positions equal: {pos_equal:.4f}; "
              f"rows where torch.topk (CUDA) also keeps the lowest positions among the tied cut value: {lowest_first}/32; "
              f"(tied at cut, kept) first rows: {tied_at_cut[:4]}")


def test_active_intersection_and_row_list(L):
    g = torch.Generator().manual_seed(4)
    B, Ln, k = 6, 512, 384
    scores = torch.randn(B, Ln, generator=g)
    depth = torch.randint(0, 4, (B, Ln), generator=g)
    for r in range(4):
        idx, rows, count = select(L, scores, k, depth, r)
        ref_idx = O.mod_select(scores, 0.75)
        assert torch.equal(idx.long(), ref_idx)
        sel = torch.zeros(B, Ln, dtype=torch.bool)
        sel.scatter_(1, ref_idx, True)
        want = torch.nonzero((sel & (depth >= r)).flatten()).flatten()
        assert count == want.numel()
        assert torch.equal(rows[:count].long().sort()[0], want)   # per-sequence segments are ascending; their order is not fixed
        assert (rows[count:] == -1).all()


def test_mor_depths_match_oracle(L):
    g = torch.Generator().manual_seed(3)
    logits = torch.cat([torch.randn(100000, generator=g) * 2, torch.tensor([0.0, -50.0, 50.0, float("inf"), -float("inf")])])
    for n_rec, min_d in [(4, 0), (2, 0), (4, 1), (6, 2), (1, 0)]:
        ref, _ = O.mor_depths(logits, n_rec, min_d)
        out = torch.full((logits.numel(),), -1, dtype=torch.int32, device="cuda")
        lc = logits.cuda()
        L.check(L.lib().hb200_mor_depths(lc.data_ptr(), out.data_ptr(), logits.numel(), n_rec, min_d,
                                         torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        diff = out.cpu().long() != ref
        if diff.any():
            # only a logit whose continuous depth sits within float rounding of a .5 boundary may differ
            sq = torch.tanh(logits[diff].double() / 2) * 3
            cont = min_d + torch.sigmoid(sq) * (n_rec - 1 - min_d)
            assert ((cont - cont.floor() - 0.5).abs() < 1e-5).all()
        assert int(diff.sum()) <= 2


def test_public_routing_wrappers():
    """hydra_b200.routing.mod_select / mor_depths: the same entry points behind a tensor-in, tensor-out interface."""
    from hydra_b200.routing import mod_k, mod_select, mor_depths
    g = torch.Generator().manual_seed(3)
    scores = torch.randn(4, 333, generator=g) * 2
    for cap in (0.75, 0.3, 1.0, 1e-6):
        assert mod_k(333, cap) == O.mod_k(333, cap)
        assert torch.equal(mod_select(scores.cuda(), cap).cpu(), O.mod_select(scores, cap))
    logits = torch.randn(3, 200, generator=g) * 2
    for R, md in ((4, 0), (4, 1), (2, 0), (1, 0)):
        assert torch.equal(mor_depths(logits.cuda(), R, md).cpu(), O.mor_depths(logits, R, md)[0])
    with pytest.raises(RuntimeError):
        mod_select(scores, 0.5)
