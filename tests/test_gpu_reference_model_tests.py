"""The inference-side cases of the reference's own model tests (tests/test_ccgqa_model.py), run against this backend
with the same model shapes (dim 128, 4 heads -> head_dim 8; 4 blocks x 2 recursions; MoD capacity 0.5; vocab 1000):
creation attributes, output shapes over batch / sequence combinations, no cross-batch mixing (their tolerance 1e-4 is for
fp32; here the runs are bit-identical), inference without NaNs, RoPE cache resize, the base model's shapes.  Their
training-side cases (losses, gradients, checkpointing) have no counterpart in an inference backend."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small_mod_mor_model():
    from hydra_b200.model import create_ccgqa_mod_mor_model
    return create_ccgqa_mod_mor_model(vocab_size=1000, dim=128, n_mor_blocks=4, recursions_per_block=2, n_heads=4,
                                      n_kv_heads=2, mod_capacity=0.5, max_seq_len=512)


@pytest.fixture(scope="module")
def small_ccgqa_model():
    from hydra_b200.model import create_ccgqa_model

    class Spec:
        vocab_size, dim, n_layers, n_heads, n_kv_heads, compression_factor, max_seq_len = 1000, 128, 4, 4, 2, 2, 512
    return create_ccgqa_model(Spec())


def test_model_creates(small_mod_mor_model):
    m = small_mod_mor_model
    assert (m.dim, m.n_mor_blocks, m.recursions_per_block, m.effective_layers) == (128, 4, 2, 8)


def test_shape_invariants(small_mod_mor_model):
    for batch, seq in [(1, 16), (2, 32), (4, 64), (1, 128)]:
        x = torch.randint(0, 1000, (batch, seq), device="cuda")
        out = small_mod_mor_model(x, return_losses=False)
        assert out.shape == (batch, seq, 1000)
        assert torch.isfinite(out.float()).all()


def test_no_cross_batch_mixing(small_mod_mor_model):
    torch.manual_seed(42)
    seq_a = torch.randint(0, 1000, (1, 32), device="cuda")
    seq_b = torch.randint(0, 1000, (1, 32), device="cuda")
    out_a_solo = small_mod_mor_model(seq_a).clone()
    out_batched = small_mod_mor_model(torch.cat([seq_a, seq_b], dim=0))
    assert torch.equal(out_a_solo, out_batched[0:1])


def test_efficient_inference(small_mod_mor_model):
    out = small_mod_mor_model(torch.randint(0, 1000, (2, 32), device="cuda"), return_losses=False)
    assert out.shape == (2, 32, 1000) and not torch.isnan(out.float()).any()


def test_rope_cache_resize(small_mod_mor_model):
    small_mod_mor_model.resize_rope_cache(1024)
    assert small_mod_mor_model.max_seq_len == 1024
    assert small_mod_mor_model(torch.randint(0, 1000, (2, 128), device="cuda")).shape == (2, 128, 1000)


def test_base_model_creates_and_forward_shape(small_ccgqa_model):
    assert small_ccgqa_model.dim == 128 and small_ccgqa_model.n_layers == 4
    out = small_ccgqa_model(torch.randint(0, 1000, (2, 64), device="cuda"))
    assert out.shape == (2, 64, 1000) and torch.isfinite(out.float()).all()


def test_routing_stats_are_reported(small_mod_mor_model):
    small_mod_mor_model(torch.randint(0, 1000, (2, 64), device="cuda"), taps=True)
    stats = small_mod_mor_model.get_routing_stats()
    assert isinstance(stats, dict) and stats
