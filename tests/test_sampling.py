"""Sampling (the demo's temperature / top-p settings) against transformers' own logits warpers, on the CPU."""
import pytest
import torch

from mixtral_offloading_b200.sampling import sample_token, top_p_filter


@pytest.mark.parametrize("top_p", [0.9, 0.5, 0.05, 1.0])
def test_top_p_filter_matches_transformers(top_p):
    from transformers.generation.logits_process import TemperatureLogitsWarper, TopPLogitsWarper
    g = torch.Generator().manual_seed(3)
    logits = 3 * torch.randn(4, 1000, generator=g)
    ids = torch.zeros(4, 1, dtype=torch.long)
    want = TemperatureLogitsWarper(0.9)(ids, logits.clone())
    if top_p < 1.0:
        want = TopPLogitsWarper(top_p)(ids, want)
    got = top_p_filter(logits / 0.9, top_p)
    assert torch.equal(torch.isinf(got), torch.isinf(want))
    keep = ~torch.isinf(want)
    assert torch.allclose(got[keep], want[keep])
    assert (keep.sum(-1) >= 1).all()


def test_sample_token_draws_from_the_nucleus_only():
    g = torch.Generator().manual_seed(0)
    logits = torch.tensor([[5.0, 4.0, 0.0, -1.0, -2.0]]).repeat(64, 1)
    toks = sample_token(logits, temperature=0.9, top_p=0.9, generator=g)
    assert toks.shape == (64,) and toks.dtype == torch.int64
    assert set(toks.tolist()) <= {0, 1}                       # tokens 0 and 1 hold > 0.9 of the mass
    assert len(set(toks.tolist())) == 2
    with pytest.raises(ValueError):
        sample_token(logits, temperature=0.0)
    with pytest.raises(ValueError):
        top_p_filter(logits, 0.0)
