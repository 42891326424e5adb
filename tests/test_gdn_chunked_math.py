"""The chunked (WY) form of the gated delta rule equals the token-by-token recurrence (CPU, fp32)."""
import pytest
import torch

from qwb200.models.gdn_chunked import scan_chunked, scan_sequential


@pytest.mark.parametrize("T,chunk", [(64, 64), (200, 64), (130, 32)])
def test_chunked_equals_sequential(T, chunk):
    g = torch.Generator().manual_seed(T)
    dk = dv = 128
    q = torch.nn.functional.normalize(torch.randn(T, dk, generator=g), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, dk, generator=g), dim=-1)
    v = torch.randn(T, dv, generator=g)
    decay = torch.exp(-torch.rand(T, generator=g) * 0.3)
    beta = torch.sigmoid(torch.randn(T, generator=g))
    S0 = torch.randn(dk, dv, generator=g) * 0.1
    o1, s1 = scan_sequential(q, k, v, decay, beta, S0)
    o2, s2 = scan_chunked(q, k, v, decay, beta, S0, chunk=chunk)
    assert (o1 - o2).abs().max() / o1.abs().max() < 1e-5
    assert (s1 - s2).abs().max() / s1.abs().max() < 1e-5


def test_strong_decay_does_not_overflow():
    T, dk = 128, 128
    g = torch.Generator().manual_seed(1)
    q = torch.randn(T, dk, generator=g) * 0.1
    k = torch.nn.functional.normalize(torch.randn(T, dk, generator=g), dim=-1)
    v = torch.randn(T, dk, generator=g)
    decay = torch.full((T,), 1e-20)
    beta = torch.full((T,), 0.5)
    o1, s1 = scan_sequential(q, k, v, decay, beta, torch.zeros(dk, dk))
    o2, s2 = scan_chunked(q, k, v, decay, beta, torch.zeros(dk, dk))
    assert torch.isfinite(o2).all() and torch.isfinite(s2).all()
    assert (o1 - o2).abs().max() < 1e-5
