"""The non-prefix-reuse experiment's mathematics on CPU: the GDN transfer of a chunk is the scan of v = 0 from the
identity, re-basing a recorded chunk onto another prefix's state is exact when the chunk's inputs are the same,
cached keys re-rotate by the position shift, and position-indexed rings move with it."""
import torch

from qwb200.engine import blend as B
from qwb200.models.config import ModelConfig
from qwb200.models.reference import rope


def chunk(T, heads, dim, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(T, heads, dim, generator=g)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, heads, dim, generator=g)
    decay = -torch.rand(T, heads, generator=g) * 0.2
    beta = torch.sigmoid(torch.randn(T, heads, generator=g))
    return k, v, decay, beta


def test_transfer_is_the_product_of_the_steps():
    heads, dim, T = 3, 16, 20
    k, _, g, beta = chunk(T, heads, dim, 1)
    M = B.transfer_advance(B.transfer_init(heads, dim), k, g, beta)
    want = torch.eye(dim).repeat(heads, 1, 1)
    for t in range(T):
        step = torch.exp(g[t]).view(-1, 1, 1) * (torch.eye(dim) - beta[t].view(-1, 1, 1) * k[t].unsqueeze(-1) * k[t].unsqueeze(1))
        want = step @ want
    assert torch.allclose(M, want, atol=1e-5)
    # recorded piece by piece (one call per prefill piece) it is the same matrix
    M2 = B.transfer_init(heads, dim)
    for a in range(0, T, 7):
        M2 = B.transfer_advance(M2, k[a:a + 7], g[a:a + 7], beta[a:a + 7])
    assert torch.allclose(M2, M, atol=1e-6)


def test_rebased_chunk_matches_a_full_scan():
    heads, dim = 4, 32
    kA, vA, gA, bA = chunk(50, heads, dim, 2)          # the prefix the chunk was recorded after
    kB, vB, gB, bB = chunk(33, heads, dim, 3)          # another prefix
    kC, vC, gC, bC = chunk(40, heads, dim, 4)          # the chunk itself
    zero = torch.zeros(heads, dim, dim)
    S_A = B.delta_scan(zero, kA, vA, gA, bA)
    S_B = B.delta_scan(zero, kB, vB, gB, bB)
    rec = B.record(S_A, kC, vC, gC, bC, start=50)
    full = B.delta_scan(S_B, kC, vC, gC, bC)
    assert B.relative_error(rec.rebase(S_B), full) < 1e-5
    assert B.relative_error(rec.rebase(S_B, with_transfer=False), full) > 1e-3     # the correction is what makes it exact
    assert rec.shift(33) == -17 and rec.length == 40
    # layers stacked on a leading axis compose the same way
    S4 = torch.stack([S_B, S_A])
    out = B.compose(S4, torch.stack([rec.M, rec.M]), torch.stack([rec.S_in, rec.S_in]), torch.stack([rec.S_out, rec.S_out]))
    assert torch.allclose(out[0], rec.rebase(S_B)) and torch.allclose(out[1], rec.S_out, atol=1e-5)


def test_rope_shift_moves_cached_keys():
    cfg = ModelConfig.tiny()
    n, delta = 9, 1234
    K = torch.randn(n, cfg.head_dim)
    pos = torch.arange(100, 100 + n)
    moved = B.rope_shift(cfg, rope(cfg, K, pos), delta)
    assert torch.allclose(moved, rope(cfg, K, pos + delta), atol=1e-4)
    assert torch.equal(moved[:, cfg.rope_dim:], K[:, cfg.rope_dim:])               # only the rotary part changes
    back = B.rope_shift(cfg, moved, -delta)
    assert torch.allclose(back, rope(cfg, K, pos), atol=1e-4)
    kb = rope(cfg, K, pos).to(torch.bfloat16)
    assert B.rope_shift(cfg, kb, 3).dtype == torch.bfloat16


def test_rings_follow_the_positions():
    ring = 8
    old = torch.arange(ring * 3, dtype=torch.float32).view(ring, 3)
    for delta in (0, 5, -3, 19, -17):
        new = B.shift_ring(old, delta)
        for c in range(ring):
            assert torch.equal(new[B.ring_cell(c, delta, ring)], old[c])
    per_layer = torch.arange(2 * ring * 3, dtype=torch.float32).view(2, ring, 3)
    moved = B.shift_ring(per_layer, 5, dim=1)
    assert torch.equal(moved[1, B.ring_cell(2, 5, ring)], per_layer[1, 2])
