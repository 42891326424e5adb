"""Vision cache, media keys, slice split and patch positions (no GPU)."""
import numpy as np
import torch


def test_cache_and_keys_and_split():
    from qwb200.vision import VisionCache, assign_slices, media_key
    calls = []

    def enc(p, h, w):
        calls.append((h, w))
        return torch.zeros(h * w // 4, 8)
    c = VisionCache(enc, budget_bytes=3 * 6 * 8 * 4)
    a = c.get(11, 0, None, 4, 6)
    assert c.get(11, 0, None, 4, 6) is a and c.hits == 1 and len(calls) == 1
    for k in range(5):
        c.get(20 + k, 0, None, 4, 6)
    assert c.bytes <= c.budget and (11, 0) not in c.lru
    keys = {media_key(123, s, t) for s in range(3) for t in range(50)}
    assert len(keys) == 150 and all(k < 0 for k in keys) and media_key(123, 0, 0) != media_key(124, 0, 0)
    parts = assign_slices([10, 1, 1, 1, 9, 8], 2)
    loads = [sum([10, 1, 1, 1, 9, 8][i] for i in p) for p in parts]
    assert sorted(i for p in parts for i in p) == list(range(6)) and abs(loads[0] - loads[1]) <= 4 and parts[0][0] == 0


def test_slice_positions_cover_the_grid_in_merge_order():
    from qwb200.vision import slice_positions
    pos, idx, wts = slice_positions(4, 6, 2, 48)
    assert pos[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]] and pos[4].tolist() == [0, 2]
    assert sorted(map(tuple, pos.tolist())) == [(r, c) for r in range(4) for c in range(6)]
    assert np.allclose(wts.sum(1), 1.0) and idx.min() >= 0 and idx.max() < 48 * 48
    # corners of the image sit on the corners of the table
    last = np.where((pos[:, 0] == 3) & (pos[:, 1] == 5))[0][0]
    assert idx[0, 0] == 0 and wts[0, 0] == 1.0 and idx[last, 0] == 47 * 48 + 47
