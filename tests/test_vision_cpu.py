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


def test_media_descriptors_read_by_address_and_mapped_by_value():
    """The C API's media structs are read into plain values (which can travel to other ranks) and registering them by value
    gives the same token ids as registering them by address."""
    import ctypes as C
    import pickle
    import numpy as np
    from qwb200.capi_impl import QwMedia
    from qwb200.models.config import ModelConfig
    from qwb200.vision import VisionConfig
    from qwb200.vision.frontend import VisionFrontend

    class Enc:          # the front end needs the tower's geometry only until a slice is looked up
        cfg = VisionConfig(depth=1, out_dim=ModelConfig.tiny().hidden)

        def encode(self, *a):
            raise AssertionError("not called")
    cfg, vc = ModelConfig.tiny(), Enc.cfg
    h, w = 4, 6
    n_img = h * w // (vc.merge * vc.merge)
    img = np.random.default_rng(1).standard_normal((2 * h * w, vc.patch_in)).astype(np.float32)
    starts = np.asarray([10, 40], dtype=np.int64)
    toks = [5 + i for i in range(10)] + [cfg.video_pad] * n_img + [7] * (30 - n_img) + [cfg.video_pad] * n_img + [9, 9]
    m = QwMedia(hash=4242, video=1, t=2, h=h, w=w, patches=img.ctypes.data_as(C.POINTER(C.c_float)),
                starts=starts.ctypes.data_as(C.POINTER(C.c_int64)))
    arr = (QwMedia * 1)(m)
    a, b = VisionFrontend(Enc(), 1 << 20), VisionFrontend(Enc(), 1 << 20)
    by_addr = a.map_media_tokens(toks, C.addressof(arr), 1)
    media = pickle.loads(pickle.dumps(b.read_media(C.addressof(arr), 1)))          # as it would reach a worker rank
    by_value = b.map_media(toks, media)
    assert by_addr == by_value and by_addr != toks
    assert all(t < 0 for t in by_addr[10:10 + n_img] + by_addr[40:40 + n_img]) and by_addr[:10] == toks[:10]
    assert media[0][0] == 4242 and media[0][1] is True and media[0][5].shape == (2 * h * w, vc.patch_in)
    assert set(a.where) == set(b.where) and len(a.where) == 2 * n_img
