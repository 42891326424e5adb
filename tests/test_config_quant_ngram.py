"""Host-side spec pieces: shapes, shard math, q4 format, n-gram hasher, PLE table."""
import numpy as np
import pytest
import torch

from qwb200.models.config import ModelConfig, ShardConfig
from qwb200.models import quant
from qwb200.models.ngram import NgramHasher, splitmix64, is_prime
from qwb200.models.ple import PleTable, f8e4m3_lut


def test_full_config_shapes():
    c = ModelConfig.full()
    c.validate()
    assert c.hch == 10240 and c.hc_down == 324 and c.idx_topk_blocks == 512
    assert c.gdn_qkv == 10240 and c.gdn_val == 6144 and c.ngram_dim == 160
    assert c.n_qsa == 12 and c.n_gdn == 36
    assert [c.is_qsa(i) for i in range(8)] == [False, False, False, True] * 2
    assert c.qsa_index(7) == 1 and c.gdn_index(4) == 3
    assert c.real_token(-3) == c.image_pad and c.real_token(-4) == c.video_pad and c.real_token(5) == 5


def test_shard_shapes_match_reference_tables():
    c = ModelConfig.full()
    s4 = ShardConfig(c, 4, 1)
    # the reference's 4-rank constants (src/core/shard.hpp)
    assert (s4.sh, s4.xw, s4.hc_send, s4.gdn_vl, s4.gdn_kl, s4.gdn_proj_l) == (640, 2560, 1300, 12, 4, 4120)
    assert (s4.qh_l, s4.kv_replicas, s4.qsa_proj_l, s4.exp_l, s4.sffn_l, s4.vocab_l, s4.ple_kv) == \
        (6, 2, 4224, 128, 160, 62080, 3200)
    assert s4.kv_primary == 0 and ShardConfig(c, 4, 3).kv_primary == 2
    s8 = ShardConfig(c, 8, 5)
    assert (s8.sh, s8.xw, s8.gdn_vl, s8.gdn_kl, s8.gdn_proj_l, s8.qh_l, s8.kv_replicas) == (320, 1280, 6, 2, 2060, 3, 4)
    assert (s8.qsa_proj_l, s8.exp_l, s8.sffn_l, s8.vocab_l, s8.ple_kv, s8.gdn_state) == (2688, 64, 80, 31040, 1600, 6 * 128 * 128)
    assert s8.kv_head0 == 1 and ShardConfig(c, 8, 3).kv_head0 == 0
    s1 = ShardConfig(c, 1, 0)
    assert s1.kvh_l == 2 and s1.qsa_proj_l == 12288 + 1024 + 640
    with pytest.raises(ValueError):
        ShardConfig(c, 3, 0)


def test_q4_roundtrip_and_engine_order():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(64, 512, generator=g) * 0.02).to(torch.bfloat16)
    pk, sc = quant.quantize_q4(w)
    assert pk.shape == (64, 64) and sc.shape == (64, 4) and pk.dtype == torch.int32
    q = quant.unpack_q4(pk)
    assert q.min() >= -8 and q.max() <= 7
    dq = quant.dequantize_q4(pk, sc)
    # error at most half a step (+ fp16 scale rounding)
    step = sc.float().repeat_interleave(128, dim=1)
    assert torch.all((dq - w.float()).abs() <= 0.5 * step * 1.01 + 1e-8)
    # a group's absolute maximum maps to +-7
    assert int(q.abs().max()) == 7
    # quantising the dequantised weights is a fixed point
    pk2, sc2 = quant.quantize_q4(dq)
    assert torch.equal(pk2, pk) and torch.equal(sc2, sc)
    # engine order: elements 2j, 2j+1 at bits 4j and 16+4j
    eo = quant.to_engine_order(pk)
    assert torch.equal(quant.from_engine_order(eo), pk)
    word = int(pk[3, 5]) & 0xFFFFFFFF
    ew = int(eo[3, 5]) & 0xFFFFFFFF
    for j in range(4):
        pair = (ew >> (4 * j)) & 0x000F000F
        assert pair & 0xF == (word >> (8 * j)) & 0xF
        assert pair >> 16 == (word >> (8 * j + 4)) & 0xF


def test_q4_known_word():
    # element 8c+i sits in bits 4i..4i+3 stored as q+8
    w = torch.zeros(1, 128)
    w[0, :8] = torch.tensor([-7., -5, -3, -1, 1, 3, 5, 7])
    pk, sc = quant.quantize_q4(w)
    assert abs(float(sc[0, 0]) - 1.0) < 1e-3
    word = int(pk[0, 0]) & 0xFFFFFFFF
    assert [(word >> (4 * i)) & 0xF for i in range(8)] == [1, 3, 5, 7, 9, 11, 13, 15]


def test_ngram_hasher_matches_direct_formula():
    c = ModelConfig.full()
    h = NgramHasher(c)
    assert len(h.sizes) == 16 and all(is_prime(s) for s in h.sizes)
    assert h.sizes[0] == 20000003 and h.sizes == sorted(h.sizes) and len(set(h.sizes)) == 16
    assert h.total_rows == sum(h.sizes) and h.total_rows <= 320_001_536
    assert all(m % 2 == 1 for m in h.mult)
    toks = [760, 6511, 248044, 314, 9338, 248044, 248044, 369, 1, 2, 3, 248319]
    got = h.ids_for([], toks)
    # direct transcription of the definition (docs/MODEL.md:192-204)
    EOS = c.eos
    ctx = [EOS, EOS] + toks
    for col in range(2, len(ctx)):
        prev = max([j for j in range(col) if ctx[j] == EOS], default=-1)
        since = col - prev - 1
        sh = [ctx[col - s] if since >= s else EOS for s in range(3)]
        ids = []
        for n in (2, 3):
            m = sh[0] * h.mult[0]
            for i in range(1, n):
                m ^= sh[i] * h.mult[i]
            for j in range(8):
                hh = (n - 2) * 8 + j
                ids.append(m % h.sizes[hh] + h.offsets[hh])
        assert got[col - 2].tolist() == ids
    # chunk boundary: history of 2 tokens gives the same ids as one pass
    a = h.ids_for(toks[:5], toks[5:])
    assert np.array_equal(a, got[5:])
    a = h.ids_for(toks[:4][-2:], toks[4:])
    assert np.array_equal(a, got[4:])
    # vision tokens hash as their pad token
    assert np.array_equal(h.ids_for([], [-3, 5]), h.ids_for([], [c.image_pad, 5]))
    assert splitmix64(0) == 0xE220A8397B1DCDAF


@pytest.mark.parametrize("layout", ["f8", "bf16", "int8", "int4"])
def test_ple_table_layouts(tmp_path, layout):
    c = ModelConfig.tiny()
    t = PleTable.synthetic(c, rows=500, layout=layout, n_shards=3, seed=1)
    ids = np.array([[0, 499, 250, 167] * 4, [166, 1, 333, 498] * 4])
    e = t.gather(ids)
    assert e.shape == (2, c.hidden) and torch.isfinite(e).all() and float(e.abs().max()) > 0
    t.save(str(tmp_path))
    t2 = PleTable.load(c, str(tmp_path))
    assert t2.layout == layout and t2.rows == 500
    assert torch.equal(t2.gather(ids), e)
    # one row read directly
    r = t.rows_f32(torch.tensor([250]))[0]
    assert torch.equal(e[0, 2 * c.ngram_dim:3 * c.ngram_dim], r)


def test_f8_lut():
    lut = f8e4m3_lut(2.0)
    assert lut[0] == 0 and lut[0x38] == 2.0 and lut[0xB8] == -2.0 and lut[0x7E] == 448 * 2.0
