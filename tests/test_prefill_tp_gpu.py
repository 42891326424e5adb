"""Token-major prefill through the native runtime: against the Python-scheduled form on one rank, as two micro-batches,
and on 2 and 4 tensor-parallel ranks emulated in one process on one GPU (``parallel/emulate.py``) against one rank."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


def rows_close(mine, ref, frac=0.9, tol=5e-2):
    """Row-wise comparison for state that follows discrete routing decisions: a token whose top-k experts flip on a
    near-tie legitimately differs, so most rows must agree closely instead of every element."""
    a, b = mine.float().reshape(mine.shape[0], -1), ref.float().reshape(ref.shape[0], -1)
    err = (a - b).abs().amax(1) / b.abs().amax(1).clamp_min(1e-6)
    return float((err < tol).float().mean()) >= frac and float(err.median()) < tol / 2


def tiny_setup(seed=21, **kw):
    from qwb200.models.config import ModelConfig
    from qwb200.models.ple import PleTable
    from qwb200.models.weights import synth_weights
    cfg = ModelConfig.tiny(hidden=512, ffn=256, q_heads=8, kv_heads=2, gdn_qk_heads=8, gdn_v_heads=16, n_experts=32, **kw)
    w = synth_weights(cfg, seed=seed)
    table = PleTable.synthetic(cfg, rows=4096, layout="f8", seed=seed)
    toks = torch.randint(0, cfg.vocab, (330,), generator=torch.Generator().manual_seed(seed)).tolist()
    return cfg, w, table, toks


def test_native_runtime_equals_python_schedule():
    """One rank: the runtime's launch sequence and the one spelled out in Python run the same kernels in the same order."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.utils import settings
    cfg, w, table, toks = tiny_setup()
    opts = EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=128)
    a = Engine.from_weights(cfg, w, table, opts)
    la = a.prefill(0, toks).clone()
    assert a.prefiller.native
    old = settings.get()
    try:
        settings.set_current(settings.Settings.from_env(prefill_py=True))
        b = Engine.from_weights(cfg, w, table, opts)
        lb = b.prefill(0, toks).clone()
        assert not b.prefiller.native
    finally:
        settings.set_current(old)
    torch.cuda.synchronize()
    a.dm.check_error()
    assert torch.equal(la, lb)
    for x, y in zip(a.dm.gdn_S, b.dm.gdn_S):
        assert torch.equal(x, y)
    for qi in range(cfg.n_qsa):          # backbone KV (the MTP layer's rows at chunk borders come from different kernels)
        assert torch.equal(a.dm.k_dev[qi], b.dm.k_dev[qi]) and torch.equal(a.dm.v_dev[qi], b.dm.v_dev[qi])
    assert torch.equal(a.dm.ple_ring, b.dm.ple_ring)


def test_two_micro_batches_equal_one():
    """One rank, a chunk as two lanes on two streams: same logits and state as one lane."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.engine.prefill import Prefiller
    cfg, w, table, toks = tiny_setup(seed=22)
    opts = EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=256)
    a = Engine.from_weights(cfg, w, table, opts)
    la = a.prefill(0, toks).clone()
    b = Engine.from_weights(cfg, w, table, opts)
    b.prefiller = Prefiller(b.dm, chunk=256, lanes=2)
    assert b.prefiller.lanes == 2 and b.prefiller.lane_split(256) == 128
    lb = b.prefill(0, toks).clone()
    torch.cuda.synchronize()
    b.dm.check_error()
    assert rel(lb, la) < 1e-5
    for x, y in zip(a.dm.gdn_S, b.dm.gdn_S):
        assert rel(y, x) < 1e-5
    for qi in range(cfg.n_qsa + 1):
        assert rel(b.dm.k_dev[qi], a.dm.k_dev[qi]) < 1e-5
    assert int(a.dm.buf["amax_idx"][0]) == int(b.dm.buf["amax_idx"][0])


@pytest.mark.parametrize("ranks", [2, 4])
def test_emulated_ranks_match_one_rank(ranks):
    """Tensor + expert parallel prefill with the collectives inside the kernels, ranks emulated on one GPU: logits, greedy
    token and slot state against the one-rank prefill; three chunks, so the pending MTP row and the rings cross chunks."""
    from qwb200.engine.engine import Engine, EngineOptions
    from qwb200.parallel.emulate import EmulatedRanks
    cfg, w, table, toks = tiny_setup(seed=23)
    opts = EngineOptions(slots=1, slot_tokens=512, use_graphs=False, prefill_chunk=128)
    one = Engine.from_weights(cfg, w, table, opts)
    want = one.prefill(0, toks).clone()
    want_tok = int(one.dm.buf["amax_idx"][0])
    grp = EmulatedRanks(cfg, w, table, opts, ranks)
    tok = grp.prefill(0, toks)
    got = grp.logits()
    assert got.shape == want.shape
    assert rel(got, want) < 3e-2
    top2 = torch.topk(want, 2).values
    assert tok == want_tok or float(top2[0] - top2[1]) < 0.05 * float(want.abs().max())
    # every rank ends with the same merged token, and with its shard of the state
    assert len({int(e.dm.buf["amax_idx"][0]) for e in grp.engines}) == 1
    vl = cfg.gdn_v_heads // ranks
    for r, e in enumerate(grp.engines):
        for gi in range(cfg.n_gdn):
            assert rel(e.dm.gdn_S[gi][0], one.dm.gdn_S[gi][0, r * vl:(r + 1) * vl]) < 5e-2
        h0, nh = e.dm.sc.kv_head0, e.dm.sc.kvh_l
        for qi in range(cfg.n_qsa + 1):          # the MTP layer's KV included
            ref = one.dm.k_dev[qi].view(-1, cfg.kv_heads, cfg.head_dim)[:len(toks) - 1, h0:h0 + nh]
            mine = e.dm.k_dev[qi].view(-1, nh, cfg.head_dim)[:len(toks) - 1]
            assert rows_close(mine, ref), (r, qi)
        cols = e.dm.sc.cols()
        ring_one = one.dm.ple_ring[0].view(-1, cfg.hc, cfg.hidden)[:, :, cols]
        assert rows_close(e.dm.ple_ring[0].view(-1, cfg.hc, e.dm.sc.sh), ring_one, frac=0.7)
        assert rel(e.slot[0].mtp_hidden, one.slot[0].mtp_hidden[:, cols]) < 1e-1


def test_stand_alone_collectives_and_a_wait_that_runs_out():
    """The channel's stand-alone collectives on four emulated ranks (sums in rank order, identical on every rank), and the
    bounded wait: a collective nobody sends makes the waiting kernel give up, report to the error word and return; after
    the word is cleared the channel works as before."""
    from qwb200.models.config import ModelConfig
    from qwb200.ops import lib as qlib, structs as S
    from qwb200.parallel import tp_channel
    L = qlib.load(True)
    dev = torch.device("cuda:0")
    cfg = ModelConfig.tiny(hidden=512)
    R, rows, n = 4, 96, 128
    chans = tp_channel.make_emulated(cfg, R, 256, dev, mtp=False, spin_limit=4000)
    err = torch.zeros(2, dtype=torch.int32, device=dev)
    L.qwk_set_error_word(C.c_void_p(err.data_ptr()))
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cpu").manual_seed(3)
    src = [torch.randn(rows, n, generator=g).to(dev) for _ in range(R)]
    dst = [torch.full((rows, n), float("nan"), device=dev) for _ in range(R)]
    # all-reduce: every rank sends, then every rank adds
    for r in range(R):
        assert L.qwk_tp_push(chans[r].ptr, S.TP_RS, src[r].data_ptr(), n * 4, rows, n * 4, 0, s) == 0
    for r in range(R):
        assert L.qwk_tp_reduce(chans[r].ptr, S.TP_RS, dst[r].data_ptr(), rows * n, s) == 0
    want = torch.zeros(rows, n, device=dev)
    for r in range(R):
        want = want + src[r]            # rank order, like the kernel
    for r in range(R):
        assert torch.equal(dst[r], want)
    # reduce-scatter: rank d ends with the sum of everybody's column block d
    wide = [torch.randn(rows, R * 32, generator=g).to(dev) for _ in range(R)]
    out = [torch.zeros(rows, 32, device=dev) for _ in range(R)]
    for r in range(R):
        assert L.qwk_tp_push(chans[r].ptr, S.TP_RS, wide[r].data_ptr(), R * 32 * 4, rows, 32 * 4, 1, s) == 0
    for r in range(R):
        assert L.qwk_tp_reduce(chans[r].ptr, S.TP_RS, out[r].data_ptr(), rows * 32, s) == 0
    for d in range(R):
        w_ = torch.zeros(rows, 32, device=dev)
        for r in range(R):
            w_ = w_ + wide[r][:, d * 32:(d + 1) * 32]
        assert torch.equal(out[d], w_)
    # all-gather into one matrix
    part = [torch.randn(rows, 16, generator=g).to(dev) for _ in range(R)]
    for r in range(R):
        assert L.qwk_tp_push(chans[r].ptr, S.TP_SMALL, part[r].data_ptr(), 64, rows, 64, 2, s) == 0
    for r in range(R):
        assert L.qwk_tp_wait(chans[r].ptr, S.TP_SMALL, s) == 0
    torch.cuda.synchronize()
    assert err.tolist() == [0, 0]
    for r in range(R):
        got = chans[r].view(S.TP_SMALL, rows * R * 64, torch.float32).view(rows, R * 16)
        assert torch.equal(got, torch.cat(part, dim=1))
    # a collective that only rank 0 believes in: its wait runs out after 4,000 polls and the kernel returns
    chans[0].struct.seq[S.TP_SMALL] += 1
    assert L.qwk_tp_wait(chans[0].ptr, S.TP_SMALL, s) == 0
    torch.cuda.synchronize()
    code, detail = err.tolist()
    assert code == 1 and (detail & 0x20000000)          # ERR_WAIT_TIMEOUT from a channel wait; bits 24..26: the missing rank
    assert ((detail >> 24) & 7) in range(R) and (detail & 0xffffff) == chans[0].struct.seq[S.TP_SMALL]
    chans[0].struct.seq[S.TP_SMALL] -= 1
    err.zero_()
    for r in range(R):
        assert L.qwk_tp_push(chans[r].ptr, S.TP_RS, src[r].data_ptr(), n * 4, rows, n * 4, 0, s) == 0
    for r in range(R):
        assert L.qwk_tp_reduce(chans[r].ptr, S.TP_RS, dst[r].data_ptr(), rows * n, s) == 0
    torch.cuda.synchronize()
    assert err.tolist() == [0, 0] and torch.equal(dst[2], want)
    L.qwk_set_error_word(None)
