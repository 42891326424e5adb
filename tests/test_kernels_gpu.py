"""Numerics of the decode kernels against plain PyTorch fp32 references (GPU only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def rel(a, b):
    return (a - b).abs().max() / b.abs().max()


@pytest.mark.parametrize("N,K", [(324, 2560), (512 + 1281, 2560), (2560, 6144), (16444, 2560), (40, 64)])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 16, 32])
def test_gemv_bf16_matches_fp32_and_rows_are_batch_invariant(N, K, M):
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(N + K + M)
    W = (torch.randn(N, K, generator=g, device=_dev()) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, generator=g, device=_dev()).to(torch.bfloat16)
    out = torch.full((M, N + 3), 777.0, device=_dev())       # guard columns detect stray writes
    K_.gemv_bf16(W, x, out=out, N=N, ldy=N + 3)
    ref = x.float() @ W.float().T
    assert torch.all(out[:, N:] == 777.0)
    assert torch.allclose(out[:, :N], ref, atol=2e-2 * (K ** 0.5) * 0.05, rtol=2e-3)
    # a row alone gives bit-identical results to the row inside the batch
    one = K_.gemv_bf16(W, x[M - 1:M].contiguous())
    assert torch.equal(one[0], out[M - 1, :N])


def test_gemv_column_splits():
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(5)
    hc, SH, R, M = 4, 640, 324, 3
    W = (torch.randn(R, hc * SH, generator=g, device=_dev()) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, hc * SH, generator=g, device=_dev()).to(torch.bfloat16)
    out = torch.zeros(M, hc + hc * R, device=_dev())
    K_.gemv_bf16(W, x, out=out[:, hc:], nsplit=hc, splits=(SH, SH, R), N=R, K=SH, ldw=hc * SH, ldy=out.stride(0))
    ref = torch.einsum("rsc,msc->msr", W.float().view(R, hc, SH), x.float().view(M, hc, SH)).reshape(M, hc * R)
    assert torch.allclose(out[:, hc:], ref, atol=5e-2, rtol=2e-3)
    assert torch.all(out[:, :hc] == 0)


def test_row_reduce_argmax_ties_and_lse():
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(1)
    l = torch.randn(5, 31040, generator=g, device=_dev())
    l[2, 100] = l[2, 30000] = 50.0       # tie: lowest index wins
    val, idx, mx, sm = K_.row_reduce(l, idx0=1000)
    assert idx.tolist()[2] == 1100
    assert torch.equal(idx.long() - 1000, torch.argmax(l, -1)) or idx.tolist()[2] == 1100
    ref = torch.logsumexp(l.double(), -1).float()
    assert torch.allclose(mx + torch.log(sm), ref, atol=1e-4)


@pytest.mark.parametrize("nb", [600, 1025, 5000])
def test_qsa_select_topk_with_ties(nb):
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(nb)
    topk, ratio = 512, 4
    sc = torch.rand(3, 8192, generator=g, device=_dev())
    sc[1, :nb] = torch.randint(0, 40, (nb,), generator=g, device=_dev()).float()     # many ties
    sc[2, :nb] = 0.0                                                                  # all equal
    pos = torch.tensor([nb * ratio + 1, nb * ratio + 3, nb * ratio], dtype=torch.int32, device=_dev())
    sel, sel_n = K_.qsa_select(sc, pos, ratio, topk)
    assert sel_n.tolist() == [topk] * 3
    for m in range(3):
        order = torch.sort(-sc[m, :nb], stable=True).indices[:topk]
        assert sel[m].tolist() == sorted(order.tolist())
    # below the budget everything is attended
    sel, sel_n = K_.qsa_select(sc, torch.tensor([100, 2047, 2050], dtype=torch.int32, device=_dev()), ratio, topk)
    assert sel_n.tolist() == [-1, -1, -1]


def test_moe_pair_kernels_match_oracle():
    from qwb200.models.config import ModelConfig
    from qwb200.models.weights import synth_layer
    from qwb200.models.reference import RefModel
    from qwb200.engine.weights_prep import prep_moe
    from qwb200.models.config import ShardConfig
    from qwb200.ops import kernels as K_
    cfg = ModelConfig.tiny(n_layers=1, layer_types=("gdn",))
    w = synth_layer(cfg, 0, seed=2)
    ref = RefModel(cfg, w)
    sc = ShardConfig(cfg, 1, 0)
    mw = prep_moe(w, "layers.0.mlp.", sc, _dev())
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, cfg.hidden, generator=g).to(torch.bfloat16)
    want = ref.moe("layers.0.mlp.", x.float())
    xd = x.to(_dev())
    rs = K_.gemv_bf16(mw["Wrs"], xd)
    pe, pw, sh = K_.moe_route(rs, cfg.n_experts, cfg.top_k, sc.sffn_l)
    idx, wgt, _ = ref.route("layers.0.mlp.", x.float())
    assert torch.equal(pe.cpu().long(), idx)
    assert torch.allclose(pw.cpu(), wgt, atol=1e-5)
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    try:
        for mask in (0, 1, 3, 12):      # scalar kernels, tensor-core gate/up, + tensor-core down, bulk-copy-fed tensor-core forms
            L.qwk_set_moe_mma(mask)
            out = K_.moe_experts_pair(mw["w13"], mw["s13"], mw["w2"], mw["s2"], xd, pe, pw, cfg.ffn, cfg.hidden, mw["Wsd"], sh)
            err = (out.cpu() - want).abs().max() / want.abs().max()
            assert err < 2e-2, (mask, float(err))
    finally:
        L.qwk_set_moe_mma(12)


@pytest.mark.parametrize("M,KL,VL", [(64, 2, 4), (200, 2, 4), (1000, 2, 4), (200, 4, 16), (200, 8, 32)])
def test_gdn_chunked_scan_matches_sequential_fp32(M, KL, VL):
    """The chunked (tensor-core) delta-rule scan against the token-by-token recurrence in PyTorch fp32 and
    against the row-by-row kernel: outputs, and the state it leaves in the slot."""
    import ctypes as C
    from qwb200.models.gdn_chunked import scan_sequential
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    dev = _dev()
    g = torch.Generator(device="cuda").manual_seed(M)
    D, slots, slot = 128, 3, 1          # VL < 16, < 32, >= 32: the three column splits of the sequential walk
    qkv_l = (2 * KL + VL) * D
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    q = torch.nn.functional.normalize(rn(M, KL, D), dim=-1) * D ** -0.5
    k = torch.nn.functional.normalize(rn(M, KL, D), dim=-1)
    v = rn(M, VL, D)
    qkv = torch.cat([q.reshape(M, -1), k.reshape(M, -1), v.reshape(M, -1)], 1).contiguous()
    decay = torch.exp(-torch.rand(M, VL, generator=g, device=dev) * 0.2).contiguous()
    beta = torch.sigmoid(rn(M, VL)).contiguous()
    ld = qkv_l + VL * D + 2 * VL
    proj = rn(M, ld).contiguous()
    S0 = (rn(slots, VL, D, D) * 0.1).contiguous()
    nw = (1 + 0.1 * rn(D)).contiguous()
    eps = 1e-6
    # fp32 oracle
    want_o = torch.empty(M, VL, D, device=dev)
    want_S = S0.clone()
    for h in range(VL):
        kh = h // (VL // KL)
        o, S = scan_sequential(q[:, kh].cpu(), k[:, kh].cpu(), v[:, h].cpu(), decay[:, h].cpu(), beta[:, h].cpu(), S0[slot, h].cpu())
        z = proj[:, qkv_l + h * D: qkv_l + (h + 1) * D].cpu()
        want_o[:, h] = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * nw.cpu() * torch.sigmoid(z)).to(dev)
        want_S[slot, h] = S.to(dev)
    P = lambda t: C.c_void_p(t.data_ptr())
    rows = torch.zeros(4, M, dtype=torch.int32, device=dev)
    rows[0] = slot
    rows[1] = torch.arange(M, device=dev)
    rows[3, 0] = M
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    nch = (M + 63) // 64
    scratch = torch.zeros(nch * VL * (2 * 64 * 128 + 64 * 64 + 64) + M * VL * 128, device=dev)
    S_c = S0.clone()
    o_c = torch.zeros(M, VL * D, dtype=torch.bfloat16, device=dev)
    rc = L.qwk_gdn_scan_chunked(P(qkv), P(decay), P(beta), P(proj), ld, P(S_c), P(nw), KL, VL, M, P(rows[0]), P(scratch),
                                P(o_c), C.c_float(eps), s)
    assert rc == 0
    S_s = S0.clone()
    o_s = torch.zeros(M, VL * D, dtype=torch.bfloat16, device=dev)
    rc = L.qwk_gdn_scan(P(qkv), P(decay), P(beta), P(proj), ld, P(S_s), None, P(nw), KL, VL, M, P(rows[0]), P(rows[1]),
                        P(rows[2]), P(rows[3]), P(o_s), C.c_float(eps), s)
    assert rc == 0
    torch.cuda.synchronize()
    w = want_o.reshape(M, -1)
    assert rel(o_s.float(), w) < 1e-2                   # the row-by-row kernel (bf16 output rounding)
    assert rel(o_c.float(), w) < 1e-2, float(rel(o_c.float(), w))
    assert rel(S_c[slot], want_S[slot]) < 5e-3, float(rel(S_c[slot], want_S[slot]))
    assert torch.equal(S_c[0], S0[0]) and torch.equal(S_c[2], S0[2])      # other slots untouched


@pytest.mark.parametrize("QL,KVL", [(24, 2), (8, 2), (3, 1)])
def test_qsa_attend_mma_matches_fp32_and_decode_kernel(QL, KVL):
    """Tensor-core prefill attention over the paged KV against PyTorch fp32 and against the decode attention kernel:
    dense rows (below the budget), sparse rows (selected groups + open tail), a shuffled page table."""
    import ctypes as C
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    dev = _dev()
    g = torch.Generator(device="cuda").manual_seed(QL)
    HD, topk, ratio, page = 256, 512, 4, 256
    n_pages = 14
    positions = [0, 1, 62, 63, 64, 200, 2047, 2048, 2049, 2050, 2051, 2500, 3001, 3583]
    M = len(positions)
    kpool = (torch.randn(n_pages, page, KVL * HD, generator=g, device=dev)).to(torch.bfloat16)
    vpool = (torch.randn(n_pages, page, KVL * HD, generator=g, device=dev)).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    page_table = perm.to(dev).contiguous()
    q = torch.randn(M, QL, HD, generator=g, device=dev).contiguous()
    ldp = QL * 2 * HD + 40
    proj = torch.randn(M, ldp, generator=g, device=dev).contiguous()
    pos = torch.tensor(positions, dtype=torch.int32, device=dev)
    slot = torch.zeros(M, dtype=torch.int32, device=dev)
    sel = torch.zeros(M, topk, dtype=torch.int32, device=dev)
    sel_n = torch.full((M,), -1, dtype=torch.int32, device=dev)
    lists = []
    for m, p in enumerate(positions):
        nb = (p + 1) // ratio
        if nb > topk:
            ch = torch.sort(torch.randperm(nb, generator=torch.Generator().manual_seed(m))[:topk]).values
            sel[m] = ch.to(dev, torch.int32)
            sel_n[m] = topk
            toks = (ch[:, None] * ratio + torch.arange(ratio)[None]).reshape(-1).tolist() + list(range(nb * ratio, p + 1))
        else:
            toks = list(range(p + 1))
        lists.append(torch.tensor(toks, dtype=torch.long, device=dev))
    kf = kpool.float()[page_table.long()].reshape(-1, KVL, HD)        # token-major view through the page table
    vf = vpool.float()[page_table.long()].reshape(-1, KVL, HD)
    per = QL // KVL
    want = torch.empty(M, QL, HD, device=dev)
    for m in range(M):
        for h in range(QL):
            kv = h // per
            sc = (kf[lists[m], kv] @ q[m, h]) / 16.0
            w = torch.softmax(sc, 0)
            gate = proj[m, h * 2 * HD + HD: h * 2 * HD + 2 * HD]
            want[m, h] = (w @ vf[lists[m], kv]) * torch.sigmoid(gate)
    P = lambda t: C.c_void_p(t.data_ptr())
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    o = torch.zeros(M, QL, HD, dtype=torch.bfloat16, device=dev)
    rc = L.qwk_qsa_attend_mma(P(q), QL, KVL, M, P(slot), P(pos), P(kpool), P(vpool), None, None, n_pages, P(page_table), n_pages,
                              P(sel), P(sel_n), topk, ratio, P(proj), ldp, P(o), s)
    assert rc == 0
    nsplit = (topk * ratio + 8 + 63) // 64 + 24
    pm = torch.zeros(M, QL, nsplit, device=dev)
    pl = torch.zeros(M, QL, nsplit, device=dev)
    pacc = torch.zeros(M, QL, nsplit, HD, device=dev)
    o2 = torch.zeros(M, QL, HD, dtype=torch.bfloat16, device=dev)
    rc = L.qwk_qsa_attend(P(q), QL, KVL, M, P(slot), P(pos), P(kpool), P(vpool), None, None, n_pages, P(page_table), n_pages,
                          P(sel), P(sel_n), topk, ratio, nsplit, P(pm), P(pl), P(pacc), P(proj), ldp, P(o2), s)
    assert rc == 0
    torch.cuda.synchronize()
    assert rel(o2.float(), want) < 1e-2
    assert rel(o.float(), want) < 2e-2, rel(o.float(), want)


@pytest.mark.parametrize("base,M", [(2040, 70), (9000, 100)])
def test_qsa_scores_tensor_core_form_matches_fp32(base, M):
    """Indexer scores of a prefill chunk (more rows than a decode batch: the tensor-core kernel) against PyTorch fp32:
    rows at and around the budget boundary, groups past a row's visible range untouched."""
    import ctypes as C
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    dev = _dev()
    g = torch.Generator(device="cuda").manual_seed(base)
    IH, ID, ratio, topk, cap = 4, 128, 4, 512, 4096
    ck = torch.randn(2, cap, ID, generator=g, device=dev).to(torch.bfloat16)
    iq = torch.randn(M, IH, ID, generator=g, device=dev).contiguous()
    slot = torch.ones(M, dtype=torch.int32, device=dev)
    pos = torch.arange(base, base + M, dtype=torch.int32, device=dev)
    scores = torch.full((M, cap), -7.0, device=dev)
    P = lambda t: C.c_void_p(t.data_ptr())
    rc = L.qwk_qsa_scores(P(iq), IH, P(ck), cap, M, P(slot), P(pos), ratio, topk, P(scores), cap, (base + M) // ratio,
                          C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    want = torch.relu(torch.einsum("mhd,cd->mhc", iq, ck[1].float())).sum(1) / ID ** 0.5
    for m in range(M):
        nb = (base + m + 1) // ratio
        if nb <= topk:
            assert torch.all(scores[m] == -7.0)
        else:
            assert torch.all(scores[m, nb:] == -7.0)
            err = (scores[m, :nb] - want[m, :nb]).abs().max() / want[m, :nb].abs().max()
            assert err < 1e-3, (m, float(err))
