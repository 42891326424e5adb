"""tcgen05 GEMM numerics against a plain fp32 matmul (GPU only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,N,K", [(128, 128, 64), (128, 128, 256), (256, 384, 2560), (200, 324, 2560), (4096, 512, 2560),
                                   (77, 130, 328),
                                   # wide enough (N >= 1024, >= 74 tiles) for the 128 x 256 tile form, with ragged edges
                                   (1024, 2560, 320), (2000, 1536, 640), (4096, 1200, 128), (1111, 10240, 64)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_matches_fp32(T, N, K, out_dtype):
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(T + N + K)
    A = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    ldc = (N + 7) // 8 * 8 + 8
    out = torch.full((T, ldc), 768.0, dtype=out_dtype, device="cuda")      # guard columns detect stray writes
    K_.gemm_bf16_tc(A, W, out=out[:, :N])
    torch.cuda.synchronize()
    ref = A.float() @ W.float().T
    assert torch.all(out[:, N:].float() == 768.0)
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    err = float((out[:, :N].float() - ref).abs().max() / ref.abs().max())
    assert err < tol, err


@pytest.mark.parametrize("Nw,K,counts", [(256, 256, [5, 0, 130, 128, 1, 300]), (1280, 2560, [80, 200, 0, 33]),
                                         (2560, 640, [77, 129, 64])])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_q4_gemm_matches_fp32(Nw, K, counts, out_dtype):
    """Grouped tcgen05 GEMM whose W operand is dequantised from q4 inside the kernel: every group's rows against
    A @ dequant(W_group)^T in fp32, rows of unused tile entries and guard rows untouched."""
    import ctypes as C
    from qwb200.models.quant import dequantize_q4, quantize_q4, to_engine_order
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(Nw + K)
    E = len(counts)
    W = torch.randn(E * Nw, K, generator=g, device=dev) * 0.05
    packed, scale = quantize_q4(W, scale_dtype=torch.bfloat16)
    Wd = dequantize_q4(packed, scale).to(torch.bfloat16).float()       # the kernel rounds value * scale to bf16
    words = to_engine_order(packed).contiguous()
    rows = sum(counts)
    A = torch.randn(rows + 128, K, generator=g, device=dev).to(torch.bfloat16)
    tiles, r0 = [], 0
    for e, n in enumerate(counts):
        for t in range(0, n, 128):
            tiles.append([r0 + t, min(128, n - t), e * Nw, 0])
        r0 += n
    tiles.append([0, 0, 0, 0])                                   # an unused entry
    tt = torch.tensor(tiles, dtype=torch.int32, device=dev)
    out = torch.full((rows + 128, Nw), 768.0, dtype=out_dtype, device=dev)
    P = lambda t: C.c_void_p(t.data_ptr())
    rc = L.qwk_gemm_q4_tc_grouped(P(A), P(words), P(scale), P(out), P(tt), len(tiles), rows, E * Nw, Nw, K, K, Nw,
                                  1 if out_dtype == torch.bfloat16 else 0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.all(out[rows:].float() == 768.0)
    r0 = 0
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    for e, n in enumerate(counts):
        if n:
            ref = A[r0:r0 + n].float() @ Wd[e * Nw:(e + 1) * Nw].float().T
            err = float((out[r0:r0 + n].float() - ref).abs().max() / ref.abs().max())
            assert err < tol, (e, err)
        r0 += n


@pytest.mark.parametrize("T,N,K,ks", [(200, 324, 10240, 3), (128, 128, 256, 2), (77, 40, 640, 1)])
def test_gemm_tc_split_k_partials_add_up(T, N, K, ks):
    """Split-K form: the partial products of the shares of K, added in order, equal the full product."""
    import ctypes as C
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    g = torch.Generator(device="cuda").manual_seed(T + N + K)
    A = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    ldc = (N + 7) // 8 * 8
    out = torch.full((ks, T + 3, ldc), 768.0, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    rc = L.qwk_gemm_bf16_tc_splitk(P(A), P(W), P(out), T, N, K, K, K, ldc, ks, (T + 3) * ldc,
                                   C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.all(out[:, T:] == 768.0) and torch.all(out[:, :, N:] == 768.0)
    ref = A.float() @ W.float().T
    got = out[:, :T, :N].sum(0)
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < 2e-3, err


@pytest.mark.parametrize("T,N,K", [(1024, 2048, 256), (1500, 512, 192), (4096, 2560, 1536)])      # the last: the out projection of a chunk on 4 ranks (CTA-pair form)
def test_gemm_tc_reduce_scatter_epilogue_on_emulated_ranks(T, N, K):
    """The tensor-parallel forms of the product on four ranks emulated on one GPU: with the reduce-scatter epilogue every
    rank's tiles land in the column owner's receive buffer and the owners' rank-order sums equal the sum of the full
    products; with the all-reduce epilogue every rank receives every part.  (2048 columns: the 256-wide tile form.)"""
    import ctypes as C
    from qwb200.models.config import ModelConfig
    from qwb200.ops import lib as qlib, structs as S
    from qwb200.parallel import tp_channel
    L = qlib.load(True)
    dev = torch.device("cuda:0")
    R = 4
    cfg = ModelConfig.tiny(hidden=N)
    chans = tp_channel.make_emulated(cfg, R, T, dev, mtp=False)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda").manual_seed(N + K)
    A = [torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16) for _ in range(R)]
    W = [(torch.randn(N, K, generator=g, device=dev) * 0.05).to(torch.bfloat16) for _ in range(R)]
    full = [a.float() @ w.float().T for a, w in zip(A, W)]
    for r in range(R):
        assert L.qwk_gemm_bf16_tc_tp(chans[r].ptr, P(A[r]), P(W[r]), None, T, N, K, K, K, N, 0, -1, 2, S.TP_RS, 0, s) == 0
    SH = N // R
    outs = [torch.zeros(T, SH, device=dev) for _ in range(R)]
    for r in range(R):
        assert L.qwk_tp_reduce(chans[r].ptr, S.TP_RS, P(outs[r]), T * SH, s) == 0
    torch.cuda.synchronize()
    want = sum(full)
    for r in range(R):
        err = float((outs[r] - want[:, r * SH:(r + 1) * SH]).abs().max() / want.abs().max())
        assert err < 2e-3, (r, err)


@pytest.fixture
def pair_form():
    """Switch the CTA-pair form of the dense kernel on for products at least 256 columns wide, and off again."""
    import ctypes as C
    from qwb200.ops import lib as qlib
    L = qlib.load(True)
    old = L.qwk_gemm_tc_pair_min_n(256)
    word = torch.zeros(2, dtype=torch.int32, device="cuda")           # bounded waits that run out report here
    L.qwk_set_error_word(C.c_void_p(word.data_ptr()))
    yield word
    torch.cuda.synchronize()
    L.qwk_set_error_word(None)
    L.qwk_gemm_tc_pair_min_n(old)


@pytest.mark.parametrize("T,N,K", [(256, 256, 64), (512, 512, 256), (4096, 2560, 640), (300, 700, 192), (1111, 1536, 128), (2048, 13952, 320)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_pair_form_matches_fp32(pair_form, T, N, K, out_dtype):
    """256 x 256 tiles computed by two CTAs with tcgen05.mma.cta_group::2, ragged rows and columns included; a run whose
    barriers did not meet would end with the error word set, which is checked too."""
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(T + N + K + 1)
    A = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    ldc = (N + 7) // 8 * 8 + 8
    out = torch.full((T + 3, ldc), 768.0, dtype=out_dtype, device="cuda")      # guard columns and rows detect stray writes
    K_.gemm_bf16_tc(A, W, out=out[:T, :N])
    torch.cuda.synchronize()
    assert pair_form.tolist() == [0, 0]
    ref = A.float() @ W.float().T
    assert torch.all(out[:, N:].float() == 768.0) and torch.all(out[T:].float() == 768.0)
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    err = float((out[:T, :N].float() - ref).abs().max() / ref.abs().max())
    assert err < tol, err


def test_gemm_tc_pair_form_reduce_scatter_on_emulated_ranks(pair_form):
    test_gemm_tc_reduce_scatter_epilogue_on_emulated_ranks(1024, 2048, 256)
