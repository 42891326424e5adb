"""qwk_moe_router_static (ops/csrc/no_alloc.h) against qwk_moe_router: same inputs, caller-provided scratch on
one side, the library's fixed scratch on the other; two calls in a row with different inputs, bit-equal outputs.
Collected last (file name) so that it also runs after every other test has used the device."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from qwb200.ops import lib
    lib.load(True)
    L = C.CDLL(lib.LIB_PATH)
    P, I = C.c_void_p, C.c_int
    L.qwk_moe_router_static_setup.restype = I
    L.qwk_moe_router_static_setup.argtypes = []
    L.qwk_moe_router_static.restype = I
    L.qwk_moe_router_static.argtypes = [P, P, I, I, I, I, I, I, I, I, I, P, P, P, P]
    L.qwk_moe_router.restype = I
    L.qwk_moe_router.argtypes = [P, P, P, I, I, I, I, I, I, I, I, I, P, P, P, P, P, P, C.c_longlong, C.c_longlong, P]
    return L


def _case(seed, M, E, top_k, F, K, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    nrs = E + 1 + 2 * F
    W = (torch.randn(nrs, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    return W, x, nrs


def _outputs(M, top_k, F, dev):
    return (torch.full((M, top_k), -7, dtype=torch.int32, device=dev), torch.full((M, top_k), -1.0, device=dev),
            torch.zeros(M, F, dtype=torch.bfloat16, device=dev))


def test_router_static_equals_router_two_calls_in_a_row():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    L = _lib()
    assert L.qwk_moe_router_static_setup() == 0
    assert L.qwk_moe_router_static_setup() == 0          # idempotent
    s = torch.cuda.current_stream().cuda_stream
    E, top_k, F, K = 512, 10, 640, 2560
    first, n_local = 128, 256                             # a rank that owns experts 128..383
    results = []
    cases = [(1, 5), (2, 32)]                             # (seed, rows): a second call with other inputs and another size
    for seed, M in cases:
        W, x, nrs = _case(seed, M, E, top_k, F, K, dev)
        pe_a, pw_a, sh_a = _outputs(M, top_k, F, dev)
        pe_b, pw_b, sh_b = _outputs(M, top_k, F, dev)
        rs = torch.empty(M, nrs, device=dev)
        ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        assert L.qwk_moe_router(W.data_ptr(), x.data_ptr(), rs.data_ptr(), nrs, K, M, K, E, top_k, F, first, n_local,
                                pe_a.data_ptr(), pw_a.data_ptr(), sh_a.data_ptr(), ticket.data_ptr(), None, None, 0, 0, s) == 0
        results.append((W, x, M, pe_a, pw_a, sh_a, pe_b, pw_b, sh_b))
    # the two static calls back to back, no synchronisation between them
    for W, x, M, pe_a, pw_a, sh_a, pe_b, pw_b, sh_b in results:
        assert L.qwk_moe_router_static(W.data_ptr(), x.data_ptr(), E + 1 + 2 * F, K, M, K, E, top_k, F, first, n_local,
                                       pe_b.data_ptr(), pw_b.data_ptr(), sh_b.data_ptr(), s) == 0
    torch.cuda.synchronize()
    for W, x, M, pe_a, pw_a, sh_a, pe_b, pw_b, sh_b in results:
        assert torch.equal(pe_a, pe_b) and torch.equal(pw_a, pw_b) and torch.equal(sh_a, sh_b)
        assert int((pe_a >= 0).sum()) > 0 and int((pe_a == -7).sum()) == 0
        # and both agree with plain fp32 arithmetic on the expert choice
        logits = x.float() @ W.float().t()
        top = logits[:, :E].topk(top_k, dim=1).indices
        want = torch.where((top >= first) & (top < first + n_local), top - first, torch.full_like(top, -1))
        got = pe_b.long()
        agree = (want.sort(dim=1).values == got.sort(dim=1).values).float().mean().item()
        assert agree > 0.98          # ties at the cut may differ between bf16-accumulated and fp32 logits


def test_router_static_refuses_what_does_not_fit():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    L = _lib()
    W, x, nrs = _case(3, 4, 512, 10, 640, 2560, dev)
    pe, pw, sh = _outputs(4, 10, 640, dev)
    s = torch.cuda.current_stream().cuda_stream
    args = lambda M, n: (W.data_ptr(), x.data_ptr(), n, 2560, M, 2560, 512, 10, 640, 0, 512, pe.data_ptr(), pw.data_ptr(), sh.data_ptr(), s)
    assert L.qwk_moe_router_static(*args(33, nrs)) == -4
    assert L.qwk_moe_router_static(*args(4, 4097)) == -4
    assert L.qwk_moe_router_static(*args(0, nrs)) == -4
    # fewer outputs per row than the routing reads (512 logits + gate + 2 x 640 shared rows): refused as an unsupported shape
    assert L.qwk_moe_router_static(*args(4, 512 + 2 * 640)) == -1
    assert L.qwk_moe_router_static(*args(4, 511)) == -1
    torch.cuda.synchronize()
    assert int((pe == -7).sum()) == pe.numel()            # nothing was launched
