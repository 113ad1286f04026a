"""The no-allocation split-K GEMM entry point, called through its exported C symbol.

Collected last on purpose (file name): it has to give the same answer whether it runs alone or after every other GPU
test has used the library, and on two calls in a row (the scratch array is reused, nothing may leak between calls).
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 4 * 1024 * 1024


@pytest.fixture(scope="module")
def lib():
    from ronn_b200 import _native
    lib = _native.cuda()
    fn = lib.ronn_gemm_splitk_no_alloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 7 + [C.c_void_p, C.c_void_p]
    lib.ronn_no_alloc_scratch_floats.restype = C.c_long
    lib.ronn_no_alloc_scratch_floats.argtypes = [C.c_int] * 4
    lib.ronn_no_alloc_strerror.restype = C.c_char_p
    lib.ronn_no_alloc_strerror.argtypes = [C.c_int]
    return lib


def _call(lib, a, w, out, bias, res, splitk, status):
    M, K = a.shape
    N = w.shape[0]
    return lib.ronn_gemm_splitk_no_alloc(a.data_ptr(), w.data_ptr(), out.data_ptr(),
                                         None if bias is None else bias.data_ptr(),
                                         None if res is None else res.data_ptr(), M, N, K, a.stride(0), w.stride(0),
                                         0 if a.dtype == torch.bfloat16 else 1, splitk, status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K,S", [(256, 1024, 4096, 4), (96, 512, 2048, 8), (37, 136, 1024, 3)])
def test_matches_the_allocating_entry_point_twice_in_a_row(lib, M, N, K, S):
    from ronn_b200 import ops
    torch.manual_seed(M + N)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for call in range(2):                              # second call: fresh operands through the same scratch
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        bias = torch.randn(N, device="cuda").to(torch.bfloat16)
        res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
        out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        rc = _call(lib, a, w, out, bias, res, S, status)
        assert rc == 0, lib.ronn_no_alloc_strerror(rc)
        ws, s_eff = ops.gemm_splitk(a, w, S)           # existing entry point: torch-allocated workspace
        want, _ = ops.splitk_finalize(ws, s_eff, M, N, torch.bfloat16, bias=bias, residual=res)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert torch.equal(out, want), f"call {call}: max diff {(out.float() - want.float()).abs().max().item()}"
        ref = a.float() @ w.float().t() + bias.float() + res.float()
        torch.testing.assert_close(out.float(), ref, atol=0.2, rtol=2e-2)


def test_rejects_what_does_not_fit_the_scratch(lib):
    M, N, K, S = 1024, 4096, 4096, 4                   # 4 x 1024 x 4096 floats = 4x the capacity
    assert lib.ronn_no_alloc_scratch_floats(M, N, K, S) > MAX_FLOATS
    a = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = _call(lib, a, w, out, None, None, S, status)
    assert rc == -40
    assert b"exceeds the built-in scratch" in lib.ronn_no_alloc_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                    # nothing was launched
    # the largest case that still fits is accepted
    assert lib.ronn_no_alloc_scratch_floats(256, 4096, 4096, 4) == MAX_FLOATS
    a2 = torch.randn(256, 4096, device="cuda").to(torch.bfloat16)
    out2 = torch.empty(256, 4096, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, a2, w, out2, None, None, 4, status) == 0
    torch.cuda.synchronize()
    assert bool((out2 == 0).all())
    assert _call(lib, a2, w, out2, None, None, 0, status) == 0      # splitk < 1 means one slice
    assert lib.ronn_gemm_splitk_no_alloc(None, w.data_ptr(), out2.data_ptr(), None, None, 256, 4096, 4096, 4096, 4096,
                                         0, 4, None, None) == -42


def test_rejects_bad_shapes_before_anything_is_launched(lib):
    """N = 12 passes the GEMM's own check (multiples of 4) but not the reduction pass's (multiples of 8): the entry
    point refuses it up front, so neither the scratch nor `out` is touched.  The same goes for rows wider than the
    reduction pass keeps in registers and for unaligned K."""
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for (M, N, K) in [(64, 12, 256), (8, 32776, 64), (64, 64, 68)]:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
        rc = _call(lib, a, w, out, None, None, 2, status)
        assert rc == -43, (M, N, K, rc)
        assert b"multiple of 8" in lib.ronn_no_alloc_strerror(rc)
        torch.cuda.synchronize()
        assert bool((out == 7.0).all()) and status.tolist() == [0, 0, 0, 0]
