"""The entry point that allocates nothing, called through its exported C symbol.

Some callers of the CUDA library cannot allocate device memory: a plugin inside an application whose
allocator owns the whole GPU, code in a region where cudaMalloc is forbidden or would stall, or an embedder
without PyTorch's allocator to lend a workspace.  For them ``hfb_linear_tc_noalloc`` keeps the split-K partial
sums of the tensor-core product in an 8 MiB array built into the library.  This test calls it the way such a
caller would (ctypes, raw pointers, no wrapper of the package) and checks it against the regular entry
point ``hfb_linear_tc`` on two calls in a row, since the second call finds the first call's numbers in the
shared array.  It is collected last so that a run that stops at the first failure has run everything else.
"""
import ctypes
from ctypes import c_int, c_size_t, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from hfcpu_b200.kernels import build
    lib = ctypes.CDLL(build.build())
    lib.hfb_last_error.restype = ctypes.c_char_p
    lib.hfb_linear_tc_workspace.restype = c_size_t
    return lib


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def test_noalloc_linear_matches_the_regular_entry_point_twice():
    lib = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(0)
    # decode-like shapes that split K (partial sums in the built-in array), one that does not, one with many rows
    for M, N, K in ((8, 4608, 3584), (1, 3584, 18944), (64, 3584, 2048), (8, 37888, 512), (300, 1024, 256)):
        a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
        need = lib.hfb_linear_tc_workspace(c_int(M), c_int(N), c_int(K))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        want = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        rc = lib.hfb_linear_tc(_ptr(a), _ptr(w), _ptr(bias), c_int(1), _ptr(want), c_int(1), c_int(0), c_int(M), c_int(N),
                               c_int(K), _ptr(ws), c_size_t(need), stream)
        assert rc == 0, lib.hfb_last_error().decode()
        ref = a.double() @ w.double().T + bias.double()
        gots = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        torch.cuda.synchronize()
        free_before = None
        for call in range(2):
            got = gots[call]
            if call == 1:
                free_before = torch.cuda.mem_get_info()[0]      # the second call must leave the free memory as it is
            rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w), _ptr(bias), c_int(1), _ptr(got), c_int(1), c_int(0), c_int(M),
                                           c_int(N), c_int(K), stream)
            assert rc == 0, lib.hfb_last_error().decode()
            torch.cuda.synchronize()
            if call == 1:
                assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
            assert torch.equal(got, want), f"call {call} differs from hfb_linear_tc at {M}x{N}x{K}"
            err = float((got.double() - ref).abs().max() / ref.abs().max())
            assert err < 1e-2, err                      # the tolerance of the bfloat16 product tests
        # accumulate into a float32 output, as the residual stream does
        res = torch.randn(M, N, device="cuda", generator=g)
        res2 = res.clone()
        lib.hfb_linear_tc(_ptr(a), _ptr(w), None, c_int(0), _ptr(res), c_int(0), c_int(1), c_int(M), c_int(N), c_int(K),
                          _ptr(ws), c_size_t(need), stream)
        rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w), None, c_int(0), _ptr(res2), c_int(0), c_int(1), c_int(M), c_int(N),
                                       c_int(K), stream)
        assert rc == 0, lib.hfb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(res, res2)


def test_noalloc_linear_refuses_what_the_array_cannot_hold():
    lib = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    M, N, K = 128, 8192, 8192                           # 2 splits x 128 x 8192 floats = 8 MiB... plus one row more than fits
    need = lib.hfb_linear_tc_workspace(c_int(M), c_int(N), c_int(K))
    a = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w), None, c_int(0), _ptr(out), c_int(1), c_int(0), c_int(M), c_int(N),
                                   c_int(K), stream)
    if need > (8 << 20):
        assert rc == 4 and "built-in" in lib.hfb_last_error().decode()       # HFB_ERANGE, with both numbers
    else:
        assert rc == 0
    # (operands sized for the call, in case the split count of this GPU lets it run)
    w2 = torch.zeros(9000, 4096, device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros(128, 9000, device="cuda", dtype=torch.bfloat16)
    rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w2), None, c_int(0), _ptr(out2), c_int(1), c_int(0), c_int(128), c_int(9000),
                                   c_int(4096), stream)
    need2 = lib.hfb_linear_tc_workspace(c_int(128), c_int(9000), c_int(4096))
    assert (rc == 4) == (need2 > (8 << 20))
    # a bias that is not 16-byte aligned is refused before anything is launched
    bias = torch.zeros(9008, device="cuda", dtype=torch.bfloat16)[1:9001]
    rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w2), _ptr(bias), c_int(1), _ptr(out2), c_int(1), c_int(0), c_int(8), c_int(9000),
                                   c_int(4096), stream)
    assert rc == 2 and "aligned" in lib.hfb_last_error().decode()
    rc = lib.hfb_linear_tc_noalloc(_ptr(a), _ptr(w), None, c_int(0), _ptr(out), c_int(1), c_int(0), c_int(8), c_int(64),
                                   c_int(12), stream)
    assert rc == 2                                      # K not a multiple of 8: HFB_ENOTSUP, as the regular entry point
