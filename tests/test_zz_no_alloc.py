"""mg_matmul_static_ws: the GEMM entry point for callers that cannot allocate device memory
(a host whose own pool already holds all free HBM, a plugin callback that must not allocate).
It keeps its scratch in an array inside the library.  The test drives it through the C ABI and
requires the same bytes as mg_matmul with a caller-provided workspace, on two calls in a row
that share the array, the second with a different shape so that leftovers of the first would
show.  Collected last on purpose: a run that stops at the first failure has by then run every
other test."""
import ctypes

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _operands(M, N, split, seed):
    import mixedgemm_b200 as mg
    KN, KS, KO = split
    K = sum(split)
    X = H.make_x(M, K, seed=seed)
    W = H.make_w(N, K, seed=seed + 1)
    idx = H.reorder_index(X).cuda()
    # the reference's dense layout: these are the buffers that need the padded copy, i.e. scratch
    A = mg.reorder_quantize_x(X.cuda(), idx, KN, KS, KO, M, N, out=mg.alloc_quantized_x(M, KN, KS, KO, "cuda", padded=False))
    B = mg.reorder_quantize_w(W.cuda(), idx, KN, KS, KO, M, N, out=mg.alloc_quantized_w(N, KN, KS, KO, "cuda", padded=False))
    return A, B


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(lib, A, B, M, N, split):
    KN, KS, KO = split
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ops = [_ptr(A[0]), _ptr(B[0]), _ptr(A[1]), _ptr(B[1]), _ptr(A[2]), _ptr(B[2])]
    sfs = [_ptr(A[3]), _ptr(B[3]), _ptr(A[4]), _ptr(B[4]), _ptr(A[5]), _ptr(B[5])]
    need = lib.mg_matmul_workspace_bytes(M, N, KN, KS, KO)
    assert 0 < need <= 24 << 20
    buf = torch.empty(need + 1024, dtype=torch.uint8, device="cuda")
    ws = buf.data_ptr() + (-buf.data_ptr()) % 1024
    D_ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    D_new = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    st = lib.mg_matmul(*ops, M, N, KN, KS, KO, None, _ptr(D_ref), N, *sfs, ctypes.c_void_p(ws), need, stream)
    assert st == 0, st
    st = lib.mg_matmul_static_ws(*ops, M, N, KN, KS, KO, None, _ptr(D_new), N, *sfs, stream)
    assert st == 0, st
    torch.cuda.synchronize()
    assert not torch.isnan(D_new.float()).any()
    # same kernels on the same operands: the results must be the same bytes
    assert torch.equal(D_ref.view(torch.int16), D_new.view(torch.int16))


def test_static_workspace_matches_caller_workspace_twice():
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    first = (200, 256, (8960, 4928, 448))   # both tails padded: 4928 -> 4992, 448 -> 512
    second = (130, 128, (256, 192, 64))     # smaller problem on top of the first call's leftovers
    for M, N, split in (first, second):
        A, B = _operands(M, N, split, seed=M)
        _both(lib, A, B, M, N, split)
    assert mg.device_status() == 0


def test_refuses_problems_beyond_the_built_in_scratch():
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    M, N, split = 16384, 16384, (8960, 4928, 448)
    assert lib.mg_matmul_workspace_bytes(M, N, *split) > 24 << 20
    # refused before any pointer is looked at and before anything is launched
    st = lib.mg_matmul_static_ws(*[None] * 6, M, N, *split, None, None, N, *[None] * 6, None)
    assert st == 4
    assert b"workspace" in lib.mg_strerror(st)
