"""Host-side mirror of the reference's Python module (MixedGemm src/bindings.cpp:311-342):
the same three entry points with the same argument lists and returned shapes, on top of
the C ABI.  torch is used only to own device memory and to name the current stream.

Differences from the reference binding, all deliberate:
  * any K = KN + KS + KO with segments that are multiples of 32 is accepted for the two
    quantisers (the reference dispatches seven compile-time K values, bindings.cpp:95-168);
  * nothing synchronises the device or prints (bindings.cpp:51-65 does both);
  * scale buffers are sized for whole 512-byte atoms, which is never smaller than the
    reference's `(M/128+1)*128*K/32` except that it also covers segments that are not a
    multiple of 128;
  * errors surface as RuntimeError (MixedGemmError), as the reference's std::runtime_error do.
"""
import torch

from . import _capi


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def sf_bytes(rows, kseg):
    return _capi.load().mg_sf_bytes(rows, kseg)


def _check_in(X, reorder_index, KN, KS, KO, what):
    if not X.is_cuda or X.dtype != torch.bfloat16 or X.dim() != 2 or not X.is_contiguous():
        raise RuntimeError("%s: expected a contiguous 2-D CUDA bfloat16 tensor" % what)
    if not reorder_index.is_cuda or reorder_index.dtype != torch.int16 or not reorder_index.is_contiguous():
        raise RuntimeError("%s: reorder_index must be a contiguous CUDA int16 tensor" % what)
    if X.size(1) != KN + KS + KO or reorder_index.numel() != X.size(1):
        raise RuntimeError("%s: K = %d does not match KN+KS+KO or the index length" % (what, X.size(1)))


def alloc_quantized_x(M, KN, KS, KO, device):
    """Output buffers of reorder_quantize_x with the reference's shapes (bindings.cpp:88-93)."""
    lib = _capi.load()
    u8 = dict(dtype=torch.uint8, device=device)
    return (torch.empty((M, KN // 2), **u8), torch.empty((M, KS // 4 * 3), **u8), torch.empty((M, KO), **u8)) + tuple(
        torch.empty(max(lib.mg_sf_bytes(M, k), (M // 128 + 1) * 128 * k // 32), **u8) for k in (KN, KS, KO))


def alloc_quantized_w(N, KN, KS, KO, device):
    """Output buffers of reorder_quantize_w (bindings.cpp:207-212)."""
    lib = _capi.load()
    u8 = dict(dtype=torch.uint8, device=device)
    return (torch.empty((N, KN // 2), **u8), torch.empty((N, KS // 2), **u8), torch.empty((N, KO // 2), **u8)) + tuple(
        torch.empty(max(lib.mg_sf_bytes(N, k), N * k // 32), **u8) for k in (KN, KS, KO))


def reorder_quantize_x(X, reorder_index, KN, KS, KO, seqlen=None, outfeatures=None, out=None):
    """bindings.cpp:69-186.  Returns (XN[M,KN/2], XS[M,3KS/4], XO[M,KO], SFXN, SFXS, SFXO), all uint8.
    `seqlen` / `outfeatures` are accepted and ignored, as in the reference.  `out` may pass the
    six buffers of alloc_quantized_x() to write into."""
    _check_in(X, reorder_index, KN, KS, KO, "reorder_quantize_x")
    lib = _capi.load()
    M = X.size(0)
    dev = X.device
    XN, XS, XO, *sfs = out if out is not None else alloc_quantized_x(M, KN, KS, KO, dev)
    with torch.cuda.device(dev):
        st = lib.mg_reorder_quantize_x(_ptr(X), M, X.size(1), _ptr(reorder_index), KN, KS, KO, _ptr(XN), _ptr(XS),
                                       _ptr(XO), _ptr(sfs[0]), _ptr(sfs[1]), _ptr(sfs[2]), _stream())
    _capi.check(st, "reorder_quantize_x")
    return XN, XS, XO, sfs[0], sfs[1], sfs[2]


def reorder_quantize_w(W, reorder_index, KN, KS, KO, seqlen=None, outfeatures=None, out=None):
    """bindings.cpp:188-305.  Returns (WN[N,KN/2], WS[N,KS/2], WO[N,KO/2], SFWN, SFWS, SFWO), all uint8."""
    _check_in(W, reorder_index, KN, KS, KO, "reorder_quantize_w")
    lib = _capi.load()
    N = W.size(0)
    dev = W.device
    WN, WS, WO, *sfs = out if out is not None else alloc_quantized_w(N, KN, KS, KO, dev)
    with torch.cuda.device(dev):
        st = lib.mg_reorder_quantize_w(_ptr(W), N, W.size(1), _ptr(reorder_index), KN, KS, KO, _ptr(WN), _ptr(WS),
                                       _ptr(WO), _ptr(sfs[0]), _ptr(sfs[1]), _ptr(sfs[2]), _stream())
    _capi.check(st, "reorder_quantize_w")
    return WN, WS, WO, sfs[0], sfs[1], sfs[2]


_workspaces = {}


def _workspace(dev, nbytes):
    """One growing scratch buffer per device (torch's caching allocator hands out 512-byte
    aligned blocks; the kernel wants 1024, so over-allocate and slice)."""
    if nbytes == 0:
        return None, 0
    key = (dev.type, dev.index)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes + 1024:
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf.data_ptr() + off, nbytes


def matmul(AN, BN, AS, BS, AO, BO, SFAN, SFBN, SFAS, SFBS, SFAO, SFBO, out=None, C=None, out_dtype=None):
    """bindings.cpp:9-67: returns a new [M,N] bfloat16 tensor = A @ B^T over the three segments.
    `out` (optional) receives the result instead; `C` (optional, bf16 [M,N]) is added before
    the single final rounding; `out_dtype=torch.float32` returns the unrounded accumulator."""
    lib = _capi.load()
    M, N = AN.size(0), BN.size(0)
    KN, KS, KO = AN.size(1) * 2, AS.size(1) * 4 // 3, AO.size(1)
    for t in (AN, BN, AS, BS, AO, BO, SFAN, SFBN, SFAS, SFBS, SFAO, SFBO):
        if not t.is_cuda or t.dtype != torch.uint8 or not t.is_contiguous():
            raise RuntimeError("matmul: operands must be contiguous CUDA uint8 tensors")
    dev = AN.device
    dt = out.dtype if out is not None else (out_dtype or torch.bfloat16)
    if dt not in (torch.bfloat16, torch.float32):
        raise RuntimeError("matmul: output dtype must be bfloat16 or float32")
    D = out if out is not None else torch.empty((M, N), dtype=dt, device=dev)
    if D.size(0) != M or D.size(1) != N or D.stride(1) != 1:
        raise RuntimeError("matmul: out must be [M,N] with unit column stride")
    fn = lib.mg_matmul if dt == torch.bfloat16 else lib.mg_matmul_f32
    with torch.cuda.device(dev):
        ws, wsb = _workspace(dev, lib.mg_matmul_workspace_bytes(M, N, KN, KS, KO))
        st = fn(_ptr(AN), _ptr(BN), _ptr(AS), _ptr(BS), _ptr(AO), _ptr(BO), M, N, KN, KS, KO,
                           _ptr(C), _ptr(D), D.stride(0), _ptr(SFAN), _ptr(SFBN), _ptr(SFAS), _ptr(SFBS),
                           _ptr(SFAO), _ptr(SFBO), ws, wsb, _stream())
    _capi.check(st, "matmul")
    return D


def device_status():
    """Reads and clears the device error word (non-zero after a kernel gave up on a wait)."""
    import ctypes
    lib = _capi.load()
    v = ctypes.c_int(0)
    _capi.check(lib.mg_device_status(ctypes.byref(v), _stream()), "device_status")
    return v.value


def test_function():
    """bindings.cpp:329."""
    return "Hello from test_function!"
