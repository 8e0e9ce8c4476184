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


def _alloc_codes(rows, logical, pitch, device):
    """[rows, logical] uint8 view of a buffer whose rows are `pitch` bytes apart."""
    buf = torch.empty((rows, pitch), dtype=torch.uint8, device=device)
    return buf[:, :logical] if pitch != logical else buf


def alloc_quantized_x(M, KN, KS, KO, device, padded=True, one_buffer=False):
    """Output buffers of reorder_quantize_x with the reference's shapes (bindings.cpp:88-93).
    With padded=True the code tensors are row-pitched views (same shape, same contents) whose pitch
    the GEMM can read in place even when a segment is only a multiple of 64.  With one_buffer=True
    all six are carved out of a single allocation, so that one transfer moves them together."""
    lib = _capi.load()
    u8 = dict(dtype=torch.uint8, device=device)
    logical = (KN // 2, KS // 4 * 3, KO)
    pitch = [lib.mg_code_pitch(0, i, k) if padded else l for i, (k, l) in enumerate(zip((KN, KS, KO), logical))]
    sf_len = [max(lib.mg_sf_bytes(M, k), (M // 128 + 1) * 128 * k // 32) for k in (KN, KS, KO)]
    if not one_buffer:
        return tuple(_alloc_codes(M, l, p, device) for l, p in zip(logical, pitch)) + tuple(
            torch.empty(n, **u8) for n in sf_len)
    sizes = [M * p for p in pitch] + sf_len
    offs, off = [], 0
    for n in sizes:
        offs.append(off)
        off += (n + 1023) // 1024 * 1024
    buf = torch.empty(off + 1024, **u8)
    base = (-buf.data_ptr()) % 1024
    out = []
    for i in range(3):
        v = buf[base + offs[i]: base + offs[i] + sizes[i]].view(M, pitch[i])
        out.append(v[:, :logical[i]] if pitch[i] != logical[i] else v)
    for i in range(3):
        out.append(buf[base + offs[3 + i]: base + offs[3 + i] + sizes[3 + i]])
    return tuple(out)


def alloc_quantized_w(N, KN, KS, KO, device, padded=True):
    """Output buffers of reorder_quantize_w (bindings.cpp:207-212); see alloc_quantized_x."""
    lib = _capi.load()
    u8 = dict(dtype=torch.uint8, device=device)
    logical = (KN // 2, KS // 2, KO // 2)
    pitch = [lib.mg_code_pitch(1, i, k) if padded else l for i, (k, l) in enumerate(zip((KN, KS, KO), logical))]
    return tuple(_alloc_codes(N, l, p, device) for l, p in zip(logical, pitch)) + tuple(
        torch.empty(max(lib.mg_sf_bytes(N, k), N * k // 32), **u8) for k in (KN, KS, KO))


def _pitches(tensors):
    import ctypes
    return (ctypes.c_size_t * len(tensors))(*[t.stride(0) if t.size(1) else 0 for t in tensors])


def _check_codes(tensors, what):
    for t in tensors:
        if not t.is_cuda or t.dtype != torch.uint8 or t.dim() != 2 or (t.size(1) and t.stride(1) != 1):
            raise RuntimeError("%s: code tensors must be 2-D CUDA uint8 with unit column stride" % what)


def _check_operands(A, B, what):
    """A = (AN, AS, AO, SFAN, SFAS, SFAO), B likewise for the weights.  The reference infers M, N and
    the K split from AN, BN, AS and AO alone (bindings.cpp:30-34); the kernels build tensor maps and
    whole-atom scale copies from those sizes, so every other tensor is held to them here."""
    lib = _capi.load()
    _check_codes(tuple(A[:3]) + tuple(B[:3]), what)
    M, N = A[0].size(0), B[0].size(0)
    KN, KS, KO = A[0].size(1) * 2, A[1].size(1) * 4 // 3, A[2].size(1)
    if A[1].size(0) != M or A[2].size(0) != M or B[1].size(0) != N or B[2].size(0) != N:
        raise RuntimeError("%s: the three code tensors of an operand must have the same row count" % what)
    if A[1].size(1) * 4 != KS * 3 or B[0].size(1) * 2 != KN or B[1].size(1) * 2 != KS or B[2].size(1) * 2 != KO:
        raise RuntimeError("%s: code widths of the two operands do not describe the same K split" % what)
    dev = A[0].device
    for t, rows, k in ((A[3], M, KN), (A[4], M, KS), (A[5], M, KO), (B[3], N, KN), (B[4], N, KS), (B[5], N, KO)):
        if not t.is_cuda or t.dtype != torch.uint8 or not t.is_contiguous():
            raise RuntimeError("%s: scale tensors must be contiguous CUDA uint8 tensors" % what)
        if t.numel() < lib.mg_sf_bytes(rows, k):
            raise RuntimeError("%s: a scale tensor holds %d bytes, %d are read (whole 512-byte atoms)" % (
                what, t.numel(), lib.mg_sf_bytes(rows, k)))
    for t in tuple(A) + tuple(B):
        if t.device != dev:
            raise RuntimeError("%s: all operands must be on one device" % what)
    return M, N, KN, KS, KO


def reorder_quantize_x(X, reorder_index, KN, KS, KO, seqlen=None, outfeatures=None, out=None):
    """bindings.cpp:69-186.  Returns (XN[M,KN/2], XS[M,3KS/4], XO[M,KO], SFXN, SFXS, SFXO), all uint8.
    `seqlen` / `outfeatures` are accepted and ignored, as in the reference.  `out` may pass the
    six buffers of alloc_quantized_x() to write into."""
    _check_in(X, reorder_index, KN, KS, KO, "reorder_quantize_x")
    lib = _capi.load()
    M = X.size(0)
    dev = X.device
    XN, XS, XO, *sfs = out if out is not None else alloc_quantized_x(M, KN, KS, KO, dev)
    _check_codes((XN, XS, XO), "reorder_quantize_x")
    with torch.cuda.device(dev):
        st = lib.mg_reorder_quantize_pitched(0, _ptr(X), M, X.size(1), _ptr(reorder_index), KN, KS, KO, _ptr(XN),
                                             _ptr(XS), _ptr(XO), _pitches((XN, XS, XO)), _ptr(sfs[0]), _ptr(sfs[1]),
                                             _ptr(sfs[2]), _stream())
    _capi.check(st, "reorder_quantize_x")
    return XN, XS, XO, sfs[0], sfs[1], sfs[2]


def reorder_quantize_x_multi(problems):
    """One launch for up to eight activations: problems = [(X, reorder_index, KN, KS, KO, out), ...]
    with `out` the six buffers to write (alloc_quantized_x) or None.  Every entry gives the bytes of
    its own reorder_quantize_x call; the CTAs are shared out in proportion to the sizes
    (mg_reorder_quantize_multi).  Returns the list of six-tuples."""
    import ctypes
    lib = _capi.load()
    n = len(problems)
    if not 1 <= n <= 8:
        raise RuntimeError("reorder_quantize_x_multi: 1 to 8 problems per launch")
    arr = (_capi.QuantProblem * n)()
    outs = []
    dev = problems[0][0].device
    for j, (X, idx, KN, KS, KO, out) in enumerate(problems):
        _check_in(X, idx, KN, KS, KO, "reorder_quantize_x_multi")
        if X.device != dev:
            raise RuntimeError("reorder_quantize_x_multi: all problems must be on one device")
        M = X.size(0)
        XN, XS, XO, *sfs = out if out is not None else alloc_quantized_x(M, KN, KS, KO, dev)
        _check_codes((XN, XS, XO), "reorder_quantize_x_multi")
        for t, k in zip(sfs, (KN, KS, KO)):
            if t.numel() < lib.mg_sf_bytes(M, k) or t.device != dev or t.dtype != torch.uint8:
                raise RuntimeError("reorder_quantize_x_multi: a scale buffer is too small or on another device")
        q = arr[j]
        q.X, q.rows, q.K, q.idx = _ptr(X), M, X.size(1), _ptr(idx)
        q.KN, q.KS, q.KO = KN, KS, KO
        q.C4, q.C6, q.C8 = _ptr(XN), _ptr(XS), _ptr(XO)
        for i, t in enumerate((XN, XS, XO)):
            q.pitch[i] = t.stride(0) if t.size(1) else 0
        q.SF4, q.SF6, q.SF8 = _ptr(sfs[0]), _ptr(sfs[1]), _ptr(sfs[2])
        outs.append((XN, XS, XO, sfs[0], sfs[1], sfs[2]))
    with torch.cuda.device(dev):
        st = lib.mg_reorder_quantize_multi(0, n, ctypes.cast(arr, ctypes.c_void_p), _stream())
    _capi.check(st, "reorder_quantize_x_multi")
    return outs


def reorder_quantize_w(W, reorder_index, KN, KS, KO, seqlen=None, outfeatures=None, out=None):
    """bindings.cpp:188-305.  Returns (WN[N,KN/2], WS[N,KS/2], WO[N,KO/2], SFWN, SFWS, SFWO), all uint8."""
    _check_in(W, reorder_index, KN, KS, KO, "reorder_quantize_w")
    lib = _capi.load()
    N = W.size(0)
    dev = W.device
    WN, WS, WO, *sfs = out if out is not None else alloc_quantized_w(N, KN, KS, KO, dev)
    _check_codes((WN, WS, WO), "reorder_quantize_w")
    with torch.cuda.device(dev):
        st = lib.mg_reorder_quantize_pitched(1, _ptr(W), N, W.size(1), _ptr(reorder_index), KN, KS, KO, _ptr(WN),
                                             _ptr(WS), _ptr(WO), _pitches((WN, WS, WO)), _ptr(sfs[0]), _ptr(sfs[1]),
                                             _ptr(sfs[2]), _stream())
    _capi.check(st, "reorder_quantize_w")
    return WN, WS, WO, sfs[0], sfs[1], sfs[2]


_workspaces = {}  # (device type, device index, stream) -> scratch buffer in use
_retired = []     # superseded buffers, kept alive: captured graphs and queued kernels hold their addresses


def _workspace(dev, nbytes):
    """Scratch for the call being issued: one buffer per (device, stream), because the split-K
    counters and partials in it must not be shared by kernels that may run at the same time, grown
    when a call needs more.  A buffer that has been handed out is never freed - a captured CUDA graph
    replays with the address it was captured with - and growing is refused while the stream is
    capturing: run the largest shape once before capturing.  (torch's caching allocator hands out
    512-byte aligned blocks; the kernels want 1024, so over-allocate and slice.)"""
    if nbytes == 0:
        return None, 0
    key = (dev.type, dev.index, torch.cuda.current_stream(dev).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes + 1024:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("mixedgemm: the scratch buffer of this stream would have to grow during stream capture; "
                               "run the largest shape once on this stream before capturing")
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf.data_ptr() + off, nbytes


def matmul(AN, BN, AS, BS, AO, BO, SFAN, SFBN, SFAS, SFBS, SFAO, SFBO, out=None, C=None, out_dtype=None):
    """bindings.cpp:9-67: returns a new [M,N] bfloat16 tensor = A @ B^T over the three segments.
    `out` (optional) receives the result instead; `C` (optional, bf16 [M,N]) is added before
    the single final rounding; `out_dtype=torch.float32` returns the unrounded accumulator."""
    lib = _capi.load()
    M, N, KN, KS, KO = _check_operands((AN, AS, AO, SFAN, SFAS, SFAO), (BN, BS, BO, SFBN, SFBS, SFBO), "matmul")
    dev = AN.device
    dt = out.dtype if out is not None else (out_dtype or torch.bfloat16)
    if dt not in (torch.bfloat16, torch.float32):
        raise RuntimeError("matmul: output dtype must be bfloat16 or float32")
    D = out if out is not None else torch.empty((M, N), dtype=dt, device=dev)
    if D.dim() != 2 or D.size(0) != M or D.size(1) != N or D.stride(1) != 1 or D.device != dev:
        raise RuntimeError("matmul: out must be [M,N] on the operands' device with unit column stride")
    if C is not None and (C.dtype != torch.bfloat16 or tuple(C.shape) != (M, N) or C.device != dev or
                          C.stride(1) != 1 or C.stride(0) != D.stride(0)):
        raise RuntimeError("matmul: C must be bf16 [M,N] on the operands' device with out's row pitch")
    pitches = _pitches((AN, BN, AS, BS, AO, BO))
    with torch.cuda.device(dev):
        ws, wsb = _workspace(dev, lib.mg_matmul_pitched_workspace_bytes(M, N, KN, KS, KO, pitches))
        st = lib.mg_matmul_pitched(_ptr(AN), _ptr(BN), _ptr(AS), _ptr(BS), _ptr(AO), _ptr(BO), pitches,
                                   int(dt == torch.float32), M, N, KN, KS, KO, _ptr(C), _ptr(D), D.stride(0),
                                   _ptr(SFAN), _ptr(SFBN), _ptr(SFAS), _ptr(SFBS), _ptr(SFAO), _ptr(SFBO), ws, wsb,
                                   _stream())
    _capi.check(st, "matmul")
    return D


def reorder_index(X, return_absmax=False):
    """Stable ascending argsort of the per-channel absmax of X [M,K] bf16 -> int16 [K]
    (what main.py:31-33 sketches with torch.max / torch.sort), computed by the library's kernels."""
    if not X.is_cuda or X.dtype != torch.bfloat16 or X.dim() != 2 or not X.is_contiguous():
        raise RuntimeError("reorder_index: expected a contiguous 2-D CUDA bfloat16 tensor")
    lib = _capi.load()
    M, K = X.shape
    idx = torch.empty(K, dtype=torch.int16, device=X.device)
    amax = torch.empty(K, dtype=torch.int16, device=X.device)
    with torch.cuda.device(X.device):
        st = lib.mg_reorder_index(_ptr(X), M, K, _ptr(idx), _ptr(amax), _stream())
    _capi.check(st, "reorder_index")
    return (idx, amax.view(torch.bfloat16)) if return_absmax else idx


def matmul_group(A, Bs, outs=None):
    """Products of one quantised activation A = (AN, AS, AO, SFAN, SFAS, SFAO) with several quantised
    weights Bs = [(BN, BS, BO, SFBN, SFBS, SFBO), ...] (q/k/v, gate/up) in one launch where the
    grouped kernel applies, otherwise one matmul per weight.  Returns the list of [M, N_j] bf16 tensors."""
    import ctypes
    lib = _capi.load()
    M = A[0].size(0)
    KN, KS, KO = A[0].size(1) * 2, A[1].size(1) * 4 // 3, A[2].size(1)
    dev = A[0].device
    n = len(Bs)
    Ns = [B[0].size(0) for B in Bs]
    if outs is None:
        outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for N in Ns]
    st = 1
    for B in Bs:
        _check_operands(A, B, "matmul_group")
    if 1 <= n <= 8 and all(o.dtype == torch.bfloat16 and o.stride(1) == 1 for o in outs):
        vp = lambda ts: (ctypes.c_void_p * n)(*[_ptr(t) for t in ts])
        pb = (ctypes.c_size_t * (3 * n))(*[B[s].stride(0) if B[s].size(1) else 0 for B in Bs for s in range(3)])
        with torch.cuda.device(dev):
            ws, wsb = None, 0
            st = lib.mg_matmul_group_pitched(
                n, _ptr(A[0]), _ptr(A[1]), _ptr(A[2]), _pitches(A[:3]), vp([B[0] for B in Bs]),
                vp([B[1] for B in Bs]), vp([B[2] for B in Bs]), pb, M, (ctypes.c_int * n)(*Ns), KN, KS, KO, vp(outs),
                (ctypes.c_int * n)(*[o.stride(0) for o in outs]), _ptr(A[3]), _ptr(A[4]), _ptr(A[5]),
                vp([B[3] for B in Bs]), vp([B[4] for B in Bs]), vp([B[5] for B in Bs]), ws, wsb, _stream())
    if st in (1, 3):  # shape or pitch the grouped kernel does not take: one launch per weight
        for B, o in zip(Bs, outs):
            matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5], out=o)
    else:
        _capi.check(st, "matmul_group")
    return outs


class ShardedActivation:
    """A quantised activation stored in row shards: `shards` = one (AN, AS, AO, SFAN, SFAS, SFAO) per
    shard, every shard with the same (multiple of 128) row count and the same shapes, and every one of
    the six tensors a constant number of bytes after its counterpart in the shard before
    (mg_problem_t.a_shard_rows).  It is how a multi-GPU exchange lays the activation out, so that a
    rank's rows of all six tensors are one contiguous block; matmul_multi takes it in place of A."""

    def __init__(self, shards):
        shards = [tuple(s) for s in shards]
        if not shards or any(len(s) != 6 for s in shards):
            raise RuntimeError("ShardedActivation: one six-tuple per shard")
        first = shards[0]
        rows = first[0].size(0)
        if len(shards) > 1 and rows % 128 != 0:
            raise RuntimeError("ShardedActivation: shards must be whole 128-row scale blocks")
        self.stride = [0] * 6
        for i in range(6):
            step = shards[1][i].data_ptr() - first[i].data_ptr() if len(shards) > 1 else 0
            for j, s in enumerate(shards):
                if (s[i].shape != first[i].shape or s[i].stride() != first[i].stride() or s[i].dtype != first[i].dtype
                        or s[i].device != first[i].device or s[i].data_ptr() != first[i].data_ptr() + j * step):
                    raise RuntimeError("ShardedActivation: shards must be equal and equally spaced in memory")
            self.stride[i] = step
        if len(shards) > 1 and any(self.stride[i] <= 0 for i in range(6) if first[i].numel()):
            raise RuntimeError("ShardedActivation: shards must follow one another in memory")
        self.shards, self.shard_rows, self.rows = shards, rows, rows * len(shards)


def matmul_multi(problems, flags=None):
    """One launch for a list of independent products (up to 8): problems = [(A, B, out), ...] with
    A = (AN, AS, AO, SFAN, SFAS, SFAO) or a ShardedActivation, B likewise for the weights, out a
    [M, N] bf16 tensor or None.  Each problem has its own activation and K split, unlike matmul_group.  `flags` (optional) gives
    per problem None or (int32 CUDA tensor, value or int32 CUDA tensor holding the value[, rows per flag, first row]): the kernel
    reads that problem's activation only once every flag has reached the value
    (mg_problem_t.ready_flags).  Problems the
    CTA-pair kernel does not take (M <= 128, N not a multiple of 256, buffers that need the padded
    copy) fall back to one matmul per problem; flags are then refused.  Returns the outputs."""
    import ctypes
    lib = _capi.load()
    n = len(problems)
    outs = []
    arr = (_capi.Problem * max(n, 1))()
    sharded = [A if isinstance(A, ShardedActivation) else None for A, _, _ in problems]
    problems = [(A.shards[0] if isinstance(A, ShardedActivation) else A, B, out) for A, B, out in problems]
    dev = problems[0][0][0].device
    for j, (A, B, out) in enumerate(problems):
        M, N, KN, KS, KO = _check_operands(A, B, "matmul_multi")
        if sharded[j] is not None and len(sharded[j].shards) > 1:
            M = sharded[j].rows
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or out.stride(1) != 1 or out.device != dev:
            raise RuntimeError("matmul_multi: outputs must be bf16 [M,N] on the operands' device with unit column stride")
        outs.append(out)
        q = arr[j]
        for name, t in zip(("AN", "AS", "AO", "SFAN", "SFAS", "SFAO"), A):
            setattr(q, name, _ptr(t))
        for name, t in zip(("BN", "BS", "BO", "SFBN", "SFBS", "SFBO"), B):
            setattr(q, name, _ptr(t))
        for i in range(3):
            q.pitch_a[i] = A[i].stride(0) if A[i].size(1) else 0
            q.pitch_b[i] = B[i].stride(0) if B[i].size(1) else 0
        q.M, q.N, q.KN, q.KS, q.KO = M, N, KN, KS, KO
        q.D_bf16, q.ldd = _ptr(out), out.stride(0)
        if sharded[j] is not None and len(sharded[j].shards) > 1:
            q.a_shard_rows = sharded[j].shard_rows
            for i in range(3):
                q.a_shard_stride[i] = sharded[j].stride[i]
                q.sfa_shard_stride[i] = sharded[j].stride[3 + i]
        f = flags[j] if flags is not None else None
        if f is not None:
            ft, fv = f[0], f[1]
            q.ready_rows = int(f[2]) if len(f) > 2 else 0
            q.first_row = int(f[3]) if len(f) > 3 else 0
            if not ft.is_cuda or ft.dtype != torch.int32 or ft.numel() < 1 or ft.device != dev:
                raise RuntimeError("matmul_multi: ready flags must be an int32 CUDA tensor on the operands' device")
            q.ready_flags, q.ready_count = ft.data_ptr(), ft.numel()
            if torch.is_tensor(fv):  # a device word that holds the target (bumped once per step)
                q.ready_epoch, q.ready_value = fv.data_ptr(), 0
            else:
                q.ready_epoch, q.ready_value = None, int(fv)
    st = 1
    if 1 <= n <= 8:
        with torch.cuda.device(dev):
            st = lib.mg_matmul_multi(n, ctypes.cast(arr, ctypes.c_void_p), _stream())
    if st in (1, 3):  # a shape or pitch the grouped kernel does not take
        if (flags is not None and any(f is not None for f in flags)) or any(a is not None and len(a.shards) > 1 for a in sharded):
            raise RuntimeError("matmul_multi: ready flags and row-sharded activations need problems the CTA-pair kernel takes")
        for (A, B, _), o in zip(problems, outs):
            matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5], out=o)
    else:
        _capi.check(st, "matmul_multi")
    return outs


def set_option(name, value):
    """mg_set_option: choose between kernels / turn a mode off at run time (names in mixedgemm_c.h)."""
    _capi.check(_capi.load().mg_set_option(name.encode(), int(value)), "set_option(%s)" % name)


def reset_options():
    _capi.load().mg_reset_options()


def set_wait_limit_us(us):
    _capi.check(_capi.load().mg_set_wait_limit_us(int(us)), "set_wait_limit_us")


def device_status():
    """Reads and clears the device error word (non-zero after a kernel gave up on a bounded wait)."""
    import ctypes
    lib = _capi.load()
    v = ctypes.c_int(0)
    st = lib.mg_device_status(ctypes.byref(v), _stream())
    if st != 7:  # MG_ERR_TIMEOUT only says that the word was non-zero
        _capi.check(st, "device_status")
    return v.value


def test_function():
    """bindings.cpp:329."""
    return "Hello from test_function!"
