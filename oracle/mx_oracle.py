"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the
smoke entry and by the CPU-baseline / reference legs of the bench, never by the product
package.

Two independent restatements of the reference's reorder-and-quantise path live here:

* `c_*`  - thin ctypes wrappers over `oracle/mx_oracle.c`, which follows the reference's
  literal float expression chain (src/reorder.cu:160-248, :320-431).
* `np_*` - a vectorised numpy formulation that uses only integer arithmetic on the bf16
  bit patterns (exponent-bit scale rule + code tables).  The CPU tests require both to
  agree with each other and with the tables produced by CUTLASS's own host converters
  (tests/golden/cutlass_tables.json).

All paths `src/...`, `include/...` are relative to the MixedGemm project.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

FMT_E2M1, FMT_E3M2, FMT_E4M3 = 0, 1, 2
FMT_MAX = {FMT_E2M1: 6, FMT_E3M2: 28, FMT_E4M3: 448}  # src/reorder.cu:17-19
# (shift, mantissa threshold) of the exponent rule: MAX = 1.5*2^2, 1.75*2^4, 1.75*2^8
_SCALE_RULE = {FMT_E2M1: (2, 64), FMT_E3M2: (4, 96), FMT_E4M3: (8, 96)}

_lib = None


def lib():
    """Load (building if needed) liboracle.so."""
    global _lib
    if _lib is None:
        from oracle import build_oracle
        path = build_oracle.build_oracle()
        L = ctypes.CDLL(path)
        u8p, u16p, i16p = (ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_uint16),
                           ctypes.POINTER(ctypes.c_int16))
        ints = [ctypes.c_int] * 3
        for name in ("orc_reorder_quantize_x", "orc_reorder_quantize_w"):
            f = getattr(L, name)
            f.argtypes = [u16p, ctypes.c_int, ctypes.c_int, i16p] + ints + [u8p] * 6
            f.restype = None
        L.orc_sf_offset.argtypes = ints
        L.orc_sf_offset.restype = ctypes.c_size_t
        L.orc_sf_bytes.argtypes = [ctypes.c_int, ctypes.c_int]
        L.orc_sf_bytes.restype = ctypes.c_size_t
        L.orc_encode.argtypes = [ctypes.c_float, ctypes.c_int]
        L.orc_encode.restype = ctypes.c_uint8
        L.orc_decode.argtypes = [ctypes.c_uint8, ctypes.c_int]
        L.orc_decode.restype = ctypes.c_float
        L.orc_dequantize.argtypes = [u8p, u8p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.POINTER(ctypes.c_float)]
        L.orc_dequantize.restype = None
        L.orc_gemm_f64.argtypes = [ctypes.POINTER(ctypes.c_float)] * 2 + ints + [
            ctypes.POINTER(ctypes.c_double)]
        L.orc_gemm_f64.restype = None
        L.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        _lib = L
    return _lib


def _p(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct))


# --------------------------------------------------------------------------- layout
def sf_offset(r, kb, kseg):
    """Byte offset of scale (row r, 32-block kb) in a segment's scale buffer
    (include/reorder.cuh:119-124, src/reorder.cu:181-185).  Works on ints or arrays."""
    katoms = (kseg + 127) // 128
    return (r % 32) * 16 + ((r // 32) % 4) * 4 + (kb % 4) + (kb // 4) * 512 + (r // 128) * 512 * katoms


def sf_bytes(rows, kseg):
    """Size of the swizzled scale buffer: whole 128x128-element atoms of 512 bytes."""
    return ((rows + 127) // 128) * ((kseg + 127) // 128) * 512


def ref_sf_alloc_x(M, kseg):
    """What the reference binding allocates for an activation scale buffer
    (src/bindings.cpp:91-93)."""
    return (M // 128 + 1) * 128 * kseg // 32


def sf_valid_mask(rows, kseg):
    """Boolean mask over sf_bytes(rows,kseg): True where a scale is actually written."""
    m = np.zeros(sf_bytes(rows, kseg), dtype=bool)
    r = np.arange(rows)[:, None]
    kb = np.arange(kseg // 32)[None, :]
    m[sf_offset(r, kb, kseg).ravel()] = True
    return m


def sf_to_rowmajor(sf, rows, kseg):
    r = np.arange(rows)[:, None]
    kb = np.arange(kseg // 32)[None, :]
    return sf[sf_offset(r, kb, kseg)]


# --------------------------------------------------------------------------- C wrappers
def c_reorder_quantize(X_bits, idx, KN, KS, KO, weights=False):
    """X_bits: uint16 [rows, K] (bf16 bit patterns); idx int16 [K].
    Returns (c4, c6|c4, c8|c4, sf4, sf6, sf8) uint8 arrays; scale buffers are sized
    sf_bytes() and zero where nothing is written."""
    L = lib()
    X_bits = np.ascontiguousarray(X_bits, dtype=np.uint16)
    idx = np.ascontiguousarray(idx, dtype=np.int16)
    R, K = X_bits.shape
    assert K == KN + KS + KO
    if weights:
        o = [np.zeros((R, KN // 2), np.uint8), np.zeros((R, KS // 2), np.uint8),
             np.zeros((R, KO // 2), np.uint8)]
        fn = L.orc_reorder_quantize_w
    else:
        o = [np.zeros((R, KN // 2), np.uint8), np.zeros((R, KS // 4 * 3), np.uint8),
             np.zeros((R, KO), np.uint8)]
        fn = L.orc_reorder_quantize_x
    s = [np.zeros(max(sf_bytes(R, k), 1), np.uint8) for k in (KN, KS, KO)]
    fn(_p(X_bits, ctypes.c_uint16), R, K, _p(idx, ctypes.c_int16), KN, KS, KO,
       *[_p(a, ctypes.c_uint8) for a in o + s])
    return tuple(o + [a[:sf_bytes(R, k)] for a, k in zip(s, (KN, KS, KO))])


def c_dequantize(codes, sf, rows, kseg, fmt):
    L = lib()
    if kseg == 0:
        return np.zeros((rows, 0), np.float32)
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    out = np.empty((rows, kseg), np.float32)
    L.orc_dequantize(_p(codes, ctypes.c_uint8), _p(sf, ctypes.c_uint8), rows, kseg, fmt,
                     _p(out, ctypes.c_float))
    return out


def c_gemm_f64(A, B):
    L = lib()
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, K = A.shape
    N = B.shape[0]
    Y = np.empty((M, N), np.float64)
    L.orc_gemm_f64(_p(A, ctypes.c_float), _p(B, ctypes.c_float), M, N, K, _p(Y, ctypes.c_double))
    return Y


# --------------------------------------------------------------------------- numpy restatement
def _rne_shift(v, s):
    """Round-to-nearest-even right shift of non-negative ints."""
    if s <= 0:
        return v << (-s)
    half = 1 << (s - 1)
    q = v >> s
    rem = v & ((1 << s) - 1)
    return q + ((rem > half) | ((rem == half) & ((q & 1) == 1)))


def code_table(fmt):
    """code_table(fmt)[n] = magnitude code of the integer n after the reference's
    float->bf16->format chain (src/reorder.cu:223-246), n = 0..MAX."""
    ebits, mbits = {FMT_E2M1: (2, 1), FMT_E3M2: (3, 2), FMT_E4M3: (4, 3)}[fmt]
    bias = (1 << (ebits - 1)) - 1
    out = np.zeros(FMT_MAX[fmt] + 1, np.uint8)
    for n in range(1, FMT_MAX[fmt] + 1):
        e = n.bit_length() - 1
        # bf16 keeps 8 significant bits
        nb = n if e <= 7 else int(_rne_shift(np.int64(n), e - 7)) << (e - 7)
        e = nb.bit_length() - 1
        # all integers >= 1 are normal numbers in the three formats (emin <= 0)
        q = int(_rne_shift(np.int64(nb), e - mbits)) if e >= mbits else nb << (mbits - e)
        out[n] = ((e + bias) << mbits) + (q - (1 << mbits))
    return out


def np_scale_bytes(absmax_bits, fmt):
    """E8M0 byte from the group's largest 15-bit bf16 magnitude (src/reorder.cu:179-180):
    the smallest power of two 2^e with maxv <= MAX * 2^e; 126 for an all-zero group."""
    a = absmax_bits.astype(np.int32)
    sh, thr = _SCALE_RULE[fmt]
    E = a >> 7
    m = a & 0x7F
    sf = E - sh + (m > thr)
    return np.where(a == 0, 126, sf).astype(np.uint8)


def np_quantise_groups(g_bits, fmt):
    """g_bits: uint16 [..., 32] reordered bf16 bit patterns of whole groups.
    Returns (codes uint8 [..., 32], sf uint8 [...])."""
    mag = (g_bits & 0x7FFF).astype(np.int32)
    sign = (g_bits >> 15).astype(np.uint8)
    sf = np_scale_bytes(mag.max(axis=-1), fmt)
    e = sf.astype(np.int32) - 127
    # |x| * 2^-e as exact rational: (128+m) * 2^(E-127-7-e); round half away from zero
    E = mag >> 7
    m = np.where(E > 0, 128 + (mag & 0x7F), mag & 0x7F).astype(np.int64)
    shl = np.where(E > 0, E, 1) - 127 - 7 - e[..., None]  # value = m * 2^shl
    pos = np.clip(shl, 0, 40)
    neg = np.clip(-shl, 0, 62)
    # half away from zero for shl < 0: floor(m / 2^neg + 1/2) = (m + 2^(neg-1)) >> neg
    n_neg = (m + (np.int64(1) << np.clip(neg - 1, 0, 62))) >> neg
    n = np.where(shl >= 0, m << pos, n_neg)
    n = np.minimum(n, FMT_MAX[fmt]).astype(np.int64)
    codes = code_table(fmt)[n]
    signbit = {FMT_E2M1: 3, FMT_E3M2: 5, FMT_E4M3: 7}[fmt]
    return (codes | (sign << signbit)).astype(np.uint8), sf


def pack_fp4(c):
    return (c[..., 0::2] & 0xF) | (c[..., 1::2] << 4)


def pack_fp6(c):
    v0, v1, v2, v3 = (c[..., i::4].astype(np.uint16) & 0x3F for i in range(4))
    out = np.empty(c.shape[:-1] + (c.shape[-1] // 4 * 3,), np.uint8)
    out[..., 0::3] = (v0 | (v1 << 6)) & 0xFF
    out[..., 1::3] = ((v1 >> 2) | (v2 << 4)) & 0xFF
    out[..., 2::3] = ((v2 >> 4) | (v3 << 2)) & 0xFF
    return out


def unpack_fp4(p):
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out


def unpack_fp6(p):
    b0, b1, b2 = (p[..., i::3].astype(np.uint16) for i in range(3))
    out = np.empty(p.shape[:-1] + (p.shape[-1] // 3 * 4,), np.uint8)
    out[..., 0::4] = b0 & 0x3F
    out[..., 1::4] = ((b0 >> 6) | (b1 << 2)) & 0x3F
    out[..., 2::4] = ((b1 >> 4) | (b2 << 4)) & 0x3F
    out[..., 3::4] = b2 >> 2
    return out


def np_reorder_quantize(X_bits, idx, KN, KS, KO, weights=False):
    """numpy restatement of reorder_quantize_x / _w; same returns as c_reorder_quantize."""
    X_bits = np.asarray(X_bits, dtype=np.uint16)
    R, K = X_bits.shape
    Xr = X_bits[:, np.asarray(idx).astype(np.uint16).astype(np.int64)]
    outs, sfs = [], []
    k0 = 0
    for kseg, fmt in ((KN, FMT_E2M1), (KS, FMT_E3M2), (KO, FMT_E4M3)):
        f = FMT_E2M1 if weights else fmt
        g = Xr[:, k0:k0 + kseg].reshape(R, kseg // 32, 32)
        k0 += kseg
        if kseg == 0:
            outs.append(np.zeros((R, 0), np.uint8))
            sfs.append(np.zeros(0, np.uint8))
            continue
        codes, sf = np_quantise_groups(g, f)
        codes = codes.reshape(R, kseg)
        outs.append(pack_fp4(codes) if f == FMT_E2M1 else pack_fp6(codes) if f == FMT_E3M2 else codes)
        buf = np.zeros(sf_bytes(R, kseg), np.uint8)
        r = np.arange(R)[:, None]
        kb = np.arange(kseg // 32)[None, :]
        buf[sf_offset(r, kb, kseg)] = sf
        sfs.append(buf)
    return tuple(outs + sfs)


# --------------------------------------------------------------------------- decode / GEMM
_DECODE = {}


def decode_table(fmt):
    if fmt not in _DECODE:
        n = {FMT_E2M1: 16, FMT_E3M2: 64, FMT_E4M3: 256}[fmt]
        L = lib()
        _DECODE[fmt] = np.array([L.orc_decode(c, fmt) for c in range(n)], np.float64)
    return _DECODE[fmt]


def np_dequantize(codes, sf, rows, kseg, fmt):
    """float64 [rows, kseg] = value(code) * 2^(sf-127)."""
    if kseg == 0:
        return np.zeros((rows, 0))
    c = unpack_fp4(codes) if fmt == FMT_E2M1 else unpack_fp6(codes) if fmt == FMT_E3M2 else codes
    v = decode_table(fmt)[c[:rows, :kseg]]
    s = sf_to_rowmajor(np.asarray(sf), rows, kseg).astype(np.int32) - 127
    return v * np.repeat(np.ldexp(1.0, s), 32, axis=1)


def gemm_f64(A_parts, B_parts, M, N, KN, KS, KO):
    """fp64 dequantise-then-matmul of the packed operands (src/gemm.cu:44-46 without the
    intermediate bf16 roundings).  A_parts = (AN, AS, AO, SFAN, SFAS, SFAO), B likewise."""
    Y = np.zeros((M, N))
    for i, (kseg, fa) in enumerate(((KN, FMT_E2M1), (KS, FMT_E3M2), (KO, FMT_E4M3))):
        if kseg == 0:
            continue
        a = np_dequantize(A_parts[i], A_parts[3 + i], M, kseg, fa)
        b = np_dequantize(B_parts[i], B_parts[3 + i], N, kseg, FMT_E2M1)
        Y += a @ b.T
    return Y


def bf16_round(y):
    """fp64/fp32 array -> nearest-even bf16 values (returned as float32)."""
    f = np.asarray(y, np.float32)
    u = f.view(np.uint32)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def f32_to_bf16_bits(x):
    f = np.ascontiguousarray(x, np.float32)
    u = f.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def np_reorder_index(X_bits):
    """Stable ascending argsort of the per-channel absmax (main.py:31-33 with the sort made stable):
    on bf16 bit patterns, the magnitude bits order like the values."""
    mag = (np.asarray(X_bits, np.uint16) & 0x7FFF).max(axis=0)
    return np.argsort(mag, kind="stable").astype(np.int16), mag
