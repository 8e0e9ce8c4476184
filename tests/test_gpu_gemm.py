"""GPU parity of the mixed block-scaled GEMM, through the C ABI (ctypes).

Oracle: float64 dequantise-then-matmul of the SAME packed operands (oracle/mx_oracle.py).
Tolerances (stated by the benchmark definition): relative Frobenius error <= 1e-3 and
max-abs error <= 1e-2 * RMS(output).  They are applied to the fp32 accumulator
(mg_matmul_f32); the bf16 result must then be exactly the nearest-even rounding of that
accumulator, and is additionally compared with the bf16-rounded float64 product.  (bf16
rounding alone costs up to 2^-9 relative, so a raw bf16-vs-float64 max-abs bound of
1e-2 RMS cannot hold for any implementation.)"""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3
MAX_ABS_TOL = 1e-2  # times the output RMS


def _quantise(M, N, K, split, seed=0, dist="normal", outlier=20.0, wstd=0.02):
    import mixedgemm_b200 as mg
    KN, KS, KO = split
    X = H.make_x(M, K, seed=seed, dist=dist, outlier=outlier)
    W = H.make_w(N, K, seed=seed + 1, std=wstd)
    idx = H.reorder_index(X).cuda()
    A = mg.reorder_quantize_x(X.cuda(), idx, KN, KS, KO, M, N)
    B = mg.reorder_quantize_w(W.cuda(), idx, KN, KS, KO, M, N)
    return A, B


def _oracle(A, B, M, N, split, rows=None):
    KN, KS, KO = split
    a = [t.cpu().numpy() for t in A]
    b = [t.cpu().numpy() for t in B]
    if rows is not None:
        # scale buffers are addressed by absolute row, so dequantise first, then sample
        Y = np.zeros((len(rows), N))
        for i, (k, fa) in enumerate(((KN, orc.FMT_E2M1), (KS, orc.FMT_E3M2), (KO, orc.FMT_E4M3))):
            if k == 0:
                continue
            ad = orc.np_dequantize(a[i], a[3 + i], M, k, fa)[rows]
            bd = orc.np_dequantize(b[i], b[3 + i], N, k, orc.FMT_E2M1)
            Y += ad @ bd.T
        return Y
    return orc.gemm_f64(a, b, M, N, KN, KS, KO)


def _check(A, B, M, N, split, rows=None, C=None):
    import mixedgemm_b200 as mg
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    Y32 = mg.matmul(*args, out_dtype=torch.float32, C=C)
    Y16 = mg.matmul(*args, C=C)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    Yo = _oracle(A, B, M, N, split, rows)
    if C is not None:
        Yo = Yo + (C.float().cpu().numpy().astype(np.float64) if rows is None else
                   C.float().cpu().numpy().astype(np.float64)[rows])
    y32 = Y32.cpu().numpy().astype(np.float64)
    y16 = Y16.float().cpu().numpy()
    if rows is not None:
        y32s, y16s = y32[rows], y16[rows]
    else:
        y32s, y16s = y32, y16
    rms = np.sqrt(np.mean(Yo ** 2))
    fro = np.linalg.norm(y32s - Yo) / np.linalg.norm(Yo)
    mx = np.abs(y32s - Yo).max() / rms
    assert fro <= REL_FRO_TOL, "fp32 accumulator: rel-Frobenius %.3e" % fro
    assert mx <= MAX_ABS_TOL, "fp32 accumulator: max-abs %.3e RMS" % mx
    # the bf16 output is the accumulator rounded once, to nearest even
    rne = orc.bf16_round(Y32.cpu().numpy())
    assert np.array_equal(y16, rne), "bf16 output is not RNE(fp32 accumulator)"
    # against the bf16-rounded float64 product: Frobenius bound, and max-abs up to one-ulp flips
    yo16 = orc.bf16_round(Yo).astype(np.float64)
    fro16 = np.linalg.norm(y16s - yo16) / np.linalg.norm(yo16)
    assert fro16 <= REL_FRO_TOL, "bf16 vs bf16(fp64): rel-Frobenius %.3e" % fro16
    diff = np.abs(y16s - yo16)
    ulp = np.abs(yo16) * 2.0 ** -7 + 1e-30
    assert np.all((diff <= MAX_ABS_TOL * rms) | (diff <= ulp)), "bf16 vs bf16(fp64): more than a one-ulp flip"
    return fro, mx


@pytest.mark.parametrize("M,N,split", [
    (128, 128, (256, 0, 0)), (128, 128, (0, 128, 0)), (128, 128, (0, 0, 128)),
    (128, 256, (256, 128, 128)), (16, 128, (128, 128, 128)), (114, 384, (2560, 896, 128)),
    (300, 512, (640, 384, 128)), (1, 128, (256, 256, 128)), (257, 1024, (2560, 1408, 128))])
def test_small_shapes(M, N, split):
    K = sum(split)
    A, B = _quantise(M, N, K, split, seed=M + N)
    _check(A, B, M, N, split)


@pytest.mark.parametrize("bn", ["128", "256"])
def test_both_tile_widths(bn, mgopt):
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    """The single-CTA kernel with 128- and 256-column tiles."""
    mgopt.setenv("MG_GEMM_2CTA", "0")
    mgopt.setenv("MG_GEMM_BN", bn)
    M, N, split = 384, 1024, (1280, 768, 128)
    A, B = _quantise(M, N, sum(split), split, seed=9)
    _check(A, B, M, N, split)


@pytest.mark.parametrize("M,N,split", [(256, 256, (256, 128, 128)), (300, 512, (640, 384, 128)),
                                       (129, 256, (128, 0, 0)), (1000, 768, (2560, 1408, 128)),
                                       (640, 256, (384, 192, 64)), (2048, 1024, (2560, 1408, 128))])
def test_cta_pair_kernel_equals_single_cta_kernel(M, N, split, mgopt):
    """The CTA-pair kernel (256 x 256 tiles over two SMs, TMA-store epilogue) and the single-CTA
    kernel accumulate the same products in the same order: same bytes, and both pass the oracle."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    A, B = _quantise(M, N, sum(split), split, seed=M)
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    mgopt.setenv("MG_GEMM_2CTA", "1")
    Yp = mg.matmul(*args)
    mgopt.setenv("MG_GEMM_2CTA", "0")
    Ys = mg.matmul(*args)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(Yp.view(torch.int16), Ys.view(torch.int16))
    mgopt.setenv("MG_GEMM_2CTA", "1")
    _check(A, B, M, N, split)


def test_segments_with_64_tails():
    """K = 14336 splits into 8960 / 4928 / 448: the last two are only multiples of 64 and go
    through the padded copy in the workspace."""
    M, N, split = 200, 256, (8960, 4928, 448)
    A, B = _quantise(M, N, sum(split), split, seed=4)
    _check(A, B, M, N, split)
    M, N, split = 130, 128, (128, 192, 64)
    A, B = _quantise(M, N, sum(split), split, seed=5)
    _check(A, B, M, N, split)


def test_dense_buffers_take_the_padded_copy_and_agree():
    """Row-pitched buffers (what the quantisers return) are read in place; the reference's dense
    buffers of a 64-tail segment go through the padded copy in the workspace.  Same result."""
    import mixedgemm_b200 as mg
    M, N, split = 384, 512, (8960, 4928, 448)
    K = sum(split)
    X = H.make_x(M, K, seed=8).cuda()
    W = H.make_w(N, K, seed=9).cuda()
    idx = H.reorder_index(X.cpu()).cuda()
    A = mg.reorder_quantize_x(X, idx, *split, M, N)
    B = mg.reorder_quantize_w(W, idx, *split, M, N)
    assert not A[1].is_contiguous() and A[1].shape == (M, split[1] // 4 * 3)
    Ad = mg.reorder_quantize_x(X, idx, *split, M, N, out=mg.alloc_quantized_x(M, *split, X.device, padded=False))
    Bd = mg.reorder_quantize_w(W, idx, *split, M, N, out=mg.alloc_quantized_w(N, *split, X.device, padded=False))
    assert Ad[1].is_contiguous()
    for i in range(3):
        assert torch.equal(A[i], Ad[i]) and torch.equal(B[i], Bd[i])
    lib = __import__("mixedgemm_b200._capi", fromlist=["load"]).load()
    assert lib.mg_matmul_workspace_bytes(M, N, *split) > 0
    y0 = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    y1 = mg.matmul(Ad[0], Bd[0], Ad[1], Bd[1], Ad[2], Bd[2], Ad[3], Bd[3], Ad[4], Bd[4], Ad[5], Bd[5])
    y2 = mg.matmul(A[0], Bd[0], A[1], Bd[1], A[2], Bd[2], A[3], Bd[3], A[4], Bd[4], A[5], Bd[5])
    torch.cuda.synchronize()
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    assert torch.equal(y0.view(torch.int16), y2.view(torch.int16))
    _check(Ad, Bd, M, N, split)


def test_accumulate_into_c():
    M, N, split = 256, 256, (512, 256, 128)
    A, B = _quantise(M, N, sum(split), split, seed=6)
    g = torch.Generator().manual_seed(1)
    C = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    _check(A, B, M, N, split, C=C)


def test_known_answer_integers():
    """main.py:24-27 style case: small-integer X and W, exactly representable after quantisation
    with power-of-two scales, so the product is exact."""
    import mixedgemm_b200 as mg
    M, N, split = 128, 128, (256, 128, 128)
    K = sum(split)
    g = torch.Generator().manual_seed(2)
    X = torch.randint(-3, 4, (M, K), generator=g).to(torch.bfloat16)
    X[:, 0::32] = 3  # every group holds its maximum so that the scale is 2^-1 and values double exactly
    W = torch.randint(-3, 4, (N, K), generator=g).to(torch.bfloat16)
    W[:, 0::32] = 3
    idx = torch.arange(K, dtype=torch.int16).cuda()
    A = mg.reorder_quantize_x(X.cuda(), idx, *split, M, N)
    B = mg.reorder_quantize_w(W.cuda(), idx, *split, M, N)
    Y = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5], out_dtype=torch.float32)
    want = X.double() @ W.double().T
    assert torch.equal(Y.cpu().double(), want)


@pytest.mark.parametrize("M,N,K,dist,outlier,wstd", [
    (2048, 4096, 4096, "normal", 20.0, 0.02), (2048, 1024, 4096, "normal", 20.0, 0.02),
    (2048, 14336, 4096, "normal", 20.0, 0.02), (2048, 4096, 14336, "normal", 20.0, 0.02),
    (4096, 1024, 8192, "student3", 30.0, 0.015), (64, 4096, 4096, "normal", 20.0, 0.02),
    (8, 14336, 4096, "normal", 20.0, 0.02), (4096, 3584, 8192, "student3", 30.0, 0.015),
    (2048, 2048, 28672, "student3", 30.0, 0.015), (512, 2048, 28672, "student3", 30.0, 0.015)])
def test_benchmark_shapes_row_sample(M, N, K, dist, outlier, wstd):
    """Benchmark-size problems: a seeded sample of output rows against the float64 oracle, plus
    linearity in the scales over the whole output (doubling every A scale doubles Y exactly)."""
    import mixedgemm_b200 as mg
    split = H.split_k(K)
    A, B = _quantise(M, N, K, split, seed=21, dist=dist, outlier=outlier, wstd=wstd)
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 46)]))
    _check(A, B, M, N, split, rows=rows)
    args = lambda A_: (A_[0], B[0], A_[1], B[1], A_[2], B[2], A_[3], B[3], A_[4], B[4], A_[5], B[5])
    Y1 = mg.matmul(*args(A), out_dtype=torch.float32)
    A2 = list(A[:3]) + [t + 1 for t in A[3:]]
    Y2 = mg.matmul(*args(A2), out_dtype=torch.float32)
    assert torch.equal(Y2, Y1 * 2)


def _dequant_sample(codes, sf, rows, kseg, fmt):
    """float64 [len(rows), kseg] of the sampled rows of a device-resident operand (scale bytes are
    addressed by absolute row, so the sample is taken before dequantising)."""
    if kseg == 0:
        return np.zeros((len(rows), 0))
    rows = np.asarray(rows)
    c = codes[torch.from_numpy(rows).cuda()].contiguous().cpu().numpy()
    c = orc.unpack_fp4(c) if fmt == orc.FMT_E2M1 else orc.unpack_fp6(c) if fmt == orc.FMT_E3M2 else c
    v = orc.decode_table(fmt)[c[:, :kseg]]
    offs = orc.sf_offset(rows[:, None], np.arange(kseg // 32)[None, :], kseg).astype(np.int64)
    s = sf[torch.from_numpy(offs).cuda()].cpu().numpy().astype(np.int32) - 127
    return v * np.repeat(np.ldexp(1.0, s), 32, axis=1)


@pytest.mark.parametrize("M,N,K,dist,outlier,wstd", [
    (8192, 8192, 8192, "normal", 20.0, 0.02), (16384, 16384, 16384, "normal", 20.0, 0.02),
    (4096, 28672, 8192, "student3", 30.0, 0.015)])
def test_largest_shapes_row_and_column_sample(M, N, K, dist, outlier, wstd):
    """The large squares and the full-width 70B gate/up projection: inputs are drawn on the device,
    a seeded sample of output rows x 128-column blocks is compared with the float64 oracle of the
    same packed operands, and over the WHOLE output bf16 == RNE(fp32 accumulator) bit for bit."""
    import mixedgemm_b200 as mg
    KN, KS, KO = split = H.split_k(K)
    g = torch.Generator(device="cuda").manual_seed(77)
    X = torch.randn(M, K, generator=g, device="cuda")
    if dist == "student3":
        chi = torch.zeros(M, K, device="cuda")
        for _ in range(3):
            chi += torch.randn(M, K, generator=g, device="cuda").pow_(2)
        X = X / (chi / 3).sqrt_() / (3 ** 0.5)
        del chi
    X[:, torch.randperm(K, generator=g, device="cuda")[:K // 32]] *= outlier
    Xb = X.to(torch.bfloat16)
    del X
    idx = mg.reorder_index(Xb)
    assert torch.equal(idx, torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16))
    A = mg.reorder_quantize_x(Xb, idx, KN, KS, KO, M, N)
    del Xb
    W = (torch.randn(N, K, generator=g, device="cuda") * wstd).to(torch.bfloat16)
    B = mg.reorder_quantize_w(W, idx, KN, KS, KO, M, N)
    del W
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    Y32 = mg.matmul(*args, out_dtype=torch.float32)
    Y16 = mg.matmul(*args)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(Y16.view(torch.int16), Y32.to(torch.bfloat16).view(torch.int16))
    rng = np.random.default_rng(M + N)
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 46)]))
    blocks = sorted({0, N // 128 - 1, int(rng.integers(0, N // 128)), int(rng.integers(0, N // 128))})
    cols = np.concatenate([np.arange(b * 128, b * 128 + 128) for b in blocks])
    fa = (orc.FMT_E2M1, orc.FMT_E3M2, orc.FMT_E4M3)
    Ao = np.concatenate([_dequant_sample(A[i], A[3 + i], rows, k, fa[i]) for i, k in enumerate(split)], 1)
    Bo = np.concatenate([_dequant_sample(B[i], B[3 + i], cols, k, orc.FMT_E2M1) for i, k in enumerate(split)], 1)
    Yo = Ao @ Bo.T
    sel = Y32[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy().astype(np.float64)
    rms = np.sqrt(np.mean(Yo ** 2))
    fro = np.linalg.norm(sel - Yo) / np.linalg.norm(Yo)
    assert fro <= REL_FRO_TOL, "rel-Frobenius %.3e" % fro
    assert np.abs(sel - Yo).max() <= MAX_ABS_TOL * rms


@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_decode_sweep_default_dispatch(N, K):
    """The decode sweep as the benchmark runs it: M in {1, 8, 16, 32, 64, 128} on the four Llama-3-8B
    layers, whatever kernel the library picks by itself (no switches set)."""
    import mixedgemm_b200 as mg
    KN, KS, KO = split = H.split_k(K)
    Xall = H.make_x(128, K, seed=N + K)
    idx = H.reorder_index(Xall).cuda()
    W = H.make_w(N, K, seed=3)
    B = mg.reorder_quantize_w(W.cuda(), idx, KN, KS, KO, 128, N)
    b = [t.cpu().numpy() for t in B]
    Bd = np.concatenate([orc.np_dequantize(b[i], b[3 + i], N, k, orc.FMT_E2M1) for i, k in enumerate(split)], 1)
    fa = (orc.FMT_E2M1, orc.FMT_E3M2, orc.FMT_E4M3)
    for M in (1, 8, 16, 32, 64, 128):
        A = mg.reorder_quantize_x(Xall[:M].cuda().contiguous(), idx, KN, KS, KO, M, N)
        args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
        Y32 = mg.matmul(*args, out_dtype=torch.float32)
        Y16 = mg.matmul(*args)
        torch.cuda.synchronize()
        assert mg.device_status() == 0
        a = [t.cpu().numpy() for t in A]
        Ad = np.concatenate([orc.np_dequantize(a[i], a[3 + i], M, k, fa[i]) for i, k in enumerate(split)], 1)
        Yo = Ad @ Bd.T
        y32 = Y32.cpu().numpy().astype(np.float64)
        rms = np.sqrt(np.mean(Yo ** 2))
        fro = np.linalg.norm(y32 - Yo) / np.linalg.norm(Yo)
        assert fro <= REL_FRO_TOL, "M=%d: rel-Frobenius %.3e" % (M, fro)
        assert np.abs(y32 - Yo).max() <= MAX_ABS_TOL * rms, "M=%d" % M
        # the bf16 entry point may cut K differently from the fp32 one (split-K needs scratch that only
        # some calls get), so it is held to one bf16 step of the rounded accumulator, not to its bytes
        rne = Y32.to(torch.bfloat16).float()
        d = (Y16.float() - rne).abs()
        assert torch.all(d <= rne.abs() * 2.0 ** -7 + 1e-30), "M=%d" % M


@pytest.mark.parametrize("fmt,with_c", [(4, False), (4, True), (6, False), (6, True), (8, False), (8, True)])
def test_single_format_entry_points(fmt, with_c):
    """mg_matmul_fp4 / fp6 / fp8 called directly through the C ABI: the replacements of the
    reference's matmul_host4 / 6 / 8 (include/fp4.h:46-56 and siblings), with and without the C
    addend those take."""
    import ctypes
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    M, N, K = 200, 256, 512
    split = {4: (K, 0, 0), 6: (0, K, 0), 8: (0, 0, K)}[fmt]
    seg = {4: 0, 6: 1, 8: 2}[fmt]
    A, B = _quantise(M, N, K, split, seed=fmt)
    C = (torch.randn(M, N, generator=torch.Generator().manual_seed(fmt)) * 0.5).to(torch.bfloat16).cuda() if with_c else None
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    fn = {4: lib.mg_matmul_fp4, 6: lib.mg_matmul_fp6, 8: lib.mg_matmul_fp8}[fmt]
    assert A[seg].is_contiguous() and B[seg].is_contiguous()
    st = fn(vp(A[seg]), vp(B[seg]), M, N, K, vp(C), vp(D), vp(A[3 + seg]), vp(B[3 + seg]),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, st
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    Yo = _oracle(A, B, M, N, split)
    if with_c:
        Yo = Yo + C.float().cpu().numpy().astype(np.float64)
    want = orc.bf16_round(Yo.astype(np.float32))
    got = D.float().cpu().numpy()
    rms = np.sqrt(np.mean(Yo ** 2))
    assert np.linalg.norm(got - Yo) / np.linalg.norm(Yo) <= 3e-3  # bf16 output rounding included
    diff = np.abs(got - want)
    assert np.all((diff <= MAX_ABS_TOL * rms) | (diff <= np.abs(want) * 2.0 ** -7 + 1e-30))
    # and the same bytes as the three-segment entry point given only this segment
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    ref = mg.matmul(*args, C=C)
    assert torch.equal(ref.view(torch.int16), D.view(torch.int16))


def test_rejects_bad_arguments():
    import mixedgemm_b200 as mg
    M, N, split = 128, 128, (256, 128, 128)
    A, B = _quantise(M, N, sum(split), split)
    with pytest.raises(RuntimeError):  # N not a multiple of 128
        mg.matmul(A[0], B[0][:100], A[1], B[1][:100], A[2], B[2][:100], A[3], B[3], A[4], B[4], A[5], B[5])
    with pytest.raises(RuntimeError):
        mg.matmul(A[0].cpu(), B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])


def test_rejects_operands_that_disagree_with_the_inferred_sizes():
    """M, N and the K split are inferred from AN, BN, AS and AO (as the reference does); tensors that
    do not fit those sizes are refused before anything is launched, by the Python mirror and by the
    drop-in module alike - a short scale buffer would otherwise be read past its end on the device."""
    import os
    import sys
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import build
    sys.path.insert(0, os.path.dirname(build.ext_path()))
    import mixedgemm as ext
    M, N, split = 256, 256, (256, 192, 64)
    A, B = _quantise(M, N, sum(split), split)
    good = [A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5]]
    mg.matmul(*good)
    ext.matmul(*good)
    cases = {
        "AS rows": (2, A[1][:128]), "BO rows": (5, B[2][:128]), "BS width": (3, B[1][:, :64]),
        "AS width": (2, A[1][:, :96]), "short SFAS": (8, A[4][:512]), "short SFBO": (11, B[5][:256]),
        # the reference's own size for a 64-wide segment is N*64/32 bytes; whole atoms need N*16
        "reference-sized SFBO": (11, B[5][:N * 64 // 32]),
    }
    for name, (pos, bad) in cases.items():
        args = list(good)
        args[pos] = bad
        for fn in (mg.matmul, ext.matmul):
            with pytest.raises(RuntimeError):
                fn(*args)
    with pytest.raises(RuntimeError):
        mg.matmul(*good, C=torch.zeros(M, N, dtype=torch.float32, device="cuda"))
    with pytest.raises(RuntimeError):
        mg.matmul(*good, out=torch.empty(M, N + 8, dtype=torch.bfloat16, device="cuda"))
    torch.cuda.synchronize()
    assert mg.device_status() == 0


@pytest.mark.parametrize("M,Ns,split", [(512, (512, 256, 256), (1280, 640, 128)), (2048, (4096, 1024, 1024), (2560, 1408, 128)),
                                        (300, (256, 768), (8960, 4928, 448)), (100, (256, 256), (256, 128, 128))])
def test_grouped_weights_equal_separate_calls(M, Ns, split, mgopt):
    """q/k/v- or gate/up-style groups in one launch give the bytes of one launch per weight
    (the last case is too small for the grouped kernel and takes the fallback)."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    KN, KS, KO = split
    K = sum(split)
    X = H.make_x(M, K, seed=31)
    idx = H.reorder_index(X).cuda()
    A = mg.reorder_quantize_x(X.cuda(), idx, KN, KS, KO, M, 0)
    Bs = [mg.reorder_quantize_w(H.make_w(N, K, seed=40 + j).cuda(), idx, KN, KS, KO, M, N) for j, N in enumerate(Ns)]
    outs = mg.matmul_group(A, Bs)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    for B, N, y in zip(Bs, Ns, outs):
        ref = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
        assert y.shape == (M, N)
        assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
    _check(A, Bs[-1], M, Ns[-1], split)


@pytest.mark.parametrize("M,N,split,force", [
    (16, 4096, (8960, 4928, 448), None), (384, 512, (8960, 4928, 448), None), (16, 4096, (2560, 1408, 128), "4"),
    (128, 1024, (2560, 1408, 128), "6"), (100, 768, (2560, 1408, 128), "7"), (300, 256, (2560, 1408, 128), "5"),
    (1, 128, (256, 128, 128), "3"), (97, 512, (1280, 704, 64), "5"), (16, 14336, (2560, 1408, 128), "2")])
def test_split_k(M, N, split, force, mgopt):
    """Problems with few tiles (decode shapes, narrow weight shards) run several CTAs per tile of the
    single-CTA kernel, each over a range of K stages; the CTA that arrives last adds the fp32
    partials in split order.  Same bounds against the oracle, bf16 == RNE(fp32 result) exactly,
    the same bytes on every call (the counters are left clear, the sum order is fixed), within one
    bf16 step of the unsplit kernel, with and without the C addend."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_CSPLIT", "0")  # otherwise the cluster form takes these shapes
    if force is not None:
        mgopt.setenv("MG_GEMM_SPLITK", force)
    A, B = _quantise(M, N, sum(split), split, seed=3 * M + N)
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    _check(A, B, M, N, split)
    C = (torch.randn(M, N, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).cuda()
    _check(A, B, M, N, split, C=C)
    y1 = mg.matmul(*args)
    y2 = mg.matmul(*args)
    # the scratch is the caller's: whatever it holds when a launch starts must not matter
    from mixedgemm_b200 import api
    for buf in list(api._workspaces.values()) + api._retired:
        buf.fill_(0xAB)
    y3 = mg.matmul(*args)
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    y0 = mg.matmul(*args)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
    assert torch.equal(y1.view(torch.int16), y3.view(torch.int16))
    d = (y1.float() - y0.float()).abs()
    assert torch.all(d <= y0.float().abs() * 2.0 ** -7 + 1e-30)


@pytest.mark.parametrize("M,N,split", [(1, 128, (256, 128, 128)), (8, 1024, (2560, 1408, 128)), (16, 4096, (2560, 1408, 128)),
                                       (17, 256, (128, 64, 64)), (32, 1024, (8960, 4928, 448)), (33, 384, (1280, 704, 64)),
                                       (64, 4096, (2560, 1408, 128)), (100, 768, (2560, 1408, 128)),
                                       (128, 14336, (2560, 1408, 128))])
def test_decode_form(M, N, split, mgopt):
    """M <= 128 runs the single-CTA kernel with the operand roles swapped (weights as the 128-row
    operand, activations as a 16/32/64/128-column operand, tile stored transposed).  Same bounds
    against the oracle, with and without the C addend, and the same bytes as the 128-row form:
    every output element is the same K-ordered sum either way."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SWAP", "1")
    A, B = _quantise(M, N, sum(split), split, seed=7 * M + N)
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    rows = None if M * N <= 1 << 20 else np.unique(np.concatenate([[0, M - 1], np.random.default_rng(0).integers(0, M, 30)]))
    _check(A, B, M, N, split, rows=rows)
    C = (torch.randn(M, N, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).cuda()
    _check(A, B, M, N, split, rows=rows, C=C)
    y1 = mg.matmul(*args)
    f1 = mg.matmul(*args, out_dtype=torch.float32)
    mgopt.setenv("MG_GEMM_SWAP", "0")
    y0 = mg.matmul(*args)
    f0 = mg.matmul(*args, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(f1.view(torch.int32), f0.view(torch.int32))
    assert torch.equal(y1.view(torch.int16), y0.view(torch.int16))


@pytest.mark.parametrize("M,N,split", [(16, 4096, (2560, 1408, 128)), (128, 1024, (2560, 1408, 128)),
                                       (64, 4096, (8960, 4928, 448)), (300, 256, (2560, 1408, 128)),
                                       (100, 768, (2560, 1408, 128)), (4096, 128, (5120, 2816, 256)),
                                       (1, 128, (1280, 704, 64)), (129, 2304, (640, 256, 128))])
def test_cluster_split_k(M, N, split, mgopt):
    """Problems whose 128 x 128 tiles occupy at most a quarter of the SMs run as clusters of four
    CTAs, each over a quarter of the K stages; the accumulators are exchanged through distributed
    shared memory and added in CTA order.  Same bounds against the oracle, bf16 == RNE(fp32 result)
    exactly, the same bytes on every call, within one bf16 step of the unsplit kernel, with and
    without the C addend, and across a tile count that makes clusters loop over several tiles."""
    import mixedgemm_b200 as mg
    A, B = _quantise(M, N, sum(split), split, seed=5 * M + N)
    args = (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    rows = None if M * N <= 1 << 20 else np.unique(np.concatenate([[0, M - 1], np.random.default_rng(0).integers(0, M, 30)]))
    _check(A, B, M, N, split, rows=rows)
    C = (torch.randn(M, N, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).cuda()
    _check(A, B, M, N, split, rows=rows, C=C)
    y1 = mg.matmul(*args)
    y2 = mg.matmul(*args)
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    mgopt.setenv("MG_GEMM_SWAP", "0")
    y0 = mg.matmul(*args)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
    d = (y1.float() - y0.float()).abs()
    assert torch.all(d <= y0.float().abs() * 2.0 ** -7 + 1e-30)
    assert not torch.equal(y1, torch.zeros_like(y1))


def _abargs(A, B):
    return (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])


def test_multi_problem_launch_equals_separate_calls(mgopt):
    """Independent problems (own activation, own K split) in one launch of the CTA-pair kernel give
    the bytes of one launch each; a list the kernel does not take falls back to separate launches."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    shapes = [(512, 512, (1280, 640, 128)), (300, 256, (8960, 4928, 448)), (2048, 1024, (2560, 1408, 128)),
              (129, 768, (128, 0, 0))]
    probs = []
    for j, (M, N, split) in enumerate(shapes):
        A, B = _quantise(M, N, sum(split), split, seed=50 + j)
        probs.append((A, B, None))
    outs = mg.matmul_multi(probs)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    for (A, B, _), y, (M, N, split) in zip(probs, outs, shapes):
        ref = mg.matmul(*_abargs(A, B))
        assert y.shape == (M, N)
        assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
    _check(probs[1][0], probs[1][1], *shapes[1][:2], shapes[1][2])
    # M <= 128 is not for the pair kernel: the list is then served by separate launches
    A, B = _quantise(64, 256, 512, (256, 128, 128), seed=60)
    outs = mg.matmul_multi([probs[0], (A, B, None)])
    assert torch.equal(outs[1].view(torch.int16), mg.matmul(*_abargs(A, B)).view(torch.int16))


def test_row_sharded_activation_equals_the_contiguous_one(mgopt):
    """The layout a multi-GPU exchange fills (every shard's codes and scales in one contiguous block,
    shards equally spaced) multiplies to the bytes of the plain layout: shard counts 2, 4 and 8, an M
    whose last tile pair is half empty, a shard smaller than a tile pair, and a second, plain problem
    in the same launch."""
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    for (M, N, split, world) in [(512, 512, (1280, 640, 128), 2), (1024, 256, (2560, 1408, 128), 4),
                                 (1024, 512, (1280, 640, 128), 8), (384, 256, (256, 128, 128), 3),
                                 (2048, 768, (3584, 0, 512), 2)]:
        K = sum(split)
        A, B = _quantise(M, N, K, split, seed=90 + world)
        want = mg.matmul(*_abargs(A, B))
        mp = M // world
        pitch = [lib.mg_code_pitch(0, i, k) for i, k in enumerate(split)]
        logical = (split[0] // 2, split[1] // 4 * 3, split[2])
        sizes = [mp * p for p in pitch] + [lib.mg_sf_bytes(mp, k) for k in split]
        offs, off = [], 0
        for n in sizes:
            offs.append(off)
            off += (n + 1023) // 1024 * 1024
        flat = torch.full((world * off + 1024,), 0x5A, dtype=torch.uint8, device="cuda")
        flat = flat[(-flat.data_ptr()) % 1024:]
        shards = []
        for r in range(world):
            blk = flat[r * off:(r + 1) * off]
            part = []
            for i in range(3):
                v = blk[offs[i]:offs[i] + sizes[i]].view(mp, pitch[i])[:, :logical[i]]
                v.copy_(A[i][r * mp:(r + 1) * mp])
                part.append(v)
            for i, k in enumerate(split):
                per_block = ((k + 127) // 128) * 512
                v = blk[offs[3 + i]:offs[3 + i] + sizes[3 + i]]
                v.copy_(A[3 + i][(r * mp // 128) * per_block:((r + 1) * mp // 128) * per_block])
                part.append(v)
            shards.append(tuple(part))
        SA = mg.ShardedActivation(shards)
        assert SA.rows == M and SA.shard_rows == mp
        other = _quantise(300, 256, K, split, seed=95)
        outs = mg.matmul_multi([(SA, B, None), (other[0], other[1], None)])
        torch.cuda.synchronize()
        assert mg.device_status() == 0
        assert torch.equal(outs[0].view(torch.int16), want.view(torch.int16)), (M, N, split, world)
        assert torch.equal(outs[1].view(torch.int16), mg.matmul(*_abargs(*other)).view(torch.int16))
    with pytest.raises(RuntimeError):
        mg.ShardedActivation([shards[1], shards[0]])       # not in memory order
    with pytest.raises(RuntimeError):
        mg.ShardedActivation([shards[0], tuple(t[:64] if t.dim() == 2 else t for t in shards[1])])


def test_cost_balanced_tile_schedule_equals_separate_calls(mgopt):
    """More tiles than SM pairs, and tiles of different cost (K): the launch then follows the host's
    schedule table (each tile to the SM pair that is free first) instead of dealing the tiles out
    round-robin.  Every tile must still be computed exactly once, whatever pair it lands on."""
    import mixedgemm_b200 as mg
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    shapes = [(2048, 2048, (2560, 1408, 128)), (1024, 1024, (8960, 4928, 448)), (512, 4096, (1280, 640, 128)),
              (300, 512, (128, 0, 0))]
    probs = []
    for j, (M, N, split) in enumerate(shapes):
        A, B = _quantise(M, N, sum(split), split, seed=110 + j)
        probs.append((A, B, torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")))
    for order in ([0, 1, 2, 3], [3, 1, 0, 2]):
        for (_, _, o) in probs:
            o.fill_(7.0)
        outs = mg.matmul_multi([probs[j] for j in order])
        torch.cuda.synchronize()
        assert mg.device_status() == 0
        for j, y in zip(order, outs):
            A, B, _ = probs[j]
            assert torch.equal(y.view(torch.int16), mg.matmul(*_abargs(A, B)).view(torch.int16)), (order, j)


def test_ready_flag_holds_a_problem_back_until_its_activation_is_there(mgopt):
    """A problem with a ready flag is not read before the flag reaches its value: the activation is
    filled, and the flag raised, by copy-engine copies on another stream AFTER the launch."""
    import mixedgemm_b200 as mg
    mg.set_wait_limit_us(2_000_000)
    M, N, split = 512, 512, (1280, 640, 128)
    A0, B0 = _quantise(M, N, sum(split), split, seed=70)
    A1, B1 = _quantise(M, N, sum(split), split, seed=72)
    want0, want1 = mg.matmul(*_abargs(A0, B0)), mg.matmul(*_abargs(A1, B1))
    late = [torch.full_like(t, 0x5A) for t in A1]     # what the kernel must NOT multiply
    for t in late[3:]:
        t.fill_(127)                                   # scale bytes of 1.0, so a premature read is finite but wrong
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    one = torch.ones(1, dtype=torch.int32).pin_memory()
    good = [t.contiguous().cpu().pin_memory() if t.is_contiguous() else None for t in A1]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    outs = mg.matmul_multi([(A0, B0, None), (tuple(late), B1, None)], flags=[None, (flag, 1)])
    with torch.cuda.stream(side):
        for dst, src, host in zip(late, A1, good):
            if host is not None:
                dst.copy_(host, non_blocking=True)     # host -> device: a copy engine, no SM needed
            else:
                dst.copy_(src, non_blocking=True)
        flag.copy_(one, non_blocking=True)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(outs[0].view(torch.int16), want0.view(torch.int16))
    assert torch.equal(outs[1].view(torch.int16), want1.view(torch.int16))


def test_bounded_waits_run_out_and_the_context_survives(mgopt):
    """Host-side fault injection: (1) the first CTA of the single-CTA kernel never loads its second
    K stage, (2) a problem's ready flag is never raised.  With the wait limit at 1 ms the kernels
    give up, store nothing, return normally; mg_device_status reports the code (and
    MG_ERR_TIMEOUT), and the next call on the same context is correct."""
    import ctypes
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    M, N, split = 128, 128, (512, 256, 128)
    A, B = _quantise(M, N, sum(split), split, seed=80)
    mgopt.setenv("MG_GEMM_CSPLIT", "0")
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    mgopt.setenv("MG_GEMM_2CTA", "0")
    want = mg.matmul(*_abargs(A, B))
    torch.cuda.synchronize()
    mg.set_wait_limit_us(1000)
    mgopt.setenv("MG_FAULT_SKIP_LOAD", "2")
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    mg.matmul(*_abargs(A, B), out=out)
    torch.cuda.synchronize()
    v = ctypes.c_int(0)
    st = lib.mg_device_status(ctypes.byref(v), None)
    assert st == 7 and b"bounded wait" in lib.mg_strerror(st)
    assert v.value & (2 | 8), v.value                   # the MMA warp's or the epilogue's wait ran out
    assert torch.all(out == 7.0)                        # nothing was stored
    mgopt.setenv("MG_FAULT_SKIP_LOAD", "0")
    assert lib.mg_device_status(ctypes.byref(v), None) == 0 and v.value == 0   # the word was cleared
    again = mg.matmul(*_abargs(A, B))
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(again.view(torch.int16), want.view(torch.int16))
    # (2) a flag that nothing raises
    M2, N2, split2 = 256, 256, (256, 128, 128)
    A2, B2 = _quantise(M2, N2, sum(split2), split2, seed=81)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    out2 = torch.full((M2, N2), 7.0, dtype=torch.bfloat16, device="cuda")
    mg.matmul_multi([(A2, B2, out2)], flags=[(flag, 1)])
    torch.cuda.synchronize()
    assert mg.device_status() & 1024
    assert torch.all(out2 == 7.0)
    # the same in a launch of many tiles per CTA pair and two problems: the roles stop issuing at once
    # instead of running through the remaining tiles, so nothing is in flight when the CTAs leave
    M3, N3, split3 = 2048, 6144, (1280, 640, 128)
    A3, B3 = _quantise(M3, N3, sum(split3), split3, seed=82)
    out3 = [torch.full((M3, N3), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags3 = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags3[:2] = 1                                       # rows 0..1023 are "there", the rest never comes
    mg.matmul_multi([(A3, B3, out3[0]), (A3, B3, out3[1])], flags=[None, (flags3, 1, 512, 0)])
    torch.cuda.synchronize()
    assert mg.device_status() & 1024
    mg.set_wait_limit_us(0)
    flags3.fill_(1)
    mg.matmul_multi([(A3, B3, out3[0]), (A3, B3, out3[1])], flags=[None, (flags3, 1, 512, 0)])
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    want3 = mg.matmul(*_abargs(A3, B3))
    assert torch.equal(out3[0].view(torch.int16), want3.view(torch.int16))
    assert torch.equal(out3[1].view(torch.int16), want3.view(torch.int16))
    flag.fill_(1)
    mg.matmul_multi([(A2, B2, out2)], flags=[(flag, 1)])
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    assert torch.equal(out2.view(torch.int16), mg.matmul(*_abargs(A2, B2)).view(torch.int16))
