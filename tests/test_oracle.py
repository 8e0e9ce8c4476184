"""CPU tests that pin the oracle: against the tables produced by CUTLASS's host converters
(tests/golden/cutlass_tables.json), and the C restatement against the numpy one."""
import json
import os

import numpy as np
import pytest

from oracle import mx_oracle as orc

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "cutlass_tables.json")))
FMTS = [(orc.FMT_E2M1, "e2m1"), (orc.FMT_E3M2, "e3m2"), (orc.FMT_E4M3, "e4m3")]


@pytest.mark.parametrize("fmt,name", FMTS)
def test_code_tables_match_cutlass(fmt, name):
    gold = np.array(GOLD["codes_" + name], np.uint8)
    assert np.array_equal(orc.code_table(fmt), gold)
    L = orc.lib()
    got = np.array([L.orc_encode(float(n), fmt) for n in range(len(gold))], np.uint8)
    # the C encoder sees the value after the bf16 step, as the reference does
    got_bf = np.array([L.orc_encode(float(orc.bf16_round(np.float32(n))), fmt) for n in range(len(gold))], np.uint8)
    assert np.array_equal(got_bf, gold)
    if fmt != orc.FMT_E4M3:  # below 256 the bf16 step is the identity
        assert np.array_equal(got, gold)
    assert L.orc_encode(-0.0, fmt) == GOLD["negzero_" + name]


def test_known_codes():
    # E2M1: 0.5 and 1.5 are never produced, 5 rounds to 4 (ties to even)
    assert list(orc.code_table(orc.FMT_E2M1)) == [0x0, 0x2, 0x4, 0x5, 0x6, 0x6, 0x7]
    t6 = orc.code_table(orc.FMT_E3M2)
    assert (t6[1], t6[8], t6[9], t6[14], t6[28]) == (0x0C, 0x18, 0x18, 0x1B, 0x1F)
    t8 = orc.code_table(orc.FMT_E4M3)
    # 431 rounds to bf16 432, which is a tie between 416 and 448 -> 448 (double rounding)
    assert (t8[1], t8[17], t8[100], t8[416], t8[431], t8[448]) == (0x38, 0x58, 0x6C, 0x7D, 0x7E, 0x7E)


@pytest.mark.parametrize("fmt,name", FMTS)
def test_scale_rule_matches_cutlass(fmt, name):
    pts = GOLD["scale_" + name]
    a = np.arange(0x80, 0x7F80, dtype=np.int32)
    gold = np.zeros_like(a)
    for (start, byte), nxt in zip(pts, pts[1:] + [[0x7F80, 0]]):
        gold[start - 0x80:nxt[0] - 0x80] = byte
    got = orc.np_scale_bytes(a, fmt).astype(np.int32)
    # magnitudes so small that the reference's scale is a subnormal float are out of range
    ok = a >= 0x0400
    assert np.array_equal(got[ok], gold[ok])
    assert orc.np_scale_bytes(np.array([0]), fmt)[0] == GOLD["scale_zero_" + name] == 126
    # MAX * 2^k  ->  127 + k
    for k in range(-20, 20):
        bits = orc.f32_to_bf16_bits(np.float32(orc.FMT_MAX[fmt] * 2.0 ** k)) & 0x7FFF
        assert orc.np_scale_bytes(bits, fmt)[0] == 127 + k


def test_golden_groups_c_and_numpy():
    for g in GOLD["groups"]:
        fmt = g["fmt"]
        bits = np.array(g["bits"], np.uint16)
        codes, sf = orc.np_quantise_groups(bits[None, :], fmt)
        assert sf[0] == g["sf"], g
        assert list(codes[0]) == g["codes"], g
        # the C oracle: put the group in the segment of its format
        KN, KS, KO = [(32, 0, 0), (0, 32, 0), (0, 0, 32)][fmt]
        out = orc.c_reorder_quantize(bits[None, :], np.arange(32), KN, KS, KO)
        packed = [orc.pack_fp4, orc.pack_fp6, lambda c: c][fmt](np.array(g["codes"], np.uint8)[None, :])
        assert np.array_equal(out[fmt], packed), g
        assert out[3 + fmt][0] == g["sf"]


def _rand_bits(rng, shape, lo=100, hi=140):
    e = rng.integers(lo, hi, size=shape, dtype=np.uint16)
    m = rng.integers(0, 128, size=shape, dtype=np.uint16)
    s = rng.integers(0, 2, size=shape, dtype=np.uint16)
    b = (s << 15) | (e << 7) | m
    z = rng.random(shape) < 0.02
    return np.where(z, s << 15, b).astype(np.uint16)


@pytest.mark.parametrize("weights", [False, True])
@pytest.mark.parametrize("R,KN,KS,KO", [(16, 2560, 1408, 128), (5, 64, 32, 32), (130, 128, 192, 64),
                                        (3, 0, 96, 32), (7, 8960 // 4, 4928 // 4 - 16, 448 // 4 + 16)])
def test_c_equals_numpy(R, KN, KS, KO, weights):
    rng = np.random.default_rng(R * 7 + KN)
    K = KN + KS + KO
    X = _rand_bits(rng, (R, K))
    idx = rng.permutation(K).astype(np.int16)
    a = orc.c_reorder_quantize(X, idx, KN, KS, KO, weights)
    b = orc.np_reorder_quantize(X, idx, KN, KS, KO, weights)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_config1_gaussian_with_outliers():
    """The single-layer CPU configuration: M=16, K=4096, 128 outlier channels x20."""
    import torch
    g = torch.Generator().manual_seed(0)
    M, K, KN, KS, KO = 16, 4096, 2560, 1408, 128
    X = torch.randn(M, K, generator=g)
    out_ch = torch.randperm(K, generator=g)[:128]
    X[:, out_ch] *= 20
    Xb = X.to(torch.bfloat16)
    idx = torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16).numpy()
    bits = Xb.view(torch.int16).numpy().view(np.uint16)
    a = orc.c_reorder_quantize(bits, idx, KN, KS, KO)
    b = orc.np_reorder_quantize(bits, idx, KN, KS, KO)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    # the outlier channels land in the FP8 segment
    assert set(idx[-128:].tolist()) == set(out_ch.numpy().astype(np.int16).tolist())


def test_sf_offset_is_a_bijection_onto_atoms():
    for rows, kseg in [(300, 128), (114, 896), (128, 448), (257, 1408), (16, 4928)]:
        r = np.arange(rows)[:, None]
        kb = np.arange(kseg // 32)[None, :]
        off = orc.sf_offset(r, kb, kseg).ravel()
        assert len(np.unique(off)) == off.size
        assert off.max() < orc.sf_bytes(rows, kseg)
        L = orc.lib()
        assert L.orc_sf_offset(rows - 1, kseg // 32 - 1, kseg) == orc.sf_offset(rows - 1, kseg // 32 - 1, kseg)
    # spot values of the swizzle: ((r%32)*16 + (r/32%4)*4 + kb%4) + (kb/4)*512 + (r/128)*512*katoms
    assert orc.sf_offset(0, 0, 256) == 0
    assert orc.sf_offset(1, 0, 256) == 16
    assert orc.sf_offset(32, 0, 256) == 4
    assert orc.sf_offset(0, 3, 256) == 3
    assert orc.sf_offset(0, 4, 256) == 512
    assert orc.sf_offset(128, 0, 256) == 1024
    assert orc.sf_offset(128, 0, 448) == 2048  # K atoms are ceil-padded


def test_pack_roundtrip():
    rng = np.random.default_rng(1)
    c4 = rng.integers(0, 16, (9, 64), dtype=np.uint8)
    c6 = rng.integers(0, 64, (9, 64), dtype=np.uint8)
    assert np.array_equal(orc.unpack_fp4(orc.pack_fp4(c4)), c4)
    assert np.array_equal(orc.unpack_fp6(orc.pack_fp6(c6)), c6)
    # little-endian bit stream (src/reorder.cu:54-63)
    assert list(orc.pack_fp6(np.array([[0x3F, 0, 0, 0]], np.uint8))[0]) == [0x3F, 0, 0]
    assert list(orc.pack_fp6(np.array([[0, 0x3F, 0, 0]], np.uint8))[0]) == [0xC0, 0x0F, 0]
    assert list(orc.pack_fp6(np.array([[0, 0, 0, 0x3F]], np.uint8))[0]) == [0, 0, 0xFC]
    assert list(orc.pack_fp4(np.array([[0x1, 0xF]], np.uint8))[0]) == [0xF1]


def test_known_answer_ones_and_half():
    """main.py:12-14 (commented case): X = 1 with one -2.5, W = 0.5, identity index."""
    M, N, KN, KS, KO = 4, 8, 64, 32, 32
    K = KN + KS + KO
    X = np.ones((M, K), np.float32)
    X[0, 1] = -2.5
    W = np.full((N, K), 0.5, np.float32)
    idx = np.arange(K, dtype=np.int16)
    A = orc.c_reorder_quantize(orc.f32_to_bf16_bits(X), idx, KN, KS, KO)
    B = orc.c_reorder_quantize(orc.f32_to_bf16_bits(W), idx, KN, KS, KO, weights=True)
    # group (0,0): max 2.5 -> scale 2^-1 (2.5 <= 6*0.5); 1 -> 2 -> code 0x4; -2.5 -> -5 -> 4 -> 0xE
    assert A[3][orc.sf_offset(0, 0, KN)] == 126
    assert A[0][0, 0] == (0x4 | (0xE << 4))
    # other rows: max 1 -> scale 2^-2 (1 <= 6/4); 1 -> 4 -> code 0x6
    assert A[3][orc.sf_offset(1, 0, KN)] == 125 and A[0][1, 0] == 0x66
    # weights 0.5: scale 2^-3 (0.5 <= 6/8); 0.5 -> 4 -> 0x6
    assert B[3][orc.sf_offset(0, 0, KN)] == 124 and B[0][0, 0] == 0x66
    Y = orc.gemm_f64(A, B, M, N, KN, KS, KO)
    # row 0: (K-1)*1*0.5 + (-2.0)*0.5 (the -2.5 became -4 * 0.5 = -2.0)
    assert np.allclose(Y[0], (K - 1) * 0.5 - 1.0)
    assert np.allclose(Y[1:], K * 0.5)


def test_dequant_and_gemm_c_vs_numpy():
    rng = np.random.default_rng(3)
    M, N, KN, KS, KO = 9, 128, 128, 64, 32
    K = KN + KS + KO
    X = _rand_bits(rng, (M, K), 120, 132)
    W = _rand_bits(rng, (N, K), 115, 125)
    idx = rng.permutation(K).astype(np.int16)
    A = orc.c_reorder_quantize(X, idx, KN, KS, KO)
    B = orc.c_reorder_quantize(W, idx, KN, KS, KO, weights=True)
    Yn = orc.gemm_f64(A, B, M, N, KN, KS, KO)
    fa = [orc.FMT_E2M1, orc.FMT_E3M2, orc.FMT_E4M3]
    Ad = np.concatenate([orc.c_dequantize(A[i], A[3 + i], M, k, fa[i]) for i, k in enumerate((KN, KS, KO))], 1)
    Bd = np.concatenate([orc.c_dequantize(B[i], B[3 + i], N, k, orc.FMT_E2M1) for i, k in enumerate((KN, KS, KO))], 1)
    Yc = orc.c_gemm_f64(Ad, Bd)
    assert np.allclose(Yc, Yn, rtol=1e-12, atol=1e-12)
    # quantisation error is bounded: dequantised X is close to the reordered X
    Xf = (X[:, idx.astype(np.uint16)].astype(np.uint32) << 16).view(np.float32)
    assert np.abs(Ad - Xf).max() <= 0.26 * np.abs(Xf).max()


def test_reorder_index_oracle_matches_torch_stable_sort():
    import torch
    from tests import helpers as H
    Xb = H.make_x(33, 512, seed=2)
    Xb[:, ::5] = Xb[:, 1:2]
    want = torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16).numpy()
    got, mag = orc.np_reorder_index(H.bits(Xb))
    assert np.array_equal(got, want)
    assert sorted(got.tolist()) == list(range(512))
