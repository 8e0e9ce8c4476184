"""GPU parity of the reorder-and-quantise kernels, through the C ABI (ctypes): bit-exact
against the CPU oracle, and against the reference's own kernels compiled for sm_100a
where the reference instantiates that K."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _run(b, idx, KN, KS, KO, weights):
    import mixedgemm_b200 as mg
    Xd = H.bits_to_torch(b, "cuda")
    idxd = torch.from_numpy(np.asarray(idx, np.int16)).cuda()
    fn = mg.reorder_quantize_w if weights else mg.reorder_quantize_x
    out = fn(Xd, idxd, KN, KS, KO, b.shape[0], b.shape[0])
    torch.cuda.synchronize()
    return out, Xd, idxd


@pytest.mark.parametrize("weights", [False, True])
@pytest.mark.parametrize("R,KN,KS,KO", [
    (1, 64, 32, 32), (3, 128, 64, 32), (16, 2560, 1408, 128), (114, 2560, 896, 128), (128, 256, 128, 128),
    (129, 2240, 1216, 128), (300, 1024, 0, 0), (257, 0, 512, 0), (33, 0, 0, 256), (40, 8960, 4928, 448),
    (9, 17920, 9856, 896)])
def test_matches_cpu_oracle(R, KN, KS, KO, weights):
    rng = np.random.default_rng(R + KN + 3 * KS + 7 * KO)
    K = KN + KS + KO
    b = H.rand_bits(rng, (R, K))
    # adversarial groups: all zero, negative zeros, exact MAX * 2^k and neighbours
    b[0, :32] = 0
    b[0, 32:64] = 0x8000
    if K >= 128:
        b[0, 64:96] = (b[0, 64:96] & 0x8000) | 0x3F80  # all +-1
        b[0, 96:128] = 0x40C0  # all 6.0
    idx = rng.permutation(K).astype(np.int16)
    got, _, _ = _run(b, idx, KN, KS, KO, weights)
    want = H.oracle_outputs(b, idx, KN, KS, KO, weights)
    H.compare_quantised(got, want, R, (KN, KS, KO), "R=%d K=%d w=%s" % (R, K, weights))


@pytest.mark.parametrize("weights", [False, True])
def test_scale_boundaries(weights):
    """Group maxima MAX*2^k and one bf16 ulp either side, for every format."""
    KN, KS, KO = 128, 128, 128
    K = KN + KS + KO
    rows = []
    for fmt_max, seg0 in ((6.0, 0), (28.0, KN), (448.0, KN + KS)):
        for k in range(-12, 10):
            for d in (-1, 0, 1):
                row = np.zeros(K, np.uint16)
                top = int(orc.f32_to_bf16_bits(np.float32(fmt_max * 2.0 ** k))) + d
                for g in range(4):
                    row[seg0 + g * 32: seg0 + g * 32 + 32] = np.arange(32, dtype=np.uint16) * 3 + (top - 200)
                    row[seg0 + g * 32 + 5 * g] = top | (0x8000 if g & 1 else 0)
                rows.append(row)
    b = np.stack(rows)
    idx = np.arange(K, dtype=np.int16)
    got, _, _ = _run(b, idx, KN, KS, KO, weights)
    want = H.oracle_outputs(b, idx, KN, KS, KO, weights)
    H.compare_quantised(got, want, b.shape[0], (KN, KS, KO), "boundaries")


@pytest.mark.parametrize("weights", [False, True])
@pytest.mark.parametrize("R,K,split", [(114, 3584, (2560, 896, 128)), (300, 4096, (2560, 1408, 128)),
                                       (64, 14336, (8960, 4928, 448)), (130, 5120, (3200, 1760, 160)),
                                       (70, 12288, (7680, 4224, 384)), (66, 13824, (8640, 4736, 448)),
                                       (34, 18944, (11840, 6528, 576))])
def test_matches_compiled_reference_kernel(R, K, split, weights):
    """Same bytes as MixedGemm's reorder_bf16_mixed_kernel / reorder_bf16_fp4_kernel run on this GPU."""
    if H.ref_lib() is None or not H.ref_lib().ref_supports_k(K):
        pytest.skip("compiled reference kernel not available")
    KN, KS, KO = split
    Xb = H.make_x(R, K, seed=R) if not weights else H.make_w(R, K, seed=R)
    idx = H.reorder_index(H.make_x(64, K, seed=5)).numpy()
    b = H.bits(Xb)
    got, Xd, idxd = _run(b, idx, KN, KS, KO, weights)
    want = H.ref_reorder(Xd, idxd, KN, KS, KO, weights)
    H.compare_quantised(got, want, R, (KN, KS, KO), "vs reference kernel K=%d" % K)
    # and the CPU oracle agrees with the reference kernel too (pins the oracle)
    cpu = H.oracle_outputs(b, idx, KN, KS, KO, weights)
    for i in range(3):
        assert np.array_equal(cpu[i], want[i])
    for i, k in enumerate((KN, KS, KO)):
        m = orc.sf_valid_mask(R, k)
        assert np.array_equal(np.asarray(cpu[3 + i])[m], want[3 + i][m])


def test_main_py_case():
    """The reference smoke script's input bands (main.py:15-19,29): M=114, K=3584, identity index."""
    M, K = 114, 3584
    KN, KS, KO = 2560, 3584 - 128 - 2560, 128
    g = torch.Generator().manual_seed(3)
    signs = torch.randint(0, 2, (M, K), generator=g).to(torch.bfloat16) * 2 - 1
    X = torch.rand(M, K, generator=g).to(torch.bfloat16) * 3
    X[:, -KS:] = torch.rand(M, KS, generator=g).to(torch.bfloat16) * 14 + 14
    X[:, -KN:] = torch.rand(M, KN, generator=g).to(torch.bfloat16) * 256 + 256
    X = X * signs
    b = H.bits(X)
    idx = np.arange(K, dtype=np.int16)
    got, Xd, idxd = _run(b, idx, KN, KS, KO, False)
    H.compare_quantised(got, H.oracle_outputs(b, idx, KN, KS, KO), M, (KN, KS, KO), "main.py")
    if H.ref_lib() is not None:
        H.compare_quantised(got, H.ref_reorder(Xd, idxd, KN, KS, KO), M, (KN, KS, KO), "main.py vs reference")


@pytest.mark.parametrize("M,K,dist,outlier", [(2048, 4096, "normal", 20.0), (2048, 14336, "normal", 20.0),
                                              (4096, 8192, "student3", 30.0), (1024, 28672, "student3", 30.0),
                                              (8192, 16384, "normal", 20.0)])
def test_benchmark_shapes_row_sample(M, K, dist, outlier):
    """Full-size benchmark shapes: rows are independent, so a seeded sample of rows is compared
    bit for bit with the oracle; every scale byte of the full output is range-checked."""
    import mixedgemm_b200 as mg
    KN, KS, KO = H.split_k(K)
    Ms = 96
    Xs = H.make_x(Ms, K, seed=11, dist=dist, outlier=outlier)
    idx = H.reorder_index(Xs)
    reps = M // Ms + 1
    Xd = Xs.cuda().repeat(reps, 1)[:M].contiguous()
    out = mg.reorder_quantize_x(Xd, idx.cuda(), KN, KS, KO, M, M)
    torch.cuda.synchronize()
    want = H.oracle_outputs(H.bits(Xs), idx.numpy(), KN, KS, KO)
    for blk in (0, reps // 2, reps - 2):
        r0 = blk * Ms
        for i in range(3):
            assert np.array_equal(out[i][r0:r0 + Ms].cpu().numpy(), want[i]), (blk, i)
        for i, k in enumerate((KN, KS, KO)):
            sf = out[3 + i].cpu().numpy()
            rr = np.arange(r0, r0 + Ms)[:, None]
            kb = np.arange(k // 32)[None, :]
            got = sf[orc.sf_offset(rr, kb, k)]
            assert np.array_equal(got, orc.sf_to_rowmajor(np.asarray(want[3 + i]), Ms, k)), (blk, i)


def test_rejects_bad_arguments():
    import mixedgemm_b200 as mg
    X = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    idx = torch.arange(128, dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError):
        mg.reorder_quantize_x(X, idx, 64, 32, 16, 4, 4)  # does not sum to K
    with pytest.raises(RuntimeError):
        mg.reorder_quantize_x(X, idx, 80, 32, 16, 4, 4)  # not multiples of 32
    with pytest.raises(RuntimeError):
        mg.reorder_quantize_x(X.float(), idx, 64, 32, 32, 4, 4)
    out = mg.reorder_quantize_x(X[:0], idx, 64, 32, 32, 0, 0)  # empty input is fine
    assert out[0].shape == (0, 32)


@pytest.mark.parametrize("M,K", [(1, 128), (16, 4096), (2048, 4096), (300, 14336), (64, 28672), (5, 136)])
def test_reorder_index_kernel(M, K):
    """Index calibration: same permutation as the stable argsort of the oracle and of torch."""
    import mixedgemm_b200 as mg
    Xb = H.make_x(M, K, seed=M + K)
    Xb[:, ::7] = Xb[:, 3:4]  # plenty of exact ties
    idx, amax = mg.reorder_index(Xb.cuda(), return_absmax=True)
    want, mag = orc.np_reorder_index(H.bits(Xb))
    assert np.array_equal(H.bits(amax.cpu()), mag)
    assert np.array_equal(idx.cpu().numpy(), want)
    tidx = torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16)
    assert torch.equal(idx.cpu(), tidx)


def test_multi_problem_launch_equals_separate_calls():
    """Several activations in one launch (mg_reorder_quantize_multi) give, problem by problem, the
    bytes of a launch each: sizes that differ by 100x, stages of 1, 4 and 8 rows in one grid, a
    single-row problem, pitched and dense outputs, an empty problem."""
    import mixedgemm_b200 as mg
    shapes = [(1024, (5120, 2816, 256)), (1024, (17920, 9856, 896)), (1, (128, 64, 64)), (77, (2560, 1408, 128)),
              (4096, (256, 128, 128)), (16, (8960, 4928, 448)), (300, (1024, 0, 0)), (513, (0, 0, 2048))]
    rng = np.random.default_rng(5)
    probs, want = [], []
    for j, (M, split) in enumerate(shapes):
        K = sum(split)
        X = H.make_x(M, K, seed=200 + j).cuda()
        idx = torch.from_numpy(rng.permutation(K).astype(np.int16)).cuda()
        out = mg.alloc_quantized_x(M, *split, X.device, padded=bool(j % 2))
        for t in out:
            t.fill_(0x5A)
        probs.append((X, idx, *split, out))
        # rows beyond M inside the last scale atom are never written: same fill on both sides
        ref = mg.alloc_quantized_x(M, *split, X.device, padded=bool(j % 2))
        for t in ref:
            t.fill_(0x5A)
        want.append(mg.reorder_quantize_x(X, idx, *split, out=ref))
    got = mg.reorder_quantize_x_multi(probs)
    torch.cuda.synchronize()
    assert mg.device_status() == 0
    lib_sf = mg.sf_bytes
    for (M, split), g, w in zip(shapes, got, want):
        for i in range(3):
            assert torch.equal(g[i], w[i]), (M, split, i)
            n = lib_sf(M, split[i])
            assert torch.equal(g[3 + i][:n], w[3 + i][:n]), (M, split, "sf", i)
    # a list of one, and a list with an empty problem in it
    one = mg.reorder_quantize_x_multi([probs[3][:5] + (None,)])[0]
    assert all(torch.equal(a, b) for a, b in zip(one[:3], want[3][:3]))
    empty = torch.empty((0, 512), dtype=torch.bfloat16, device="cuda")
    idx512 = torch.arange(512, dtype=torch.int16, device="cuda")
    two = mg.reorder_quantize_x_multi([(empty, idx512, 256, 128, 128, None), probs[0][:5] + (None,)])
    assert torch.equal(two[1][0], want[0][0]) and two[0][0].shape == (0, 128)
    with pytest.raises(RuntimeError):
        mg.reorder_quantize_x_multi([probs[0]] * 9)


def test_multi_problem_launch_of_weights_through_the_c_abi():
    """mg_reorder_quantize_multi with weights = 1 (every segment to E2M1): the bytes of
    reorder_quantize_w, problem by problem, and the argument checks of the entry point."""
    import ctypes
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    shapes = [(512, (2560, 1408, 128)), (1024, (256, 128, 128)), (128, (5120, 2816, 256))]   # whole scale atoms
    arr = (_capi.QuantProblem * len(shapes))()
    keep, want = [], []
    rng = np.random.default_rng(11)
    for j, (N, split) in enumerate(shapes):
        K = sum(split)
        W = H.make_w(N, K, seed=300 + j).cuda()
        idx = torch.from_numpy(rng.permutation(K).astype(np.int16)).cuda()
        out = mg.alloc_quantized_w(N, *split, W.device)
        keep.append((W, idx, out))
        want.append(mg.reorder_quantize_w(W, idx, *split))
        q = arr[j]
        q.X, q.rows, q.K, q.idx = W.data_ptr(), N, K, idx.data_ptr()
        q.KN, q.KS, q.KO = split
        q.C4, q.C6, q.C8 = out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr()
        for i in range(3):
            q.pitch[i] = out[i].stride(0)
        q.SF4, q.SF6, q.SF8 = out[3].data_ptr(), out[4].data_ptr(), out[5].data_ptr()
    st = lib.mg_reorder_quantize_multi(1, len(shapes), ctypes.cast(arr, ctypes.c_void_p), None)
    assert st == 0
    torch.cuda.synchronize()
    for (N, split), (_, _, out), w in zip(shapes, keep, want):
        for i in range(3):
            assert torch.equal(out[i], w[i]), (N, split, i)
            n = mg.sf_bytes(N, split[i])
            assert torch.equal(out[3 + i][:n], w[3 + i][:n])
    assert lib.mg_reorder_quantize_multi(1, 9, ctypes.cast(arr, ctypes.c_void_p), None) == 1     # MG_ERR_SHAPE
    assert lib.mg_reorder_quantize_multi(1, 2, None, None) == 2                                  # MG_ERR_NULL
    assert lib.mg_reorder_quantize_multi(1, 0, None, None) == 0
    arr[1].K = 500                                                                               # K != KN + KS + KO
    assert lib.mg_reorder_quantize_multi(1, 3, ctypes.cast(arr, ctypes.c_void_p), None) == 1
