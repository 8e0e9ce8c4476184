"""Shared helpers of the test-suite: seeded synthetic inputs with the shapes and value
distributions of the benchmark configurations, and access to the checkers (CPU oracle,
compiled reference kernel)."""
import ctypes
import os

import numpy as np
import torch

from oracle import mx_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def split_k(K):
    """The 62.5 / 34.375 / 3.125 % split of every benchmark configuration."""
    KO = K // 32
    KN = K * 5 // 8
    return KN, K - KN - KO, KO


def make_x(M, K, seed=0, dist="normal", outlier=20.0):
    """bf16 activations: N(0,1) or unit-variance Student-t(3), K/32 seeded channels scaled up."""
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g)
    if dist == "student3":
        chi = torch.randn(M, K, 3, generator=g).pow(2).sum(-1) / 3
        X = X / chi.sqrt() / (3 ** 0.5)
    ch = torch.randperm(K, generator=g)[:K // 32]
    X[:, ch] *= outlier
    return X.to(torch.bfloat16)


def make_w(N, K, seed=1, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * std).to(torch.bfloat16)


def reorder_index(Xb):
    """Stable ascending argsort of the per-channel absmax (main.py:31-33, made stable)."""
    return torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16)


def bits(t):
    """bf16 torch tensor (CPU) -> uint16 numpy bit patterns."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def rand_bits(rng, shape, lo=100, hi=140, pzero=0.02):
    e = rng.integers(lo, hi, size=shape, dtype=np.uint16)
    m = rng.integers(0, 128, size=shape, dtype=np.uint16)
    s = rng.integers(0, 2, size=shape, dtype=np.uint16)
    b = (s << 15) | (e << 7) | m
    z = rng.random(shape) < pzero
    return np.where(z, s << 15, b).astype(np.uint16)


def bits_to_torch(b, device="cpu"):
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16).to(device)


def oracle_outputs(b, idx, KN, KS, KO, weights=False):
    return orc.c_reorder_quantize(b, np.asarray(idx), KN, KS, KO, weights)


def compare_quantised(got, want, rows, ks, label=""):
    """got: 6 torch CUDA tensors from the library; want: 6 numpy arrays from a checker.
    Codes must match everywhere, scales at every real (row, block) position."""
    for i in range(3):
        g = got[i].cpu().numpy()
        assert g.shape == want[i].shape, (label, i, g.shape, want[i].shape)
        if not np.array_equal(g, want[i]):
            bad = np.argwhere(g != want[i])
            raise AssertionError("%s: codes of segment %d differ at %d places, first %s: got %d want %d" % (
                label, i, len(bad), bad[0], g[tuple(bad[0])], want[i][tuple(bad[0])]))
    for i, k in enumerate(ks):
        if k == 0:
            continue
        n = orc.sf_bytes(rows, k)
        mask = orc.sf_valid_mask(rows, k)
        g = got[3 + i].cpu().numpy()[:n]
        w = np.asarray(want[3 + i])[:n]
        if not np.array_equal(g[mask], w[mask]):
            bad = np.argwhere((g != w) & mask)
            raise AssertionError("%s: scales of segment %d differ at %d places, first offset %d: got %d want %d" % (
                label, i, len(bad), bad[0][0], g[bad[0][0]], w[bad[0][0]]))


_ref = None


def ref_lib():
    """The reference's own reorder kernels compiled for sm_100a (oracle/_ref), or None."""
    global _ref
    if _ref is None:
        path = os.path.join(ROOT, "oracle", "_ref", "libref_reorder.so")
        if not os.path.exists(path):
            _ref = False
        else:
            L = ctypes.CDLL(path)
            vp, i = ctypes.c_void_p, ctypes.c_int
            for n in ("ref_reorder_quantize_x", "ref_reorder_quantize_w"):
                f = getattr(L, n)
                f.argtypes = [vp, i, i, i, vp, i, i, i] + [vp] * 6
                f.restype = i
            L.ref_supports_k.argtypes = [i]
            L.ref_supports_k.restype = i
            _ref = L
    return _ref or None


def ref_reorder(Xd, idxd, KN, KS, KO, weights=False):
    """Run the compiled reference kernel on device tensors; returns 6 numpy arrays with scale
    buffers sized in whole atoms (pre-zeroed: the reference leaves the padding unwritten)."""
    L = ref_lib()
    R, K = Xd.shape
    u8 = dict(dtype=torch.uint8, device=Xd.device)
    if weights:
        o = [torch.zeros((R, KN // 2), **u8), torch.zeros((R, KS // 2), **u8), torch.zeros((R, KO // 2), **u8)]
    else:
        o = [torch.zeros((R, KN // 2), **u8), torch.zeros((R, KS // 4 * 3), **u8), torch.zeros((R, KO), **u8)]
    s = [torch.zeros(max(orc.sf_bytes(R, k), 16), **u8) for k in (KN, KS, KO)]
    fn = L.ref_reorder_quantize_w if weights else L.ref_reorder_quantize_x
    torch.cuda.synchronize()
    # (seq_len, out_features): the row count goes where the kernel takes its grid from
    rc = fn(Xd.data_ptr(), R, R, K, idxd.data_ptr(), KN, KS, KO, *[t.data_ptr() for t in o + s])
    assert rc == 0, "reference kernel returned %d" % rc
    return [t.cpu().numpy() for t in o] + [t.cpu().numpy()[:orc.sf_bytes(R, k)] for t, k in zip(s, (KN, KS, KO))]
