"""The callers either side of the hot path: a quantised-weight container and a Linear-style
module that runs  x -> reorder_quantize_x -> matmul  against it.

The reference re-quantises its weights on every run (main.py:36) and has no module of this
kind; in deployment the weight side is done once.  `QuantizedWeights` holds what
`reorder_quantize_w` produces (codes, scales) together with the reorder index and the K split,
and can be saved / loaded; `MixedLinear` owns one or several of them that share an input
(q/k/v, gate/up) and launches them as one grouped GEMM.
"""
import torch

from . import api

_FORMAT_VERSION = 1


def split_k(K):
    """The reference's 62.5 / 34.375 / 3.125 % split (KN, KS, KO), all multiples of 32."""
    KO = K // 32
    KN = K * 5 // 8
    return KN, K - KN - KO, KO


class QuantizedWeights:
    """MXFP4 weights of one projection: (WN, WS, WO, SFWN, SFWS, SFWO) + index + split."""

    def __init__(self, parts, reorder_index, split, out_features):
        self.parts = tuple(parts)
        self.reorder_index = reorder_index
        self.split = tuple(int(v) for v in split)
        self.out_features = int(out_features)

    @property
    def in_features(self):
        return sum(self.split)

    @classmethod
    def from_dense(cls, W, reorder_index, split=None):
        """Quantise a [N, K] bfloat16 weight on its device (mg_reorder_quantize_w)."""
        N, K = W.shape
        split = tuple(split) if split is not None else split_k(K)
        parts = api.reorder_quantize_w(W.contiguous(), reorder_index, *split, 0, N)
        return cls(parts, reorder_index, split, N)

    def state(self):
        """Plain tensors and ints: code buffers are stored dense (the reference's layout), so a
        saved file does not depend on the row pitch this build happens to use."""
        return {"version": _FORMAT_VERSION, "split": list(self.split), "out_features": self.out_features,
                "reorder_index": self.reorder_index.cpu(),
                "codes": [p.contiguous().cpu() for p in self.parts[:3]],
                "scales": [p.cpu() for p in self.parts[3:]]}

    def save(self, path):
        torch.save(self.state(), path)

    @classmethod
    def from_state(cls, st, device):
        if st.get("version") != _FORMAT_VERSION:
            raise RuntimeError("QuantizedWeights: unknown container version %r" % (st.get("version"),))
        KN, KS, KO = st["split"]
        N = st["out_features"]
        bufs = api.alloc_quantized_w(N, KN, KS, KO, device)
        for dst, src in zip(bufs[:3], st["codes"]):
            if tuple(dst.shape) != tuple(src.shape):
                raise RuntimeError("QuantizedWeights: code buffer of shape %s where %s is expected" % (
                    tuple(src.shape), tuple(dst.shape)))
            dst.copy_(src)  # into the row-pitched view the GEMM reads in place
        for dst, src in zip(bufs[3:], st["scales"]):
            dst[:src.numel()].copy_(src[:dst.numel()])
        return cls(bufs, st["reorder_index"].to(device), (KN, KS, KO), N)

    @classmethod
    def load(cls, path, device="cuda"):
        return cls.from_state(torch.load(path, map_location="cpu"), device)


class MixedLinear(torch.nn.Module):
    """y_j = x @ W_j^T for one or several projections that share x, through the quantised path.

    forward(x) quantises x once (reorder index and split of the weights) and multiplies it with
    every weight in one grouped launch where the kernel takes the shapes; returns one tensor, or
    a list when the module holds several weights."""

    def __init__(self, weights):
        super().__init__()
        self.weights = list(weights) if isinstance(weights, (list, tuple)) else [weights]
        w0 = self.weights[0]
        for w in self.weights[1:]:
            if w.split != w0.split or not torch.equal(w.reorder_index, w0.reorder_index):
                raise ValueError("projections that share an input must share the reorder index and the K split")
        self.split = w0.split
        self.reorder_index = w0.reorder_index
        self._a = None

    @classmethod
    def from_dense(cls, Ws, calibration_x):
        """Ws: one or several [N_j, K] bf16 weights; calibration_x: [M, K] bf16 sample whose
        per-channel absmax orders the channels (mg_reorder_index)."""
        Ws = list(Ws) if isinstance(Ws, (list, tuple)) else [Ws]
        idx = api.reorder_index(calibration_x.contiguous())
        return cls([QuantizedWeights.from_dense(W, idx) for W in Ws])

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M = x2.size(0)
        if self._a is None or self._a[0].size(0) != M or self._a[0].device != x2.device:
            self._a = api.alloc_quantized_x(M, *self.split, x2.device)  # reused across calls of one shape
        A = api.reorder_quantize_x(x2, self.reorder_index, *self.split, M, 0, out=self._a)
        outs = api.matmul_group(A, [w.parts for w in self.weights])
        outs = [o.reshape(*lead, o.size(-1)) for o in outs]
        return outs[0] if len(outs) == 1 else outs
