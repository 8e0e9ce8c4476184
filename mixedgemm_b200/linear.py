"""The callers either side of the hot path: a quantised-weight container and a Linear-style
module that runs  x -> reorder_quantize_x -> matmul  against it.

The reference re-quantises its weights on every run (main.py:36) and has no module of this
kind; in deployment the weight side is done once.  `QuantizedWeights` holds what
`reorder_quantize_w` produces (codes, scales) together with the reorder index and the K split,
and can be saved / loaded; `MixedLinear` owns one or several of them that share an input
(q/k/v, gate/up) and launches them as one grouped GEMM.
"""
from typing import List

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

    @classmethod
    def cat(cls, weights):
        """One weight whose rows are the rows of `weights` in order (q, k, v -> one [Nq+Nk+Nv, K]
        weight), so that a single product serves them all; every out_features must be a multiple of
        128 (whole scale blocks).  The inputs are re-pointed at row ranges of the new buffers, so
        nothing is held twice."""
        w0 = weights[0]
        for w in weights:
            if w.split != w0.split or not torch.equal(w.reorder_index, w0.reorder_index) or w.out_features % 128:
                raise ValueError("weights to concatenate must share index and split and have out_features % 128 == 0")
        N = sum(w.out_features for w in weights)
        KN, KS, KO = w0.split
        bufs = api.alloc_quantized_w(N, KN, KS, KO, w0.parts[0].device)
        n0 = 0
        for w in weights:
            n = w.out_features
            views = []
            for i in range(3):
                bufs[i][n0:n0 + n].copy_(w.parts[i])
                views.append(bufs[i][n0:n0 + n])
            for i, k in enumerate(w0.split):
                per_block = ((k + 127) // 128) * 512
                dst = bufs[3 + i][(n0 // 128) * per_block:((n0 + n) // 128) * per_block]
                dst.copy_(w.parts[3 + i][:dst.numel()])
                views.append(dst)
            w.parts = tuple(views)
            n0 += n
        return cls(bufs, w0.reorder_index, w0.split, N)

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


# ----------------------------------------------------------------------------- custom op
# quantise -> grouped GEMM as ONE torch operator, so that the module below is an ordinary op to
# torch's dispatcher (autograd-free inference graphs, stream capture, fake-tensor tracing): every
# launch goes to the current stream and nothing synchronises or allocates outside torch's caching
# allocator, which is what CUDA-graph capture asks of an op.
@torch.library.custom_op("mixedgemm_b200::mixed_linear", mutates_args=("act_scratch",))
def mixed_linear(x: torch.Tensor, reorder_index: torch.Tensor, split: List[int], weight_parts: List[torch.Tensor],
                 fused_parts: List[torch.Tensor], act_scratch: List[torch.Tensor]) -> List[torch.Tensor]:
    """x [M, K] bf16 -> [x @ W_j^T for every weight] (or, on the decode path, the one-element list
    [x @ concat(W)^T]); weight_parts holds six tensors per weight
    (codes and scales as QuantizedWeights keeps them); fused_parts, when not empty, the six tensors
    of the row-concatenation of all weights; act_scratch the six buffers of alloc_quantized_x(M, ...)
    that receive the quantised activation.
    Up to 128 tokens (decode) the concatenated weight is multiplied in ONE launch and the result is
    handed out as column ranges: a launch per projection costs about 5 us of launch gap, prologue and
    first-load latency each, more than the product itself.  Beyond that the CTA-pair kernel takes
    the projections as one grouped launch."""
    KN, KS, KO = split
    M = x.size(0)
    A = api.reorder_quantize_x(x, reorder_index, KN, KS, KO, M, 0, out=tuple(act_scratch))
    Bs = [tuple(weight_parts[6 * j:6 * j + 6]) for j in range(len(weight_parts) // 6)]
    if M <= 128 and len(fused_parts) == 6 and len(Bs) > 1:
        F = fused_parts
        # one [M, sum N_j] result; the caller hands out its column ranges (an operator's outputs
        # must not alias one another)
        return [api.matmul(A[0], F[0], A[1], F[1], A[2], F[2], A[3], F[3], A[4], F[4], A[5], F[5])]
    return api.matmul_group(A, Bs)


@mixed_linear.register_fake
def _(x, reorder_index, split, weight_parts, fused_parts, act_scratch):
    n = len(weight_parts) // 6
    if x.size(0) <= 128 and len(fused_parts) == 6 and n > 1:
        return [x.new_empty((x.size(0), fused_parts[0].size(0)))]
    return [x.new_empty((x.size(0), weight_parts[6 * j].size(0))) for j in range(n)]


class MixedLinear(torch.nn.Module):
    """y_j = x @ W_j^T for one or several projections that share x, through the quantised path.

    forward(x) quantises x once (reorder index and split of the weights) and multiplies it with
    every weight in one grouped launch where the kernel takes the shapes; returns one tensor, or
    a list when the module holds several weights."""

    def __init__(self, weights, bias=None, max_tokens=None):
        """weights: one QuantizedWeights or several that share an input; bias: None, or one bf16
        [N_j] tensor (or None) per weight, added to the bf16 product; max_tokens: when given, the
        buffers for the quantised activation are allocated now for that many rows (forward then
        allocates only its outputs, which is what a captured graph needs from one call to the next)."""
        super().__init__()
        self.weights = list(weights) if isinstance(weights, (list, tuple)) else [weights]
        w0 = self.weights[0]
        for w in self.weights[1:]:
            if w.split != w0.split or not torch.equal(w.reorder_index, w0.reorder_index):
                raise ValueError("projections that share an input must share the reorder index and the K split")
        self.split = w0.split
        self.reorder_index = w0.reorder_index
        if bias is None:
            bias = [None] * len(self.weights)
        elif torch.is_tensor(bias):
            bias = [bias]
        if len(bias) != len(self.weights):
            raise ValueError("one bias (or None) per weight")
        for b_, w in zip(bias, self.weights):
            if b_ is not None and (b_.dim() != 1 or b_.numel() != w.out_features):
                raise ValueError("a bias must be a vector of out_features elements")
        self.bias = [None if b_ is None else b_.to(torch.bfloat16) for b_ in bias]
        # several projections: their rows also live in one concatenated weight (the decode path)
        self.fused = None
        if len(self.weights) > 1 and all(w.out_features % 128 == 0 for w in self.weights):
            self.fused = QuantizedWeights.cat(self.weights)
        self._parts = [t for w in self.weights for t in w.parts]
        self._fused_parts = list(self.fused.parts) if self.fused is not None else []
        self._a = None
        if max_tokens is not None:
            self._a = api.alloc_quantized_x(int(max_tokens), *self.split, self.reorder_index.device)

    @classmethod
    def from_dense(cls, Ws, calibration_x):
        """Ws: one or several [N_j, K] bf16 weights; calibration_x: [M, K] bf16 sample whose
        per-channel absmax orders the channels (mg_reorder_index)."""
        Ws = list(Ws) if isinstance(Ws, (list, tuple)) else [Ws]
        idx = api.reorder_index(calibration_x.contiguous())
        return cls([QuantizedWeights.from_dense(W, idx) for W in Ws])

    def _scratch(self, M, device):
        """Buffers for the quantised activation of M rows: the first M rows of the pre-allocated ones
        when they are large enough (row views keep the row pitch; a scale buffer for fewer rows is a
        prefix of the larger one), else a fresh allocation that is kept for the next call."""
        if self._a is None or self._a[0].size(0) < M or self._a[0].device != device:
            self._a = api.alloc_quantized_x(M, *self.split, device)
        if self._a[0].size(0) == M:
            return list(self._a)
        lib_sf = [api.sf_bytes(M, k) for k in self.split]
        return [self._a[i][:M] for i in range(3)] + [self._a[3 + i][:max(lib_sf[i], 1)] for i in range(3)]

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M = x2.size(0)
        outs = torch.ops.mixedgemm_b200.mixed_linear(x2, self.reorder_index, list(self.split), self._parts,
                                                     self._fused_parts, self._scratch(M, x2.device))
        if len(outs) != len(self.weights):  # the decode path: one product over the concatenated weight
            Y, outs, n0 = outs[0], [], 0
            for w in self.weights:
                outs.append(Y[:, n0:n0 + w.out_features])
                n0 += w.out_features
        outs = [o if b_ is None else o + b_.to(o.device) for o, b_ in zip(outs, self.bias)]
        outs = [o.reshape(*lead, o.size(-1)) for o in outs]
        return outs[0] if len(outs) == 1 else outs
