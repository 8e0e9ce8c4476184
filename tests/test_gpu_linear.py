"""The callers either side of the path: weight container round trip and the Linear-style module."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_container_round_trip_and_module(tmp_path):
    import mixedgemm_b200 as mg
    from mixedgemm_b200.linear import MixedLinear, QuantizedWeights
    M, K = 300, 14336  # 64-tail segments: buffers are row-pitched on the device, dense in the file
    X = H.make_x(M, K, seed=1).cuda()
    Ws = [H.make_w(N, K, seed=2 + j).cuda() for j, N in enumerate((512, 256))]
    lin = MixedLinear.from_dense(Ws, X)
    # index = stable argsort of the per-channel absmax
    want_idx, _ = orc.np_reorder_index(H.bits(X.cpu()))
    assert np.array_equal(lin.reorder_index.cpu().numpy(), want_idx)
    y = lin(X)
    assert [tuple(t.shape) for t in y] == [(M, 512), (M, 256)]
    # save / load: same bytes, same product
    p = tmp_path / "w0.pt"
    lin.weights[0].save(str(p))
    w0 = QuantizedWeights.load(str(p), "cuda")
    for a, b in zip(w0.parts[:3], lin.weights[0].parts[:3]):
        assert torch.equal(a, b)
    y0 = MixedLinear(w0)(X)
    torch.cuda.synchronize()
    assert torch.equal(y0.view(torch.int16), y[0].view(torch.int16))
    # and the product tracks the unquantised one
    ref = X.float() @ Ws[0].float().T
    rel = (y[0].float() - ref).norm() / ref.norm()
    assert rel < 0.2, rel
    # batched input keeps its leading dimensions
    yb = MixedLinear(w0)(X[:256].reshape(2, 128, K))
    assert tuple(yb.shape) == (2, 128, 512)
    assert mg.device_status() == 0
